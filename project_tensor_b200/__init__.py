"""B200-native TurboQuant: the quantizers of Project-Tensor's ``tensor_gpu_v2/_quant.py`` with every
array operation in hand-written sm_100a CUDA kernels.

    import project_tensor_b200 as tg
    quant = tg.TurboQuantProd(128, 4, seed=2026)
    enc = quant.quantize(keys)                  # NumPy, CuPy, torch CUDA tensor or Tensor-like
    scores = quant.attention_score(query, enc)

The six public names of the reference module are exported unchanged.
"""
from .turboquant import (Tensor, TurboQuantMSE, TurboQuantMSEEncoding, TurboQuantProd,
                         TurboQuantProdEncoding, packed_buffers, packed_to_host, quantize_to_host, turboquant_mse,
                         turboquant_prod)
from .codebook import _build_lloyd_max_codebook  # used by the reference's own tests
from .packed_format import PackedFormatError, load_encoding, read_packed, save_encoding, write_packed
from .cache import PackedKeyCache, PackedKVCache
from .quality import quality_report

__all__ = ["Tensor", "TurboQuantMSE", "TurboQuantMSEEncoding", "TurboQuantProd",
           "TurboQuantProdEncoding", "packed_buffers", "packed_to_host", "quantize_to_host", "turboquant_mse",
           "turboquant_prod", "quality_report", "PackedFormatError", "PackedKeyCache", "PackedKVCache", "load_encoding", "read_packed", "save_encoding", "write_packed"]


def set_device(device: str) -> None:
    """Accepted for source compatibility with ``tensor_gpu_v2.set_device``; the reference's
    TurboQuant code never consulted it (it dispatches on the array type), and here everything
    runs on the GPU."""
    return None
