"""tq_mse_quantize_noalloc: the quantize entry point for hosts that cannot allocate at call time (a
serving process with a frozen memory pool, a foreign runtime that passes through pre-registered
buffers only).  It must give exactly what tq_mse_quantize gives, call after call, while keeping its
work lists in the library's own static device array.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call_pair(lib, handle, x, n, code_bytes, stream, torch):
    dev = x.device
    codes_a = torch.zeros((n, code_bytes), dtype=torch.uint8, device=dev)
    norms_a = torch.zeros((n,), dtype=torch.float32, device=dev)
    need = int(lib.tq_quantize_scratch_bytes(handle, n))
    scratch = torch.empty((max(need, 16),), dtype=torch.uint8, device=dev)
    rc = lib.tq_mse_quantize(handle, x.data_ptr(), n, codes_a.data_ptr(), norms_a.data_ptr(),
                             scratch.data_ptr(), scratch.numel(), stream)
    assert rc == 0, lib.tq_last_error()
    codes_b = torch.full((n, code_bytes), 0xAB, dtype=torch.uint8, device=dev)
    norms_b = torch.full((n,), -1.0, dtype=torch.float32, device=dev)
    rc = lib.tq_mse_quantize_noalloc(handle, x.data_ptr(), n, codes_b.data_ptr(), norms_b.data_ptr(), stream)
    assert rc == 0, lib.tq_last_error()
    torch.cuda.synchronize()
    return codes_a, norms_a, codes_b, norms_b


def test_noalloc_quantize_matches_regular_entry_point_twice(lib_built):
    import torch
    assert torch.cuda.is_available()
    import project_tensor_b200 as tg
    from project_tensor_b200 import _native
    lib = _native.load()
    dev = torch.device("cuda", 0)
    quant = tg.TurboQuantMSE(128, 4, seed=2026)
    handle = quant._plans.handle(dev)
    code_bytes = int(lib.tq_code_row_bytes(handle))
    stream = torch.cuda.current_stream(dev).cuda_stream
    gen = torch.Generator(device=dev).manual_seed(77)
    # two calls in a row with different sizes and data: the second must not see leftovers of the first
    for n in (50000, 1537):
        x = torch.randn((n, 128), generator=gen, device=dev, dtype=torch.float32)
        codes_a, norms_a, codes_b, norms_b = _call_pair(lib, handle, x, n, code_bytes, stream, torch)
        assert torch.equal(codes_a, codes_b)
        assert torch.equal(norms_a, norms_b)
    # the exact kernels (any dimension) go through the same entry point
    small = tg.TurboQuantMSE(24, 5, seed=3, grid_size=2049, max_iter=32)
    h2 = small._plans.handle(dev)
    x = torch.randn((333, 24), generator=gen, device=dev, dtype=torch.float32)
    codes_a, norms_a, codes_b, norms_b = _call_pair(lib, h2, x, 333, int(lib.tq_code_row_bytes(h2)), stream, torch)
    assert torch.equal(codes_a, codes_b) and torch.equal(norms_a, norms_b)


def test_noalloc_quantize_rejects_batches_beyond_its_limit(lib_built):
    import torch
    import project_tensor_b200 as tg
    from project_tensor_b200 import _native
    lib = _native.load()
    dev = torch.device("cuda", 0)
    quant = tg.TurboQuantMSE(128, 4, seed=2026)
    handle = quant._plans.handle(dev)
    n = 262144 + 1
    x = torch.zeros((16, 128), device=dev)   # never read: the size check comes first
    out = torch.zeros((16, 64), dtype=torch.uint8, device=dev)
    norms = torch.zeros((16,), device=dev)
    rc = lib.tq_mse_quantize_noalloc(handle, x.data_ptr(), n, out.data_ptr(), norms.data_ptr(), None)
    assert rc == -2
    assert b"at most 262144 rows" in lib.tq_last_error()


def test_noalloc_quantize_at_its_largest_batch_leaves_device_memory_as_it_was(lib_built):
    """262,144 rows is the largest batch the entry point takes, and the one for which its static work lists are
    tightest.  The call must agree with the regular entry point there too, and the device's free memory must read the
    same before and after it: nothing was allocated or freed on its behalf (inputs and outputs exist beforehand)."""
    import torch
    import project_tensor_b200 as tg
    from project_tensor_b200 import _native
    lib = _native.load()
    dev = torch.device("cuda", 0)
    quant = tg.TurboQuantMSE(128, 4, seed=2026)
    handle = quant._plans.handle(dev)
    code_bytes = int(lib.tq_code_row_bytes(handle))
    stream = torch.cuda.current_stream(dev).cuda_stream
    n = 262144
    x = torch.randn((n, 128), generator=torch.Generator(device=dev).manual_seed(78), device=dev, dtype=torch.float32)
    codes_a, norms_a, codes_b, norms_b = _call_pair(lib, handle, x, n, code_bytes, stream, torch)   # includes the first-call set-up
    assert torch.equal(codes_a, codes_b) and torch.equal(norms_a, norms_b)
    codes_b.fill_(0xAB)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    for _ in range(2):
        rc = lib.tq_mse_quantize_noalloc(handle, x.data_ptr(), n, codes_b.data_ptr(), norms_b.data_ptr(), stream)
        assert rc == 0, lib.tq_last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before
    assert torch.equal(codes_a, codes_b) and torch.equal(norms_a, norms_b)
