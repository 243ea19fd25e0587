#!/usr/bin/env python3
"""Benchmark of the TurboQuant hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (one "step" = one pass of the hot path over one batch, per GPU):
TurboQuantProd(dimension=128, bits=4, seed=2026) -- quantize 1,048,576 float32 N(0,1) keys, then
score 32 float32 N(0,1) queries against all of them (32 x 1,048,576 float32 score matrix) with the
per-query top-100 fused into the same pass.  With N > 1 GPUs every rank owns its own shard of that
size (weak scaling, no collective on the data path) and the per-shard top-100 candidates are
all-gathered over NCCL and merged, which is the only exchange the path has.

The JSON line carries: `value` = quantize throughput with inputs resident in HBM (whole job, all
ranks), `attention_score` = the scoring throughput of the same step, `roofline` for each against
the measured HBM copy bandwidth, `e2e` = the same quantize metric through the public Python API
with pinned host buffers (H2D of the keys and D2H of the packed encoding inside the timed
region), and `cpu_baseline` = the NumPy oracle on this host's cores on a bounded sample.

`--impl reference` times the CPU restatement of the reference's NumPy path (oracle/) on all host
threads, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, BITS, SEED = 128, 4, 2026
N_KEYS, N_QUERIES, TOPK = 1 << 20, 32, 100
B_MSE = max(BITS - 1, 1)
QUANT_BYTES_PER_VEC = 4 * D + D * B_MSE // 8 + D // 8 + 8            # read fp32 row, write codes+signs+2 norms
SCORE_BYTES_PER_KEY = D * B_MSE // 8 + D // 8 + 8 + 4 * N_QUERIES    # read packed key, write 32 scores
METRIC = "quantize Mvec/s & attention_score Gkeys/s; % HBM roofline"


def workload_config(world):
    return {"workload": f"TurboQuantProd d={D} bits={BITS} seed={SEED}: quantize {N_KEYS} keys + attention_score "
                        f"{N_QUERIES} queries ({N_QUERIES}x{N_KEYS} float32 score matrix) + per-query top-{TOPK}, per GPU",
            "keys_per_gpu": N_KEYS, "queries": N_QUERIES, "parallelism": f"shard{world}",
            "l2": "inputs (512 MiB of keys per GPU) are larger than L2; no flush needed"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle-reason samples taken by a background thread through NVML while the timed
    region runs (the region lasts tens of milliseconds, too short for nvidia-smi's own polling)."""

    REASONS = (("hw_slowdown", 0x8), ("sw_power_cap", 0x4), ("sw_thermal_slowdown", 0x20),
               ("hw_thermal_slowdown", 0x40))

    def __init__(self, gpu_index, period_s=0.004):
        self.gpu_index, self.period_s = gpu_index, period_s
        self.samples, self.reason_bits, self.max_mhz = [], 0, None
        self._stop = False
        self._thread = None
        self._err = None
        self._nvml = None
        self._handle = None

    def _open(self):
        """NVML is opened on the caller's thread, before the timed region: opening it takes longer than
        the region lasts."""
        try:
            import pynvml
            pynvml.nvmlInit()
            phys = self.gpu_index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                ids = [v for v in vis.split(",") if v.strip()]
                if self.gpu_index < len(ids) and ids[self.gpu_index].strip().isdigit():
                    phys = int(ids[self.gpu_index])
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception as exc:  # no NVML: report that instead of inventing numbers
            self._err = repr(exc)

    def sample_now(self):
        """One sample on the caller's thread (called between launches while the GPU is busy)."""
        if self._nvml is None:
            return
        try:
            self.samples.append(float(self._nvml.nvmlDeviceGetClockInfo(self._handle, self._nvml.NVML_CLOCK_SM)))
            self.reason_bits |= int(self._nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
        except Exception as exc:
            self._err = repr(exc)

    def _run(self):
        while not self._stop:
            self.sample_now()
            time.sleep(self.period_s)

    def start(self):
        import threading
        self._open()
        if self._nvml is None:
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop = True
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0,
                    "reasons": ["no NVML samples" + (": " + self._err if self._err else "")]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "samples": len(self.samples),
                "reasons": sorted(name for name, bit in self.REASONS if self.reason_bits & bit)}


def oracle_params():
    from oracle import turboquant_oracle as orc
    return orc, orc.prod_params(D, BITS, seed=SEED)


def time_oracle(n_quant, n_score_keys, n_score_queries, repeats):
    """Best-of-`repeats` CPU times of the oracle on a bounded sample: (quantize s, score s per query)."""
    orc, pp = oracle_params()
    rng = np.random.default_rng(20262)
    keys = rng.standard_normal((n_quant, D)).astype(np.float32)
    queries = rng.standard_normal((n_score_queries, D)).astype(np.float32)
    tq = []
    enc = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        enc = orc.prod_quantize(pp, keys)
        tq.append(time.perf_counter() - t0)
    sub = tuple(a[:n_score_keys] if hasattr(a, "shape") and a.shape[:1] == (n_quant,) else a for a in enc[:4]) + ((n_score_keys,),)
    ts = []
    for q in queries:
        t0 = time.perf_counter()
        orc.prod_attention_score(pp, q, *sub)
        ts.append(time.perf_counter() - t0)
    return min(tq), min(ts)


def host_threads():
    try:
        from threadpoolctl import threadpool_info
        n = [i.get("num_threads") for i in threadpool_info() if i.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return len(os.sched_getaffinity(0))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = 65536  # about half a second of CPU work per step
    tq_steps, ts_steps = [], []
    for _ in range(args.warmup):
        time_oracle(n_sample, n_sample, 1, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        a, b = time_oracle(n_sample, n_sample, 1, 1)
        tq_steps.append(a)
        ts_steps.append(b)
    wall = time.perf_counter() - t0
    mvec = n_sample / statistics.mean(tq_steps) / 1e6
    # the reference scores one query per call: 32 queries cost 32 passes over the keys
    gkeys = n_sample / (statistics.mean(ts_steps) * N_QUERIES) / 1e9
    cores = host_threads()
    sample = (f"oracle port of the reference NumPy path, {n_sample} of {N_KEYS} keys per step; scoring timed for 1 of "
              f"{N_QUERIES} queries and multiplied by {N_QUERIES}")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": mvec, "unit": "Mvec/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * wall / max(args.steps, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "attention_score": {"value": gkeys, "unit": "Gkeys/s", "queries": N_QUERIES},
        "cpu_baseline": {"value": mvec, "unit": "Mvec/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": mvec, "unit": "Mvec/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import project_tensor_b200 as tg
    from project_tensor_b200 import quantize_to_host
    from project_tensor_b200.sharded import merge_topk_across_ranks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    quant = tg.TurboQuantProd(D, BITS, seed=SEED)
    gen = torch.Generator(device=dev).manual_seed(20262 * 1000 + rank)
    keys = torch.randn((N_KEYS, D), generator=gen, device=dev, dtype=torch.float32)
    queries = torch.randn((N_QUERIES, D), generator=torch.Generator(device=dev).manual_seed(20272),
                          device=dev, dtype=torch.float32)
    idx_base = rank * N_KEYS

    ev = lambda: torch.cuda.Event(enable_timing=True)
    q_ms, s_ms = [], []

    def step(record):
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        enc = quant.quantize(keys)
        e1.record()
        scores = quant.attention_scores(queries, enc)                      # the 32 x N score matrix
        e2.record()
        top_s, top_i = quant.attention_scores(queries, enc, topk=TOPK, index_base=idx_base)
        if world > 1:
            top_s, top_i = merge_topk_across_ranks(top_s, top_i)           # the only exchange: NCCL all-gather
        if record is not None:
            record.append((e0, e1, e2))
        return top_s, top_i, scores

    for _ in range(args.warmup):
        step(None)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    torch.cuda.synchronize()
    recs = []
    t_start, t_end = ev(), ev()
    t_start.record()
    for it in range(args.steps):
        out = step(recs)
    t_end.record()
    if rank == 0:
        sampler.sample_now()       # the GPU is still working through the launches queued above
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    total_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop() if rank == 0 else None
    for e0, e1, e2 in recs:
        q_ms.append(e0.elapsed_time(e1))
        s_ms.append(e1.elapsed_time(e2))
    mine = torch.tensor([total_ms, statistics.mean(q_ms), statistics.mean(s_ms)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(mine, op=dist.ReduceOp.MAX)
    total_ms, q_mean, s_mean = (float(v) for v in mine.tolist())

    if args.skip_host_legs:
        # profiler captures also want the MSE quantizer and the dequantizers of the same sizes
        mse = tg.TurboQuantMSE(D, BITS, seed=SEED)
        enc_m = mse.quantize(keys)
        mse.dequantize(enc_m)
        quant.dequantize(quant.quantize(keys))
        kv, kv_q = decode_cache(tg, torch, quant, mse, keys, dev)
        kv.attend(kv_q)
        kv.keys.scores(kv_q)
        torch.cuda.synchronize()
        if rank == 0:
            print(json.dumps({"note": "profiling run without host legs", "keys": N_KEYS, "quantize_ms": q_mean,
                              "score_ms": s_mean, "ms_per_step": total_ms / args.steps}))
        if world > 1:
            dist.destroy_process_group()
        return
    # ---- the other calls of the path, each timed alone with CUDA events (median of 10), rank 0 only --------
    other = {}
    if rank == 0:
        def timed(fn, reps=10, inner=4):     # `inner` calls back to back between the events: the rate of the call, not the
                                             # latency of one launch into an idle GPU
            for _ in range(3):
                fn()
            ms = []
            for _ in range(reps):
                a_, b_ = ev(), ev()
                a_.record()
                for _ in range(inner):
                    fn()
                b_.record()
                torch.cuda.synchronize()
                ms.append(a_.elapsed_time(b_) / inner)
            return statistics.median(ms)

        mse = tg.TurboQuantMSE(D, BITS, seed=SEED)
        enc_m = mse.quantize(keys)
        enc_p = quant.quantize(keys)
        mse_bytes = 4 * D + D * BITS // 8 + 4
        rows = (
            ("mse_quantize", lambda: mse.quantize(keys), mse_bytes, "B/vector: fp32 row in, packed codes + norm out"),
            ("mse_dequantize", lambda: mse.dequantize(enc_m), mse_bytes, "B/vector: packed codes + norm in, fp32 row out"),
            ("prod_dequantize", lambda: quant.dequantize(enc_p), QUANT_BYTES_PER_VEC, "B/vector: packed encoding in, fp32 row out"),
            ("attention_score_one_query", lambda: quant.attention_score(queries[0], enc_p),
             D * B_MSE // 8 + D // 8 + 8 + 4, "B/key: packed key in, one score out (the reference's own call)"),
            ("attention_score_top%d_no_matrix" % TOPK,
             lambda: quant.attention_scores(queries, enc_p, topk=TOPK, index_base=idx_base),
             D * B_MSE // 8 + D // 8 + 8, "B/key: packed key in; scores stay in scratch"),
        )
        peak_o, _ = measured_peaks()
        for name, fn, nbytes, what in rows:
            ms = timed(fn)
            gbs = nbytes * N_KEYS / (ms * 1e-3) / 1e9
            other[name] = {"ms": ms, "M_per_s": N_KEYS / (ms * 1e-3) / 1e6, "bytes_per_unit": nbytes, "bytes": what,
                           "achieved_GBps": gbs, "frac_of_measured_hbm": gbs / peak_o}
        del enc_m, enc_p
        # decode attention over a packed key/value cache of the same keys: DECODE_GROUPS sequences x heads,
        # DECODE_QPG queries each (grouped-query attention), values TurboQuantMSE(d, bits)
        kv, kv_q = decode_cache(tg, torch, quant, mse, keys, dev)
        ms = timed(lambda: kv.attend(kv_q))
        nbytes = D * B_MSE // 8 + D // 8 + 8 + D * BITS // 8 + 4
        gbs = nbytes * N_KEYS / (ms * 1e-3) / 1e9
        other["decode_attention"] = {
            "ms": ms, "M_per_s": N_KEYS / (ms * 1e-3) / 1e6, "bytes_per_unit": nbytes,
            "bytes": "B/key: packed key and packed value in; scores and dequantized values never leave the SM",
            "achieved_GBps": gbs, "frac_of_measured_hbm": gbs / peak_o,
            "groups": DECODE_GROUPS, "queries_per_group": DECODE_QPG, "keys_per_group": N_KEYS // DECODE_GROUPS}
        # the decode step's scores alone: every group of keys scored by its DECODE_QPG query heads, matrix out
        enc_g = kv.keys.encoding(0)     # plans and buffers of the cache; scored through the cache's own call
        ms = timed(lambda: kv.keys.scores(kv_q))
        nbytes = D * B_MSE // 8 + D // 8 + 8 + 4 * DECODE_QPG
        gbs = nbytes * N_KEYS / (ms * 1e-3) / 1e9
        other["attention_score_%d_queries_per_group" % DECODE_QPG] = {
            "ms": ms, "M_per_s": N_KEYS / (ms * 1e-3) / 1e6, "bytes_per_unit": nbytes,
            "bytes": "B/key: packed key in, %d scores out (grouped-query decode: %d groups)" % (DECODE_QPG, DECODE_GROUPS),
            "achieved_GBps": gbs, "frac_of_measured_hbm": gbs / peak_o}
        del kv, kv_q, enc_g
    # ---- end to end through the public API with host buffers (pinned), rank-local -------------------
    host_keys = torch.empty((N_KEYS, D), dtype=torch.float32).pin_memory()
    host_keys.copy_(keys)
    host_np = host_keys.numpy()
    e2e_ms = []
    d2h = 0
    host_out = None
    for it in range(2 + 3):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        host_out = quantize_to_host(quant, host_np, out=host_out)   # chunked: H2D, kernels and D2H overlap
        torch.cuda.synchronize()
        if it >= 2:
            e2e_ms.append(1e3 * (time.perf_counter() - t0))
        d2h = sum(t.numel() * t.element_size() for t in host_out.values() if t is not None)
    e2e = torch.tensor([statistics.mean(e2e_ms)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    e2e_mean = float(e2e.item())

    if rank == 0:
        peak, peak_kind = measured_peaks()
        quant_gbs = QUANT_BYTES_PER_VEC * N_KEYS / (q_mean * 1e-3) / 1e9
        score_gbs = SCORE_BYTES_PER_KEY * N_KEYS / (s_mean * 1e-3) / 1e9
        line = {
            "metric": METRIC,
            "value": world * N_KEYS / (q_mean * 1e-3) / 1e6,
            "unit": "Mvec/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (rotation as 3 fp16 tensor-core passes, fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world),
            "attention_score": {
                "value": world * N_KEYS / (s_mean * 1e-3) / 1e9, "unit": "Gkeys/s", "queries": N_QUERIES,
                "ms": s_mean,
                "roofline": {"bound": "hbm", "achieved": score_gbs, "peak": peak, "unit": "GB/s",
                             "frac": score_gbs / peak, "frac_of_8TBs": score_gbs / 8000.0,
                             "traffic": traffic_bytes(18.95e6, 33.5e6),
                             "bytes_per_key": SCORE_BYTES_PER_KEY, "peak_kind": peak_kind}},
            "quantize_ms": q_mean,
            "roofline": {"bound": "hbm", "achieved": quant_gbs, "peak": peak, "unit": "GB/s",
                         "frac": quant_gbs / peak, "frac_of_8TBs": quant_gbs / 8000.0,
                         "traffic": traffic_bytes(135.7e6, 19.3e6),
                         "bytes_per_vector": QUANT_BYTES_PER_VEC, "peak_kind": peak_kind,
                         "kernel": "tq_prod_quantize call (tensor-core kernel + exact second stage)"},
            "e2e": {"value": world * N_KEYS / (e2e_mean * 1e-3) / 1e6, "unit": "Mvec/s",
                    "h2d_bytes_per_step": N_KEYS * D * 4, "d2h_bytes_per_step": d2h,
                    "what": "quantize_to_host(TurboQuantProd, pinned NumPy keys): chunked H2D, quantize, D2H into reused pinned buffers"},
            "gpu_launches": args.steps * 9,   # per step: 3 quantize kernels, 2 for the score matrix, 4 for the top-k call
            "clocks": clocks,
            "other_calls": other,
        }
        if world == 1:
            n_sample = 262144
            cq, cs = time_oracle(n_sample, n_sample, 2, 3)
            line["cpu_baseline"] = {
                "value": n_sample / cq / 1e6, "unit": "Mvec/s", "cores": host_threads(), "kind": "port",
                "attention_score_Gkeys_per_s": n_sample / (cs * N_QUERIES) / 1e9,
                "sample": f"NumPy oracle, quantize {n_sample} of {N_KEYS} keys (best of 3); scoring 1 query x {n_sample} "
                          f"keys (best of 2) multiplied by {N_QUERIES} queries"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


DECODE_GROUPS, DECODE_QPG = 64, 4


def decode_cache(tg, torch, quant, mse, keys, dev):
    """A PackedKVCache of DECODE_GROUPS groups filled with the bench keys (and as many random values), and
    DECODE_QPG queries per group."""
    per_group = N_KEYS // DECODE_GROUPS
    kv = tg.PackedKVCache(quant, mse, DECODE_GROUPS, per_group)
    gen = torch.Generator(device=dev).manual_seed(20290)
    values = torch.randn((DECODE_GROUPS, per_group, D), device=dev, generator=gen)
    kv.append(keys[:DECODE_GROUPS * per_group].view(DECODE_GROUPS, per_group, D), values)
    del values
    kv_q = torch.randn((DECODE_GROUPS, DECODE_QPG, D), device=dev, generator=gen)
    return kv, kv_q


def traffic_bytes(read_262144, write_262144):
    """DRAM bytes of one launch of the dominant kernel at this run's size.  ncu counted dram__bytes_read.sum and
    dram__bytes_write.sum for a launch over 262,144 keys (the capture summarised in profiles/); both grow in
    proportion to the keys, so they are scaled.  A write that was still in L2 when the capture ended is taken
    at its algorithmic size.  None for a workload other than the captured one (d = 128, bits = 4, 32 queries)."""
    if D != 128 or BITS != 4 or N_QUERIES != 32:
        return None
    return (read_262144 + write_262144) * N_KEYS / 262144.0


def run_retrieval(args):
    """Sharded retrieval at box scale (the largest configuration of the reference's benchmark list): `--total-keys`
    TurboQuantProd(128, 4) keys split evenly over the ranks, 64 queries, per-shard top-100 merged over NCCL into a
    global top-100 per query.  Keys are generated on the device per chunk of 2^20 (torch Philox, seed
    20265 * 2^32 + chunk), quantized and dropped; only the packed encoding stays (72 B/key).  Prints one JSON line
    with the quantize and search rates and the outcome of size-independent checks: descending scores, unique
    in-range indices, and agreement with an independent pass over the chunk that holds query 0's best key."""
    import torch
    import torch.distributed as dist
    import project_tensor_b200 as tg
    from project_tensor_b200.sharded import ShardedKeyIndex, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    chunk, n_total, n_q, k = 1 << 20, args.total_keys, 64, TOPK
    if n_total % (chunk * world):
        raise SystemExit("--total-keys must be a multiple of 2^20 keys per rank")
    quant = tg.TurboQuantProd(D, BITS, seed=SEED)
    index = ShardedKeyIndex(quant, n_total)
    queries = torch.from_numpy(np.random.default_rng(20275).standard_normal((n_q, D)).astype(np.float32)).to(dev)

    def make_chunk(c):
        gen = torch.Generator(device=dev).manual_seed(20265 * 2 ** 32 + c)
        return torch.randn((chunk, D), generator=gen, device=dev, dtype=torch.float32)

    ev = lambda: torch.cuda.Event(enable_timing=True)
    start, stop = shard_range(n_total, rank, world)
    for _ in range(3):      # first calls load the kernels and build the plan: not part of the rate
        quant.quantize(make_chunk(start // chunk))
    torch.cuda.synchronize()
    pairs = []
    for c in range(start // chunk, stop // chunk):
        x = make_chunk(c)
        e0, e1 = ev(), ev()
        e0.record()
        index.add(x)
        e1.record()
        pairs.append((e0, e1))
        del x
    torch.cuda.synchronize()
    add_ms = sum(a.elapsed_time(b) for a, b in pairs)
    for _ in range(max(args.warmup, 1)):
        top_s, top_i = index.search(queries, k)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    steps = min(args.steps, 5)
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(steps):
        top_s, top_i = index.search(queries, k)
    e1.record()
    torch.cuda.synchronize()
    times = torch.tensor([add_ms, e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    add_ms, search_ms = (float(v) for v in times.tolist())

    # ---- checks that do not depend on the size --------------------------------------------------
    checks = {"descending": bool((top_s[:, :-1] >= top_s[:, 1:]).all()),
              "indices_in_range": bool(((top_i >= 0) & (top_i < n_total)).all()),
              "indices_unique": all(len(set(row)) == k for row in top_i.tolist())}
    c_best = int(top_i[0, 0].item()) // chunk
    enc = quant.quantize(make_chunk(c_best))
    part = quant.attention_scores(queries, enc)                       # 64 x 2^20 scores of that chunk, computed alone
    scale = float(top_s.abs().max())
    inside = (top_i // chunk) == c_best
    got = top_s[inside]
    want = part[torch.nonzero(inside)[:, 0], (top_i[inside] - c_best * chunk)]
    checks["chunk_scores_agree"] = bool((got - want).abs().max() <= 1e-4 * scale) if got.numel() else True
    # nothing in the chunk beats the global 100th score without being in the global list
    kth = top_s[:, -1:].clone()
    beats = (part > kth + 1e-4 * scale).sum(dim=1)
    checks["chunk_has_no_missed_key"] = bool((beats <= inside.sum(dim=1)).all())
    if rank == 0:
        print(json.dumps({
            "metric": "sharded retrieval: quantize Mvec/s and top-%d search Gkeys/s" % k, "n_gpus": world,
            "config": {"workload": f"TurboQuantProd d={D} bits={BITS}: {n_total} keys over {world} GPU(s), {n_q} queries, "
                                   f"per-shard top-{k} + NCCL all-gather + merge", "keys_per_gpu": n_total // world},
            "quantize_Mvec_per_s": n_total / (add_ms * 1e-3) / 1e6, "quantize_ms_total": add_ms,
            "search_ms": search_ms, "search_Gkeys_per_s": n_total / (search_ms * 1e-3) / 1e9,
            "search_Gpairs_per_s": n_total * n_q / (search_ms * 1e-3) / 1e9,
            "packed_GB_per_gpu": (n_total // world) * 72 / 1e9, "data": "synthetic", "checks": checks}))
    if world > 1:
        dist.destroy_process_group()
    if not all(checks.values()):
        raise SystemExit("retrieval checks failed: %r" % (checks,))


def main():
    global N_KEYS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--keys", type=int, default=N_KEYS,
                    help="keys per GPU; the default is the benchmark's workload, smaller values are for profiler captures only")
    ap.add_argument("--skip-host-legs", action="store_true",
                    help="leave out the end-to-end and CPU-baseline legs (profiler captures)")
    ap.add_argument("--workload", default="headline", choices=["headline", "retrieval"],
                    help="retrieval: the sharded top-100 search over --total-keys keys (not the headline line)")
    ap.add_argument("--total-keys", type=int, default=134217728, help="keys over all GPUs for --workload retrieval")
    args = ap.parse_args()
    N_KEYS = args.keys
    if args.workload == "retrieval" and args.impl == "b200":
        return run_retrieval(args)
    if args.warmup < 3 and args.impl == "b200":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
