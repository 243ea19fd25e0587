#!/usr/bin/env python3
"""Benchmark of the TurboQuant hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload retrieval]

Workload (one "step" = one pass of the hot path over one batch, per GPU):
TurboQuantProd(dimension=128, bits=4, seed=2026) -- quantize 1,048,576 float32 N(0,1) keys, then
score 32 float32 N(0,1) queries against all of them (32 x 1,048,576 float32 score matrix), then take the
per-query top-100 without a matrix.  With N > 1 GPUs every rank owns its own shard of that size (weak
scaling, no collective on the data path); the per-shard top-100 candidates are written straight into a send
block, all-gathered over NCCL while the next step's quantize runs, and merged: the only exchange of the path.

The timed region is exactly K steps between a barrier + synchronize on both sides, device time, maximum over
ranks.  It lasts about 15 ms, so it is repeated (`repeats`, each again exactly K steps) until half a second is
covered and the median repeat is reported; the clock samples are taken over all repeats.

The JSON line carries: `value` = quantize throughput with inputs resident in HBM (whole job, all ranks),
`attention_score` = the scoring throughput of the same step, `roofline` for each against the measured HBM copy
bandwidth, `e2e` = the same metrics through the public Python API with host buffers (host-to-device and
device-to-host copies inside the timed region), `parity` = differences against the NumPy oracle on a bounded
sample of this run's keys, `configs` = the other benchmark configurations (one GPU only) and `cpu_baseline` =
the NumPy oracle on this host's cores on a bounded sample.

`--impl reference` times the CPU restatement of the reference's NumPy path (oracle/) on all host threads.
"""
from __future__ import annotations

import argparse
import json
import math
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
WINDOW, REL_RECON, REL_SCORE = 1e-5, 1e-5, 1e-4


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


def prod_bytes(d, bits):
    b = max(bits - 1, 1)
    return 4 * d + d * b // 8 + d // 8 + 8


def mse_bytes(d, bits):
    return 4 * d + d * bits // 8 + 4


def key_bytes(d, bits):
    return d * max(bits - 1, 1) // 8 + d // 8 + 8


class ClockSampler:
    """SM clock and throttle-reason samples taken by a background thread through NVML while the timed
    regions run."""

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
        """NVML is opened on the caller's thread, before the timed region."""
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


# ---------------------------------------------------------------------------------------------------------
# CPU side: the oracle as baseline and as checker
# ---------------------------------------------------------------------------------------------------------
def oracle_params(d=D, bits=BITS):
    from oracle import turboquant_oracle as orc
    return orc, orc.prod_params(d, bits, seed=SEED)


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
    """The reference's CPU path (oracle port) on every host thread NumPy uses.  One step = quantize all 1,048,576
    keys and score one of the 32 queries against them (the reference scores one query per call; the other 31 calls
    cost the same and are accounted by multiplication).  If the run would not end within a few minutes at that
    size, the step shrinks to a power-of-two sample and says so."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = N_KEYS
    t0 = time.perf_counter()
    time_oracle(65536, 65536, 1, 1)
    probe = time.perf_counter() - t0                      # seconds per 65,536 keys (quantize + one query)
    total_steps = max(args.steps, 1) + args.warmup
    while n_sample > 65536 and probe * (n_sample / 65536) * total_steps > 240.0:
        n_sample //= 2
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


def parity_report(quant, keys_dev, queries_dev, n):
    """Differences between the CUDA path and the NumPy oracle on the first `n` keys of this run: packed codes and QJL
    signs (counts, rate, how many lie outside the 1e-5 window of their decision point), norms, residual norms and
    the scores of two queries."""
    orc, _ = oracle_params()
    d = quant.dimension
    x = keys_dev[:n].cpu().numpy()
    q = queries_dev.cpu().numpy()
    inner = orc.mse_params(d, max(quant.bits - 1, 1), rotation=quant.mse.rotation, codebook=quant.mse.codebook)
    pp = orc.ProdParams(d, quant.bits, inner, quant.projection)
    want = orc.prod_quantize(pp, x)
    enc = quant.quantize(keys_dev[:n])
    host = lambda t: t.cpu().numpy() if hasattr(t, "cpu") else np.asarray(t)
    codes, qjl = host(enc.indices), host(enc.qjl)
    norms, rnorms = host(enc.norms), host(enc.residual_norms)
    crow, ccol = np.nonzero(codes != want[0])
    rows = np.unique(np.concatenate([crow, np.nonzero(np.any(qjl != want[1], axis=1))[0]]))
    code_out = sign_out = 0
    same = ~np.any(codes != want[0], axis=1)
    sdiff = (qjl != want[1]) & same[:, None]
    if len(rows):
        x64 = x[rows].astype(np.float64)
        unit = x64 / np.linalg.norm(x64, axis=1, keepdims=True)
        pos = {r: i for i, r in enumerate(rows.tolist())}
        rot = unit @ quant.mse.rotation.astype(np.float64).T
        bnd = quant.mse.boundaries.astype(np.float64)
        for r, c in zip(crow.tolist(), ccol.tolist()):
            code_out += int(np.min(np.abs(rot[pos[r], c] - bnd)) > WINDOW)
        resid = unit - quant.mse.codebook.astype(np.float64)[want[0][rows]] @ quant.mse.rotation.astype(np.float64)
        proj = resid @ quant.projection.astype(np.float64).T
        srow, scol = np.nonzero(sdiff)
        for r, c in zip(srow.tolist(), scol.tolist()):
            sign_out += int(abs(proj[pos[r], c]) > WINDOW)
    rel = lambda a, b: float(np.max(np.abs(a.astype(np.float64) - b) / np.where(b != 0, np.abs(b), 1.0)))
    got = host(quant.attention_scores(queries_dev, enc))
    score_err = 0.0
    for qi in (0, q.shape[0] - 1):
        ref = orc.prod_attention_score(pp, q[qi], *want)
        scale = np.linalg.norm(q[qi]) * want[3] / math.sqrt(d)
        score_err = max(score_err, float(np.max((np.abs(got[qi] - ref) / scale)[same])))
    total = int(codes.size)
    return {"keys": int(n), "coordinates": total,
            "code_flips": int(len(crow)), "code_flip_rate": len(crow) / total, "code_flips_outside_1e-5_window": code_out,
            "sign_flips": int(sdiff.sum()), "sign_flip_rate": float(sdiff.sum()) / total, "sign_flips_outside_1e-5_window": sign_out,
            "norms_max_rel": rel(norms, want[3]), "residual_norms_max_rel": rel(rnorms[same], want[2][same]),
            "scores_max_err_over_qk_sqrt_d": score_err, "queries_checked": 2,
            "bounds": {"flip_rate": 1e-6, "outside_window": 0, "norms": REL_RECON, "scores": REL_SCORE},
            "ok": bool(code_out == 0 and sign_out == 0 and len(crow) <= max(1, 1e-6 * total) and sdiff.sum() <= max(1, 1e-6 * total)
                       and rel(norms, want[3]) <= REL_RECON and score_err <= REL_SCORE),
            "oracle": "oracle/turboquant_oracle.py (NumPy restatement pinned bit for bit on fixtures recorded from the reference)"}


# ---------------------------------------------------------------------------------------------------------
# GPU side
# ---------------------------------------------------------------------------------------------------------
def make_timed(torch):
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=10, inner=4):
        """Median device time of one call: `inner` calls back to back between two events (the rate of the call,
        not the latency of one launch into an idle GPU)."""
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
    return timed


def rate_row(ms, units, nbytes, what, peak, **extra):
    gbs = nbytes * units / (ms * 1e-3) / 1e9
    row = {"ms": ms, "M_per_s": units / (ms * 1e-3) / 1e6, "bytes_per_unit": nbytes, "bytes": what,
           "achieved_GBps": gbs, "frac_of_measured_hbm": gbs / peak}
    row.update(extra)
    return row


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import project_tensor_b200 as tg
    from project_tensor_b200 import _native, packed_to_host, quantize_to_host
    from project_tensor_b200.sharded import TopkExchange

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _native.load()

    quant = tg.TurboQuantProd(D, BITS, seed=SEED)
    gen = torch.Generator(device=dev).manual_seed(20262 * 1000 + rank)
    keys = torch.randn((N_KEYS, D), generator=gen, device=dev, dtype=torch.float32)
    queries = torch.randn((N_QUERIES, D), generator=torch.Generator(device=dev).manual_seed(20272),
                          device=dev, dtype=torch.float32)
    idx_base = rank * N_KEYS
    ev = lambda: torch.cuda.Event(enable_timing=True)
    timed = make_timed(torch)

    def step(record):
        """quantize -> score matrix -> per-shard top-100 written into the send block -> all-gather enqueued.  The merge
        of a step is enqueued by the caller after the next step's kernels, so the collective overlaps them."""
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        enc = quant.quantize(keys)
        e1.record()
        scores = quant.attention_scores(queries, enc)                      # the 32 x N score matrix
        e2.record()
        ex = TopkExchange(N_QUERIES, TOPK, dev)
        quant.attention_scores(queries, enc, topk=TOPK, index_base=idx_base, out=(ex.top_scores, ex.top_idx))
        ex.start()                                                         # the only exchange: NCCL all-gather
        if record is not None:
            record.append((e0, e1, e2))
        return ex, scores

    def run_steps(k, record):
        prev, out = None, None
        for _ in range(k):
            ex, _scores = step(record)
            if prev is not None:
                out = prev.finish()
            prev = ex
        return prev.finish() if prev is not None else out

    run_steps(args.warmup, None)
    torch.cuda.synchronize()
    # how many repeats of the K-step region cover half a second
    a_, b_ = ev(), ev()
    a_.record()
    run_steps(2, None)
    b_.record()
    torch.cuda.synchronize()
    est_ms = a_.elapsed_time(b_) / 2
    repeats = 1 if args.skip_host_legs else max(1, min(64, int(math.ceil(500.0 / max(args.steps * est_ms, 1e-3)))))
    if world > 1:
        rt = torch.tensor([repeats], device=dev)
        dist.all_reduce(rt, op=dist.ReduceOp.MAX)
        repeats = int(rt.item())
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    recs, totals = [], []
    import ctypes
    handle = quant._plans.handle(dev)
    _native.check(lib.tq_plan_time_kernels(handle, 1))      # an event pair around every launch of the two main kernels
    launches0 = int(lib.tq_kernel_launches())
    for _ in range(repeats):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t_start, t_end = ev(), ev()
        t_start.record()
        run_steps(args.steps, recs)
        t_end.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        totals.append(t_start.elapsed_time(t_end))
    launches = (int(lib.tq_kernel_launches()) - launches0) // repeats
    buf = (ctypes.c_float * 1024)()
    nq_k = int(lib.tq_plan_kernel_ms(handle, 0, buf, 1024))
    kq_ms = statistics.median(list(buf)[:nq_k]) if nq_k > 0 else float("nan")
    ns_k = int(lib.tq_plan_kernel_ms(handle, 1, buf, 1024))
    # scoring launches alternate: score matrix, then the top-k call of the same step (the last one is a top-k call)
    ks_all = list(buf)[:ns_k]
    ks_ms = statistics.median([v for i, v in enumerate(ks_all) if (ns_k - 1 - i) % 2 == 1]) if ns_k > 1 else float("nan")
    _native.check(lib.tq_plan_time_kernels(handle, 0))
    clocks = sampler.stop() if rank == 0 else None
    q_all = [e0.elapsed_time(e1) for e0, e1, _ in recs]
    s_all = [e1.elapsed_time(e2) for _, e1, e2 in recs]
    mine = torch.tensor(totals + [kq_ms, ks_ms, statistics.median(q_all), statistics.median(s_all)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(mine, op=dist.ReduceOp.MAX)       # every repeat: the slowest rank's time
    vals = [float(v) for v in mine.tolist()]
    totals, kq_ms, ks_ms, q_med, s_med = vals[:-4], vals[-4], vals[-3], vals[-2], vals[-1]
    total_ms = statistics.median(totals)

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
            print(json.dumps({"note": "profiling run without host legs", "keys": N_KEYS, "quantize_ms": q_med,
                              "score_ms": s_med, "ms_per_step": total_ms / args.steps}))
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    # ---- the other calls of the path, each timed alone (median of 10 groups of 4 calls), rank 0 only --------
    other, configs, parity, quality = {}, None, None, None
    if rank == 0:
        mse = tg.TurboQuantMSE(D, BITS, seed=SEED)
        enc_m = mse.quantize(keys)
        enc_p = quant.quantize(keys)
        kb = key_bytes(D, BITS)
        rows = (
            ("prod_quantize_back_to_back", lambda: quant.quantize(keys), QUANT_BYTES_PER_VEC, "B/vector: fp32 row in, packed key out (the headline call, four calls in a row)"),
            ("mse_quantize", lambda: mse.quantize(keys), mse_bytes(D, BITS), "B/vector: fp32 row in, packed codes + norm out"),
            ("mse_dequantize", lambda: mse.dequantize(enc_m), mse_bytes(D, BITS), "B/vector: packed codes + norm in, fp32 row out"),
            ("prod_dequantize", lambda: quant.dequantize(enc_p), QUANT_BYTES_PER_VEC, "B/vector: packed encoding in, fp32 row out"),
            ("attention_score_one_query", lambda: quant.attention_score(queries[0], enc_p), kb + 4,
             "B/key: packed key in, one score out (the reference's own call)"),
            ("attention_score_top%d_no_matrix" % TOPK,
             lambda: quant.attention_scores(queries, enc_p, topk=TOPK, index_base=idx_base), kb,
             "B/key: packed key in; scores stay in scratch"),
        )
        for name, fn, nbytes, what in rows:
            other[name] = rate_row(timed(fn), N_KEYS, nbytes, what, peak)
        del enc_m
        # the quantizers at the other two dimensions of the reference's grid, same number of vectors
        for d_other in (64, 256):
            keys_o = torch.randn((N_KEYS, d_other), generator=gen, device=dev, dtype=torch.float32)
            for cls, nbytes in ((tg.TurboQuantMSE, mse_bytes(d_other, BITS)), (tg.TurboQuantProd, prod_bytes(d_other, BITS))):
                q_o = cls(d_other, BITS, seed=SEED)
                name = ("mse" if cls is tg.TurboQuantMSE else "prod") + "_quantize_d%d" % d_other
                other[name] = rate_row(timed(lambda: q_o.quantize(keys_o)), N_KEYS, nbytes,
                                       "B/vector: fp32 row in, packed encoding out, d = %d" % d_other, peak)
            if d_other == 256:      # q_o is the TurboQuantProd of d = 256: the same 32 x N score matrix as the headline
                enc_o = q_o.quantize(keys_o)
                q32 = torch.randn((N_QUERIES, d_other), generator=gen, device=dev, dtype=torch.float32)
                other["attention_score_matrix_d256"] = rate_row(
                    timed(lambda: q_o.attention_scores(q32, enc_o)), N_KEYS, key_bytes(d_other, BITS) + 4 * N_QUERIES,
                    "B/key: packed key in, %d scores out, d = 256" % N_QUERIES, peak)
                del enc_o, q32
            del keys_o
        q64 = torch.randn((64, D), generator=gen, device=dev, dtype=torch.float32)
        other["attention_score_matrix_64_queries"] = rate_row(
            timed(lambda: quant.attention_scores(q64, enc_p)), N_KEYS, kb + 4 * 64,
            "B/key: packed key in, 64 scores out (one pass of 64 queries)", peak)
        del q64
        kv, kv_q = decode_cache(tg, torch, quant, mse, keys, dev)
        other["decode_attention"] = rate_row(
            timed(lambda: kv.attend(kv_q)), N_KEYS, kb + D * BITS // 8 + 4,
            "B/key: packed key and packed value in; scores and dequantized values never leave the SM", peak,
            groups=DECODE_GROUPS, queries_per_group=DECODE_QPG, keys_per_group=N_KEYS // DECODE_GROUPS)
        other["attention_score_%d_queries_per_group" % DECODE_QPG] = rate_row(
            timed(lambda: kv.keys.scores(kv_q)), N_KEYS, kb + 4 * DECODE_QPG,
            "B/key: packed key in, %d scores out (grouped-query decode: %d groups)" % (DECODE_QPG, DECODE_GROUPS), peak)
        del kv, kv_q
        if world == 1:
            parity = parity_report(quant, keys, queries, 131072)
            quality = tg.quality_report(mse, quant, keys, queries, ks=(1, 10, 100))
            quality["what"] = ("the reference harness's metrics (validate_turboquant.py) on this run's 1,048,576 N(0,1) keys and 32 queries, "
                               "computed on the device chunk by chunk; recall against the exact float32 products")
    # ---- end to end through the public API with host buffers, every rank ---------------------------------
    host_keys = torch.empty((N_KEYS, D), dtype=torch.float32).pin_memory()
    host_keys.copy_(keys)
    host_np = host_keys.numpy()

    def wall_ms(fn, reps=5, warm=2):
        """Wall-clock time of one call, median of `reps` (the host is shared: a mean would carry every hiccup of it)."""
        out = []
        for it in range(warm + reps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn()
            torch.cuda.synchronize()
            if it >= warm:
                out.append(1e3 * (time.perf_counter() - t0))
        wall_ms.last = out
        return statistics.median(out)

    state = {"out": None}

    def chunked():
        state["out"] = quantize_to_host(quant, host_np, out=state["out"])   # chunked: H2D, kernels and D2H overlap
    e2e_ms = wall_ms(chunked, reps=9)
    e2e_runs = [round(v, 3) for v in wall_ms.last]
    d2h = sum(t.numel() * t.element_size() for t in state["out"].values() if t is not None)
    e2e_extra = {}
    if rank == 0:
        back = {"out": None}

        def drop_in():          # what a user of the reference writes: NumPy in, encoding out, packed fields read back
            enc = quant.quantize(host_np)
            back["out"] = packed_to_host(enc, out=back["out"])
        drop_ms = wall_ms(drop_in)
        q_np = queries.cpu().numpy()
        enc_p = quant.quantize(keys)
        topk_ms = wall_ms(lambda: quant.attention_scores(q_np, enc_p, topk=TOPK), reps=5)
        mat_ms = wall_ms(lambda: quant.attention_scores(q_np, enc_p), reps=5)
        e2e_extra = {
            "quantize_drop_in_call": {
                "value": N_KEYS / (drop_ms * 1e-3) / 1e6, "unit": "Mvec/s", "ms": drop_ms,
                "what": "TurboQuantProd.quantize(NumPy keys) -> encoding, packed fields copied to reused pinned host buffers"},
            "attention_score_top%d" % TOPK: {
                "value": N_KEYS / (topk_ms * 1e-3) / 1e9, "unit": "Gkeys/s", "ms": topk_ms,
                "h2d_bytes_per_step": N_QUERIES * D * 4, "d2h_bytes_per_step": N_QUERIES * TOPK * 12,
                "what": "attention_scores(NumPy queries, device-resident packed keys, topk=100) -> NumPy scores and indices"},
            "attention_score_matrix": {
                "value": N_KEYS / (mat_ms * 1e-3) / 1e9, "unit": "Gkeys/s", "ms": mat_ms,
                "h2d_bytes_per_step": N_QUERIES * D * 4, "d2h_bytes_per_step": N_QUERIES * N_KEYS * 4,
                "what": "attention_scores(NumPy queries, device-resident packed keys) -> NumPy 32 x N matrix (page-locked block of the caching host allocator behind the array)"}}
        del enc_p
    e2e = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e.item())
    del host_keys, host_np

    if rank == 0 and world == 1:
        del keys
        torch.cuda.empty_cache()
        configs = run_configs(tg, torch, timed, peak, dev)

    if rank == 0:
        quant_call_gbs = QUANT_BYTES_PER_VEC * N_KEYS / (q_med * 1e-3) / 1e9
        score_call_gbs = SCORE_BYTES_PER_KEY * N_KEYS / (s_med * 1e-3) / 1e9
        quant_gbs = QUANT_BYTES_PER_VEC * N_KEYS / (kq_ms * 1e-3) / 1e9
        score_gbs = SCORE_BYTES_PER_KEY * N_KEYS / (ks_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC,
            "value": world * N_KEYS / (q_med * 1e-3) / 1e6,
            "unit": "Mvec/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps,
            "repeats": repeats,
            "ms_per_step_min_max": [min(totals) / args.steps, max(totals) / args.steps],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 (rotation as 3 fp16 tensor-core passes, fp32 accumulate)", "data": "synthetic",
            "config": workload_config(world),
            "attention_score": {
                "value": world * N_KEYS / (s_med * 1e-3) / 1e9, "unit": "Gkeys/s", "queries": N_QUERIES,
                "ms": s_med,
                "roofline": {"bound": "hbm", "achieved": score_gbs, "peak": peak, "unit": "GB/s",
                             "frac": score_gbs / peak, "frac_of_8TBs": score_gbs / 8000.0,
                             "traffic": traffic_bytes(*TRAFFIC_SCORE_262144),
                             "traffic_source": "ncu dram__bytes of one launch over 262,144 keys (profiles/), scaled by the keys",
                             "bytes_per_key": SCORE_BYTES_PER_KEY, "peak_kind": peak_kind,
                             "kernel": "score_tc_kernel<3,32,128>: median launch duration inside the timed steps (CUDA events recorded by the library around the launch)",
                             "kernel_ms": ks_ms, "call_ms": s_med, "call_achieved": score_call_gbs, "call_frac": score_call_gbs / peak,
                             "call": "attention_scores call: preparation kernel + scoring kernel"}},
            "quantize_ms": q_med,
            "roofline": {"bound": "hbm", "achieved": quant_gbs, "peak": peak, "unit": "GB/s",
                         "frac": quant_gbs / peak, "frac_of_8TBs": quant_gbs / 8000.0,
                         "traffic": traffic_bytes(*TRAFFIC_QUANT_262144),
                         "traffic_source": "ncu dram__bytes of one launch over 262,144 keys (profiles/), scaled by the keys",
                         "bytes_per_vector": QUANT_BYTES_PER_VEC, "peak_kind": peak_kind,
                         "kernel": "tensor_quantize_kernel<128,3,true>: median launch duration inside the timed steps (CUDA events recorded by the library around the launch)",
                         "kernel_ms": kq_ms, "call_ms": q_med, "call_achieved": quant_call_gbs, "call_frac": quant_call_gbs / peak,
                         "call": "tq_prod_quantize call: clearing of the work lists + tensor-core kernel + exact second stage (two launches)"},
            "e2e": dict({"value": world * N_KEYS / (e2e_ms * 1e-3) / 1e6, "unit": "Mvec/s", "ms_runs_rank0": e2e_runs,
                         "h2d_bytes_per_step": N_KEYS * D * 4, "d2h_bytes_per_step": d2h,
                         "what": "quantize_to_host(TurboQuantProd, pinned NumPy keys): chunked H2D, quantize, D2H into reused pinned buffers"},
                        **e2e_extra),
            "gpu_launches": launches,
            "gpu_launches_what": "kernels of libtq_sm100.so launched inside one timed region of K steps (tq_kernel_launches), this rank",
            "clocks": clocks,
            "other_calls": other,
        }
        if parity is not None:
            line["parity"] = parity
        if quality is not None:
            line["quality"] = quality
        if configs is not None:
            line["configs"] = configs
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


# DRAM bytes (read, written) of one launch of the dominant kernels over 262,144 keys, from the ncu captures
# summarised in profiles/ (dram__bytes_read.sum, dram__bytes_write.sum); both grow in proportion to the keys.
# (the score matrix of the small case stays in L2 during the capture: its 33.5 MB are counted as written here, as they
# are at the bench's size, where the matrix is larger than L2)
TRAFFIC_QUANT_262144 = (136.1e6, 21.1e6)
TRAFFIC_SCORE_262144 = (18.95e6, 33.5e6)

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
    """DRAM bytes of one launch of the dominant kernel at this run's size, scaled from the capture over 262,144
    keys.  None for a workload other than the captured one (d = 128, bits = 4, 32 queries)."""
    if D != 128 or BITS != 4 or N_QUERIES != 32:
        return None
    return (read_262144 + write_262144) * N_KEYS / 262144.0


def run_configs(tg, torch, timed, peak, dev):
    """The other configurations of the benchmark list on one GPU, device-resident inputs, CUDA events:
    1: TurboQuantMSE(128, 4) quantize + dequantize of 65,536 vectors (inputs rotate through eight buffers, so
       that no call finds its input in L2);
    3: KV-cache keys, batch 8 x 8 KV heads x 32,768 tokens x 128 with four outlier channels per head scaled x10,
       TurboQuantProd bits = 3, decode-step scores for 32 query heads (4 per KV head);
    4: bits 1..4 x dimension 64 / 128 / 256, 4,194,304 vectors, both classes: quantize, dequantize, scores for 16
       queries;
    5: the sharded retrieval configuration, see run_retrieval (here on this one GPU)."""
    out = {}
    # ---- 1 ------------------------------------------------------------------------------------------
    n1, sets = 65536, 8
    mse = tg.TurboQuantMSE(128, 4, seed=SEED)
    bufs = [torch.randn((n1, 128), device=dev, generator=torch.Generator(device=dev).manual_seed(20261 + i)) for i in range(sets)]
    encs = [mse.quantize(b) for b in bufs]
    turn = {"i": 0}

    def q1():
        turn["i"] = (turn["i"] + 1) % sets
        return mse.quantize(bufs[turn["i"]])

    def d1():
        turn["i"] = (turn["i"] + 1) % sets
        return mse.dequantize(encs[turn["i"]])
    nb = mse_bytes(128, 4)
    out["config1_mse_d128_b4_n65536"] = {
        "quantize": rate_row(timed(q1, inner=8), n1, nb, "B/vector", peak),
        "dequantize": rate_row(timed(d1, inner=8), n1, nb, "B/vector", peak),
        "reconstruction_mse": float(torch.mean((bufs[0] - mse.dequantize(encs[0])) ** 2)),
        "note": "a call of 65,536 vectors lasts ~20 us: launch-bound, three kernels per quantize"}
    del bufs, encs
    # ---- 3 ------------------------------------------------------------------------------------------
    b, h, t, d = 8, 8, 32768, 128
    gen = torch.Generator(device=dev).manual_seed(20263)
    kx = torch.randn((b, h, t, d), device=dev, generator=gen)
    out_rng = np.random.default_rng(20280)
    for hh in range(h):
        ch = torch.as_tensor(out_rng.choice(d, 4, replace=False), device=dev)
        kx[:, hh, :, ch] *= 10.0
    p3 = tg.TurboQuantProd(d, 3, seed=SEED)
    flat = kx.view(-1, d)
    enc3 = p3.quantize(flat)
    q3 = torch.randn((b * h * 4, d), device=dev, generator=gen)      # query head g of a sequence uses KV head g // 4
    kb3 = key_bytes(d, 3)
    out["config3_kv_cache_8x8x32768_bits3"] = {
        "quantize": rate_row(timed(lambda: p3.quantize(flat), inner=2), b * h * t, prod_bytes(d, 3), "B/key", peak),
        "decode_scores_4_queries_per_kv_head": rate_row(
            timed(lambda: p3.attention_scores(q3, enc3, groups=b * h)), b * h * t, kb3 + 16,
            "B/key: packed key in, 4 scores out", peak, groups=b * h)}
    del kx, flat, enc3, q3
    torch.cuda.empty_cache()
    # ---- 4 ------------------------------------------------------------------------------------------
    n4 = 4194304
    grid = {}
    for d in (64, 128, 256):
        x4 = torch.randn((n4, d), device=dev, generator=torch.Generator(device=dev).manual_seed(20264 + d))
        q4 = torch.randn((16, d), device=dev, generator=torch.Generator(device=dev).manual_seed(20274))
        for bits in (1, 2, 3, 4):
            m = tg.TurboQuantMSE(d, bits, seed=SEED)
            p = tg.TurboQuantProd(d, bits, seed=SEED)
            em, ep = m.quantize(x4), p.quantize(x4)
            inner = 1 if d == 256 else 2
            reps = 3 if d == 256 else 5
            grid[f"d{d}_b{bits}"] = {
                "mse_quantize": rate_row(timed(lambda: m.quantize(x4), reps=reps, inner=inner), n4, mse_bytes(d, bits), "B/vector", peak),
                "mse_dequantize": rate_row(timed(lambda: m.dequantize(em), reps=reps, inner=inner), n4, mse_bytes(d, bits), "B/vector", peak),
                "prod_quantize": rate_row(timed(lambda: p.quantize(x4), reps=reps, inner=inner), n4, prod_bytes(d, bits), "B/vector", peak),
                "prod_dequantize": rate_row(timed(lambda: p.dequantize(ep), reps=reps, inner=inner), n4, prod_bytes(d, bits), "B/vector", peak),
                "scores_16_queries": rate_row(timed(lambda: p.attention_scores(q4, ep), reps=reps, inner=inner), n4,
                                              key_bytes(d, bits) + 64, "B/key: packed key in, 16 scores out", peak)}
            del em, ep, m, p
        del x4
        torch.cuda.empty_cache()
    out["config4_sweep_n4194304"] = grid
    # ---- 5 ------------------------------------------------------------------------------------------
    out["config5_retrieval_134217728_keys"] = retrieval(tg, torch, dev, 134217728, 5, 2, peak, oracle_chunk=True)
    return out


def retrieval(tg, torch, dev, n_total, steps, warmup, peak, oracle_chunk):
    """Sharded retrieval at box scale: `n_total` TurboQuantProd(128, 4) keys split evenly over the ranks, 64 queries,
    per-shard top-100 merged over NCCL into a global top-100 per query.  Keys are generated on the device per chunk of
    2^20 (torch Philox, seed 20265 * 2^32 + chunk), quantized and dropped; only the packed encoding stays (72 B/key).
    Returns the rates and the outcome of the checks: descending scores, unique in-range indices, agreement with an
    independent pass over the chunk that holds query 0's best key and, with `oracle_chunk`, that chunk copied to the
    host and fed to the NumPy oracle (two queries, top-100 compared as index sets)."""
    import torch.distributed as dist
    from project_tensor_b200.sharded import ShardedKeyIndex, shard_range
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    chunk, n_q, k = 1 << 20, 64, TOPK
    quant = tg.TurboQuantProd(D, BITS, seed=SEED)
    index = ShardedKeyIndex(quant, n_total)
    q_np = np.random.default_rng(20275).standard_normal((n_q, D)).astype(np.float32)
    queries = torch.from_numpy(q_np).to(dev)

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
    for _ in range(max(warmup, 1)):
        top_s, top_i = index.search(queries, k)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(steps):
        top_s, top_i = index.search(queries, k)
    e1.record()
    torch.cuda.synchronize()
    # end to end: NumPy queries in, NumPy top-100 out, packed keys resident
    t0 = time.perf_counter()
    for _ in range(steps):
        hs, hi = index.search(q_np, k)
        hs, hi = hs.cpu(), hi.cpu()
    e2e_ms = 1e3 * (time.perf_counter() - t0) / steps
    times = torch.tensor([add_ms, e0.elapsed_time(e1) / steps, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    add_ms, search_ms, e2e_ms = (float(v) for v in times.tolist())

    # ---- checks that do not depend on the size --------------------------------------------------
    checks = {"descending": bool((top_s[:, :-1] >= top_s[:, 1:]).all()),
              "indices_in_range": bool(((top_i >= 0) & (top_i < n_total)).all()),
              "indices_unique": all(len(set(row)) == k for row in top_i.tolist())}
    c_best = int(top_i[0, 0].item()) // chunk
    x_best = make_chunk(c_best)
    enc = quant.quantize(x_best)
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
    if oracle_chunk and rank == 0:
        # that chunk on the CPU: the oracle's encoding and its scores for two queries; the 100 best keys of the chunk must
        # be the ones the CUDA path finds in it (a key whose score ties the 100th within the tolerance may swap)
        orc, pp = oracle_params()
        xh = x_best.cpu().numpy()
        enc_o = orc.prod_quantize(pp, xh)
        loc_s, loc_i = quant.attention_scores(queries, enc, topk=k)
        agree = []
        for qi in (0, n_q - 1):
            ref = orc.prod_attention_score(pp, q_np[qi], *enc_o)
            ref_top = np.argsort(-ref, kind="stable")[:k]
            mine = set(loc_i[qi].tolist())
            tol = 1e-4 * float(np.linalg.norm(q_np[qi]) * np.max(enc_o[3])) / math.sqrt(D)
            missing = [j for j in ref_top.tolist() if j not in mine and ref[j] > ref[ref_top[-1]] + 2 * tol]
            agree.append((len(mine & set(ref_top.tolist())), len(missing)))
        checks["oracle_chunk_top100_sets_agree"] = all(m == 0 and a >= k - 2 for a, m in agree)
        checks["oracle_chunk_overlap"] = [a for a, _ in agree]
    del x_best, enc, part
    kb = key_bytes(D, BITS)
    search_gbs = kb * n_total / (search_ms * 1e-3) / 1e9
    return {
        "n_gpus": world, "keys": n_total, "keys_per_gpu": n_total // world, "queries": n_q, "topk": k,
        "quantize_Mvec_per_s": n_total / (add_ms * 1e-3) / 1e6, "quantize_ms_total": add_ms,
        "quantize_frac_of_measured_hbm": QUANT_BYTES_PER_VEC * n_total / (add_ms * 1e-3) / 1e9 / peak / world,
        "search_ms": search_ms, "search_Gkeys_per_s": n_total / (search_ms * 1e-3) / 1e9,
        "search_Gpairs_per_s": n_total * n_q / (search_ms * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "achieved": search_gbs / world, "peak": peak, "unit": "GB/s", "frac": search_gbs / peak / world,
                     "bytes_per_key": kb, "traffic": None,
                     "note": "per GPU; 64 queries cost 5 x 2 x 128 x 64 = 82 KFLOP of tensor work per 72-byte key, so the contractions bound this call, not HBM"},
        "e2e": {"value": n_total / (e2e_ms * 1e-3) / 1e9, "unit": "Gkeys/s", "ms": e2e_ms,
                "h2d_bytes_per_step": n_q * D * 4, "d2h_bytes_per_step": n_q * k * 12,
                "what": "ShardedKeyIndex.search(NumPy queries) -> global top-100 copied to the host; packed keys resident"},
        "packed_GB_per_gpu": (n_total // world) * kb / 1e9, "data": "synthetic (torch Philox per 2^20-key chunk)", "checks": checks}


def run_retrieval(args):
    import torch
    import torch.distributed as dist
    import project_tensor_b200 as tg
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.total_keys % ((1 << 20) * world):
        raise SystemExit("--total-keys must be a multiple of 2^20 keys per rank")
    peak, _ = measured_peaks()
    res = retrieval(tg, torch, dev, args.total_keys, min(args.steps, 5), args.warmup, peak, oracle_chunk=(world == 1))
    if rank == 0:
        line = {"metric": "sharded retrieval: quantize Mvec/s and top-%d search Gkeys/s" % TOPK,
                "value": res["search_Gkeys_per_s"], "unit": "Gkeys/s", "n_gpus": world, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"TurboQuantProd d={D} bits={BITS}: {args.total_keys} keys over {world} GPU(s), 64 queries, "
                                       f"per-shard top-{TOPK} + NCCL all-gather + merge", "keys_per_gpu": args.total_keys // world}}
        line.update(res)
        if world == 1:
            n_sample = 262144
            cq, cs = time_oracle(n_sample, n_sample, 2, 2)
            line["cpu_baseline"] = {"value": n_sample / (cs * 64) / 1e9, "unit": "Gkeys/s", "cores": host_threads(), "kind": "port",
                                    "quantize_Mvec_per_s": n_sample / cq / 1e6,
                                    "sample": f"NumPy oracle: one query x {n_sample} keys (best of 2) multiplied by 64 queries; no top-k pass"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if not all(v for v in res["checks"].values() if isinstance(v, bool)):
        raise SystemExit("retrieval checks failed: %r" % (res["checks"],))


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
                    help="leave out the end-to-end, parity, configuration and CPU-baseline legs (profiler captures)")
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
