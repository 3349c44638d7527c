#!/usr/bin/env python
"""Benchmark of the vt:: data-parallel op path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-suite]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Headline line (one JSON object on stdout, printed by rank 0):

  workload  the sharded fp32 sum over a [2^32] tensor (16 GiB, N(0,1)), split along dim 0
            across the N ranks: every rank reduces its shard to an fp32 partial with one
            kernel launch, and (N > 1) one 4-byte NCCL all-reduce on the same stream combines
            the partials.  Total work is fixed ("strong" scaling); value = 2^32 elements /
            step time, whole job, max over ranks, timed with CUDA events.  Shards are
            >= 2 GiB, far above the 126 MB L2, so no flush is needed between iterations.
  roofline  the local reduce kernel: algorithmic bytes (4 B per element of the shard) per
            launch / mean CUDA-event duration of that launch, against the measured HBM copy
            bandwidth in MEASURED_PEAKS.json.
  e2e       the same sum with the input in PINNED HOST memory: every step copies the shard
            host->device in chunks (copy stream) overlapped with per-chunk partial sums
            (compute stream), combines, and reads the 4-byte result back.
  ops       (N = 1 only) the per-op table the metric asks for: every named vt:: op at the
            shapes of the other benchmark configurations, each with ms, GB/s and the fraction
            of the measured HBM bandwidth and of the nominal 8 TB/s.
  cpu_baseline  (N = 1 only) the reference's own single-threaded CPU sum
            (vbt_default_sum_impl compiled from its sources) on a bounded sample.

--impl reference times the reference's CPU implementation of the headline workload on the
host (a bounded sample per step; the reference's CPU path is serial, so one thread) and prints
the same line with "impl": "reference"; `host_parallel` adds the figure a caller gets who
shards the slice over all host threads himself.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOTAL_ELEMS = 1 << 32
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per element moved by one launch of the local reduce kernel, from the ncu capture
# of a 2 GiB shard (dram__bytes_read.sum + dram__bytes_write.sum; traffic grows in proportion
# to the shard).
REDUCE_TRAFFIC_BYTES_PER_ELEM = 2151534080 / (1 << 29)  # 2 147 509 504 B read + 4 024 576 B written for 2^29 elements


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms during a timed region."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.tmp.flush()
        rows = []
        with open(self.tmp.name) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 8:
                    rows.append(parts)
        os.unlink(self.tmp.name)
        if not rows:
            return out
        sm = sorted(float(r[1]) for r in rows if r[1].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(r[4 + k].lower().startswith("active") for r in rows)]
        out.update(sm_mhz=sm[len(sm) // 2] if sm else None,
                   sm_max_mhz=float(rows[0][2]) if rows[0][2].replace(".", "").isdigit() else None,
                   power_w_max=max(float(r[3]) for r in rows if r[3].replace(".", "").isdigit()),
                   reasons=reasons, samples=len(rows))
        return out


def env_ranks():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


# ------------------------------------------------------------------------------------------
# reference arm: the reference's CPU sum on the host cores
# ------------------------------------------------------------------------------------------
def cpu_reference_sum(sample_elems: int, reps: int):
    """Times vbt_default_sum_impl (reference CPU code, single-threaded by design:
    include/vbt/core/tensor_iterator/core.h:210) when oracle/_ref is present, else the C
    restatement, on `sample_elems` fp32 N(0,1) values; returns (elements/s, kind)."""
    import numpy as np
    import oracle
    rng = np.random.default_rng(4)
    x = rng.standard_normal(sample_elems, dtype=np.float32)
    if oracle.have_ref():
        fn, kind = (lambda: oracle.ref().sum(x, oracle.F32, [])), "reference"
    else:
        fn, kind = (lambda: oracle.port().reduce("sum", x, oracle.F32)), "port"
    result = float(fn())
    best = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        best.append(time.perf_counter() - t0)
    return sample_elems / (sum(best) / len(best)), kind, sum(best), x, result


def run_reference(args):
    rank, _, world = env_ranks()
    if rank != 0:
        return
    # The reference's CPU path has no threading anywhere (its reduce loops, TensorIterator and
    # Fabric are serial), so the arm's value is its sum on ONE thread.  For transparency the
    # line also carries what a caller gets who shards the tensor over all host threads himself,
    # each thread running the reference's sum on its slice (`host_parallel`): that variant is
    # bound by host DRAM bandwidth.
    import concurrent.futures as cf
    import numpy as np
    import oracle
    if oracle.have_ref():
        ref = oracle.ref()
        one, kind = (lambda x: float(ref.sum(x, oracle.F32, []))), "reference"
    else:
        port = oracle.port()
        one, kind = (lambda x: float(port.reduce("sum", x, oracle.F32))), "port"
    rng = np.random.default_rng(4)
    sample = 1 << 28  # 1 GiB of the 16 GiB tensor per step
    x = rng.standard_normal(sample, dtype=np.float32)
    for _ in range(max(1, min(args.warmup, 3))):
        one(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one(x)
    dt = (time.perf_counter() - t0) / args.steps
    value = sample / dt
    sample_desc = f"{sample} of {TOTAL_ELEMS} fp32 elements per step (contiguous slice), 1 thread"
    threads = max(1, min(os.cpu_count() or 1, 64))
    host_parallel = None
    if threads > 1:
        per_thread = sample // threads
        xs = [x[i * per_thread:(i + 1) * per_thread] for i in range(threads)]
        pool = cf.ThreadPoolExecutor(max_workers=threads)
        for _ in range(2):
            sum(pool.map(one, xs))
        t0 = time.perf_counter()
        for _ in range(max(3, args.steps)):
            sum(pool.map(one, xs))
        dtp = (time.perf_counter() - t0) / max(3, args.steps)
        pool.shutdown()
        host_parallel = {"value": per_thread * threads / dtp, "unit": "elements/s", "threads": threads,
                         "note": "not a reference code path: the caller shards the slice over threads, "
                                 "each runs the reference's single-threaded sum"}
    threads = 1
    line = {
        "impl": "reference", "metric": "sharded fp32 sum throughput (elements/s; HBM GB/s in roofline)",
        "value": value, "unit": "elements/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "elements/s", "cores": threads, "kind": kind, "sample": sample_desc},
        "e2e": {"value": value, "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host_cores": os.cpu_count(),
    }
    if host_parallel is not None:
        line["host_parallel"] = host_parallel
    emit(line)


def workload_config(n, fused=False):
    if n == 1:
        coll = "none"
    elif fused:
        coll = ("inside the reduce kernel: every partial goes to every rank's exchange buffer as one 8-byte word "
                "(value + the call's epoch) by peer stores over NVLink; the reader polls the word itself and folds "
                "in rank order (no flags, no fence, no collective library call)")
    else:
        coll = "ncclAllReduce(sum, 4 bytes) after the local kernel"
    return {"workload": "c5_sharded_sum_f32_2p32" if TOTAL_ELEMS == 1 << 32 else "c5_sharded_sum_f32_reduced",
            "tensor": f"[{TOTAL_ELEMS}] fp32 N(0,1), seed 4",
            "sharding": f"sharded_1d_row over {n} rank(s), {TOTAL_ELEMS // n} elements per rank",
            "collective": coll,
            "l2_policy": "inputs larger than L2 (>= 2 GiB per rank); no flush needed"}


# ------------------------------------------------------------------------------------------
# per-op suite (N = 1): every named op at the benchmark configurations' shapes
# ------------------------------------------------------------------------------------------
def time_op(torch, fn, iters, warm=3, graph=True):
    """Mean device time of fn(i) in ms.  The calls are captured once into a CUDA graph and the
    graph is replayed, so that host-side launch cost (Python, ctypes) does not sit between
    kernels of a few microseconds; falls back to an eager loop if capture is refused."""
    for _ in range(warm):
        fn(0)
    torch.cuda.synchronize()
    s = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    if graph:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(iters):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            reps = 3
            s.record()
            for _ in range(reps):
                g.replay()
            e.record()
            torch.cuda.synchronize()
            ms = s.elapsed_time(e) / (iters * reps)
            del g
            return ms, "cuda-graph replay"
        except Exception:
            torch.cuda.synchronize()
    s.record()
    for i in range(iters):
        fn(i)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters, "eager loop"


def op_suite(torch, peak_gbs, scale="full", which=("c1", "c2", "c3", "c4", "ew")):
    """Returns a list of {op, config, bytes, elements, ms, gbs, frac_measured, frac_8tbs}.
    Inputs smaller than L2 are rotated over enough distinct buffers to exceed it."""
    import numpy as np
    from vibetensor_b200 import kernels, ops
    dev = "cuda"
    res = []

    small = scale == "small"

    def add(op, config, nbytes, nelem, timed, launches=1, note=None):
        ms, how = timed
        gbs = nbytes / (ms * 1e-3) / 1e9
        r = {"op": op, "config": config, "bytes": int(nbytes), "elements": int(nelem), "ms": round(ms, 5),
             "gbs": round(gbs, 1), "frac_measured": round(gbs / peak_gbs, 4),
             "frac_8tbs": round(gbs / NOMINAL_HBM_GBS, 4), "elements_per_s": nelem / (ms * 1e-3),
             "launches": launches, "timing": how}
        if note:
            r["note"] = note
        res.append(r)

    # the reference's own Triton kernels for the row ops, timed beside ours when an unmodified copy
    # of its kernel package is present (single-GPU runs; baseline/install_ref.sh)
    ref_k = None
    try:
        from baseline import ref_kernels
        if ref_kernels.available():
            ref_k = ref_kernels.load()
    except Exception:
        ref_k = None

    g = torch.Generator(device=dev)
    # ---- C1: [4096,4096] fp32 reductions, contiguous and transposed view; 4 buffers = 256 MiB > L2
    g.manual_seed(0)
    xs = [torch.randn((4096, 4096), device=dev, generator=g) for _ in range(4 if "c1" in which else 0)]
    for name, fn, dim, outb in (("sum", ops.sum, -1, 4), ("mean", ops.mean, 0, 4), ("amax", ops.amax, -1, 4),
                                ("argmax", ops.argmax, -1, 8)):
        for label, view in ((("contig", lambda t: t), ("transposed", lambda t: t.t())) if "c1" in which else ()):
            ms = time_op(torch, lambda i: fn(view(xs[i % 4]), dim), 40)
            add(f"{name}(dim={dim})", f"C1 [4096,4096] fp32 {label}", 4096 * 4096 * 4 + 4096 * outb,
                4096 * 4096, ms, note="rotating 4 inputs (256 MiB) to defeat L2")
    del xs
    # ---- C4: row ops
    for shape in (() if "c4" not in which else ((4096, 4096), (32768, 128)) if small else ((32768, 4096), (262144, 128))):
        for dt, es in ((torch.float32, 4), (torch.bfloat16, 2)):
            g.manual_seed(3)
            nbuf = max(1, int(np.ceil(300e6 / (shape[0] * shape[1] * es))))
            xs = [(3 * torch.randn(shape, device=dev, generator=g)).to(dt) for _ in range(nbuf)]
            gamma = 1 + 0.02 * torch.randn(shape[1], device=dev, generator=g)
            n = shape[0] * shape[1]
            ms = time_op(torch, lambda i: kernels.softmax(xs[i % nbuf]), 20)
            add("softmax", f"C4 {list(shape)} {str(dt)[6:]}", 2 * n * es, n, ms)
            ms = time_op(torch, lambda i: kernels.rmsnorm(xs[i % nbuf], gamma, 1e-6), 20)
            add("rmsnorm", f"C4 {list(shape)} {str(dt)[6:]}", 2 * n * es + shape[1] * 4 + shape[0] * 4, n, ms)
            if ref_k is not None:
                try:
                    with torch.no_grad():
                        ms = time_op(torch, lambda i: ref_k.softmax(xs[i % nbuf], -1), 10)
                        add("softmax -- reference Triton kernel, same box", f"C4 {list(shape)} {str(dt)[6:]}",
                            2 * n * es, n, ms, note="vibe_kernels/softmax/impl/triton_impl.py, unmodified; same algorithmic bytes")
                        ms = time_op(torch, lambda i: ref_k.rmsnorm_fn.apply(xs[i % nbuf], gamma, 1e-6), 10)
                        add("rmsnorm -- reference Triton kernel, same box", f"C4 {list(shape)} {str(dt)[6:]}",
                            2 * n * es + shape[1] * 4 + shape[0] * 4, n, ms,
                            note="vibe_kernels/rmsnorm/impl/triton_impl.py, unmodified; same algorithmic bytes")
                except Exception as ex:
                    res.append({"op": "reference Triton kernels", "config": f"C4 {list(shape)} {str(dt)[6:]}",
                                "error": str(ex)[:200]})
            # backward: the saved tensor rotates through the forward's buffers and dy through as
            # many buffers of its own, so that neither stream is served from L2
            inv = kernels.rmsnorm(xs[0], gamma, 1e-6)[1]
            dys = [torch.randn(shape, device=dev, generator=g).to(dt) for _ in range(nbuf)]
            ms = time_op(torch, lambda i: kernels.rmsnorm_backward(dys[i % nbuf], xs[i % nbuf], inv, gamma), 20)
            add("rmsnorm_backward (dx, dgamma)", f"C4 {list(shape)} {str(dt)[6:]}",
                3 * n * es + 2 * shape[1] * 4 + shape[0] * 4, n, ms, launches=2,
                note="per-block dgamma partial rows + fixed-order fold, no atomics")
            ms = time_op(torch, lambda i: kernels.softmax_backward(dys[i % nbuf], xs[i % nbuf]), 20)
            add("softmax_backward", f"C4 {list(shape)} {str(dt)[6:]}", 3 * n * es, n, ms)
            del xs, dys
    if "c2" in which:
        # ---- C2: gather / scatter_add on a [1,048,576 x 256] table with 4,194,304 indices
        V, D, N = 1 << 20, 256, (1 << 19 if small else 1 << 22)
        rng = np.random.default_rng(2)
        table = torch.randn((V, D), device=dev)
        idx_u = torch.from_numpy(rng.integers(0, V, N).astype(np.int64)).to(dev)
        p = np.arange(1, V + 1, dtype=np.float64) ** -1.1
        ranks = np.searchsorted(np.cumsum(p / p.sum()), rng.random(N))
        idx_z = torch.from_numpy(rng.permutation(V)[np.minimum(ranks, V - 1)].astype(np.int64)).to(dev)
        U = int(torch.unique(idx_z).numel())
        out = torch.empty((N, D), device=dev)
        st = ops.IndexStatus(dev)
        ms = time_op(torch, lambda i: ops.index_rows(table, idx_u, status=st, out=out), 5)
        add("index_rows/gather", f"C2 table [1048576,256] fp32, {N} uniform int64 indices", 2 * N * D * 4 + N * 8,
            N * D, ms)
        upd = torch.randn((N, D), device=dev)
        acc = torch.zeros((V, D), device=dev)
        ms = time_op(torch, lambda i: ops.index_put_rows_(acc, idx_z, upd, accumulate=True, status=st), 5)
        add("index_put_(accumulate)/scatter_add fp32", f"C2 Zipf(1.1) indices, {U} distinct rows",
            N * D * 4 + N * 8 + 2 * U * D * 4, N * D, ms, launches=8,
            note="rows grouped by two radix passes over a 16-bit hash of the row + per-run sums "
                 "(the default engine from 2^21 updates on)")
        acc.zero_()
        ms = time_op(torch, lambda i: ops.index_put_rows_(acc, idx_z, upd, accumulate=True, status=st,
                                                          deterministic=False), 5)
        add("index_put_(accumulate)/scatter_add fp32, atomics", f"C2 Zipf(1.1) indices, {U} distinct rows",
            N * D * 4 + N * 8 + 2 * U * D * 4, N * D, ms, note="block-local aggregation + vector atomics")
        del upd, acc, out, table
        updi = torch.randint(-1000, 1001, (N, D), device=dev, dtype=torch.int64)
        acci = torch.zeros((V, D), device=dev, dtype=torch.int64)
        ms = time_op(torch, lambda i: ops.index_put_rows_(acci, idx_z, updi, accumulate=True, status=st), 5)
        add("index_put_(accumulate)/scatter_add int64", f"C2 Zipf(1.1) indices, {U} distinct rows",
            N * D * 8 + N * 8 + 2 * U * D * 8, N * D, ms, launches=11,
            note="radix sort of (row, position) + per-row sums (the default engine for integer tables)")
        ms = time_op(torch, lambda i: ops.index_put_rows_(acci, idx_z, updi, accumulate=True, status=st,
                                                          deterministic=False), 5)
        add("index_put_(accumulate)/scatter_add int64, atomics", f"C2 Zipf(1.1) indices, {U} distinct rows",
            N * D * 8 + N * 8 + 2 * U * D * 8, N * D, ms, note="block-local aggregation + 64-bit atomics")
        st.check("bench", V)
        del updi, acci
        # ---- the reference's CUDA advanced-index form x[..., idx] and the bool-mask front end
        Bn, K0 = (1024, 65536) if small else (4096, 65536)
        src = torch.randn((Bn, K0), device=dev)
        idxl = torch.from_numpy(rng.integers(0, K0, K0).astype(np.int64)).to(dev)
        ms = time_op(torch, lambda i: ops.index_lastdim(src, idxl, status=st), 5)
        add("index (x[..., idx])", f"[{Bn},{K0}] fp32, {K0} uniform int64 indices", 2 * Bn * K0 * 4 + K0 * 8, Bn * K0, ms)
        del src
        Bn2, K02 = (4096, 16384) if small else (16384, 16384)
        src = torch.randn((Bn2, K02), device=dev)
        idx2 = torch.from_numpy(rng.integers(0, K02, K02).astype(np.int64)).to(dev)
        ms = time_op(torch, lambda i: ops.index_lastdim(src, idx2, status=st), 5)
        add("index (x[..., idx]), rows of 64 KiB", f"[{Bn2},{K02}] fp32, {K02} uniform int64 indices",
            2 * Bn2 * K02 * 4 + K02 * 8, Bn2 * K02, ms, note="row staged in shared memory")
        del src
        nm = 1 << (26 if small else 28)
        mask = torch.from_numpy(rng.random(nm) < 0.5).to(dev)
        cnt = int(mask.sum().item())
        ms = time_op(torch, lambda i: ops.mask_select(mask), 5)
        add("bool mask -> indices (device part)", f"[{nm}] bool, half true", nm + 8 * cnt, nm, ms, launches=3,
            note="count + scan + ranked writes on the stream; bytes = the mask once + 8 per true element")
        ms = time_op(torch, lambda i: ops.mask_to_indices(mask), 5, graph=False)
        add("bool mask -> indices, with the count read back", f"[{nm}] bool, half true", nm + 8 * cnt, nm, ms,
            launches=3, note="adds the 8-byte D2H read of the count and the stream synchronise; eager timing")
        del mask
    if "c3" in which:
        # ---- C3: bf16 broadcast chain into a transposed output view
        g.manual_seed(1)
        n0 = 8 if small else 64
        a = torch.randn((n0, 1, 512, 1), device=dev, generator=g).bfloat16()
        b = torch.randn((1, 128, 1, 1024), device=dev, generator=g).bfloat16()
        c = torch.randn((n0, 128, 1, 1024), device=dev, generator=g).bfloat16()
        base = torch.empty((n0, 1024, 512, 128), device=dev, dtype=torch.bfloat16)
        outv = base.transpose(1, 3)
        n = outv.numel()
        ms = time_op(torch, lambda i: ops.where_gt0_addcmul(a, b, c, out=outv), 5)
        add("where(a>0, a+b*c, 0) fused", f"C3 bf16 a[{n0},1,512,1] b[1,128,1,1024] c[{n0},128,1,1024] -> transpose(1,3) view",
            n * 2 + (a.numel() + b.numel() + c.numel()) * 2, n, ms)
        # the same expression as the reference has to run it: four launches with dense
        # temporaries (b*c is [n0,128,1,1024]; a + t1, a > 0 and the result are full size)
        if not small:
            zero = torch.zeros(1, device=dev, dtype=torch.bfloat16)
            shp = (n0, 128, 512, 1024)
            t1 = torch.empty((n0, 128, 1, 1024), device=dev, dtype=torch.bfloat16)
            t2 = torch.empty(shp, device=dev, dtype=torch.bfloat16)
            m = torch.empty((n0, 1, 512, 1), device=dev, dtype=torch.bool)

            def chain(i):
                ops.mul(b, c, out=t1)
                ops.add(a, t1, out=t2)
                ops.gt(a, zero, out=m)
                ops.where(m, t2, zero, out=outv)
            ms = time_op(torch, chain, 3)
            moved = 2 * t1.numel() * 2 + 3 * n * 2   # t1 written + read, t2 written + read, out written
            add("mul -> add -> gt -> where (4 launches)", "C3 bf16, same inputs, one launch per vt:: op",
                moved, n, ms, launches=4,
                note="bytes = traffic of the four launches (t2 written, t2 read, out written); same result as the fused op")
            del t1, t2, m
        del base, outv
    if "ew" in which:
        nE = 1 << 28
        x = torch.randn(nE, device=dev)
        y = torch.randn(nE, device=dev)
        o = torch.empty_like(x)
        for name, fn, nb in (("add fp32 dense", lambda i: ops.add(x, y, out=o), 12 * nE),
                             ("relu fp32 dense", lambda i: ops.relu(x, out=o), 8 * nE),
                             ("gelu fp32 dense", lambda i: ops.gelu(x, out=o), 8 * nE),
                             ("add fp32, host scalar operand", lambda i: ops.add(x, 1.5, out=o), 8 * nE)):
            ms = time_op(torch, fn, 10)
            add(name, f"[{nE}] contiguous", nb, nE, ms)
        xb, yb = x.bfloat16(), y[: 1 << 14].bfloat16()
        ob = torch.empty_like(xb)
        ms = time_op(torch, lambda i: ops.mul(xb.view(-1, 1 << 14), yb, out=ob.view(-1, 1 << 14)), 10)
        add("mul bf16, row-broadcast operand", f"[{nE >> 14},16384] * [16384]", 4 * nE, nE, ms)
        ycol = yb[: nE >> 14].reshape(-1, 1)
        ms = time_op(torch, lambda i: ops.mul(xb.view(-1, 1 << 14), ycol, out=ob.view(-1, 1 << 14)), 10)
        add("mul bf16, column-broadcast operand", f"[{nE >> 14},16384] * [{nE >> 14},1]", 4 * nE, nE, ms)
        ms = time_op(torch, lambda i: ops.add(x.view(-1, 1 << 14), y[: nE >> 14].reshape(-1, 1), out=o.view(-1, 1 << 14)), 10)
        add("add fp32, column-broadcast operand", f"[{nE >> 14},16384] + [{nE >> 14},1]", 8 * nE, nE, ms)
        cm = x > 0
        ms = time_op(torch, lambda i: ops.where(cm, x, y, out=o), 10)
        add("where fp32 dense", f"[{nE}] contiguous, bool condition", 13 * nE, nE, ms)
        xt = x.view(1 << 14, 1 << 14)
        ot = torch.empty_like(xt)
        ms = time_op(torch, lambda i: ops.copy_(ot, xt.t()), 10)
        add("contiguous() of a transposed view", "[16384,16384] fp32 transpose -> dense", 8 * nE, nE, ms)
        xbt = xb.view(1 << 14, 1 << 14)
        obt = torch.empty_like(xbt)
        ms = time_op(torch, lambda i: ops.copy_(obt, xbt.t()), 10)
        add("contiguous() of a transposed view", "[16384,16384] bf16 transpose -> dense", 4 * nE, nE, ms)
        ms = time_op(torch, lambda i: ops.add(xbt, xbt.t(), out=obt), 10)
        add("add bf16, tensor + its transpose", "[16384,16384] bf16", 6 * nE, nE, ms)
        del x, y, o, xb, yb, ob, cm, xt, ot, xbt, obt
    torch.cuda.empty_cache()
    return res


# ------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    rank, local_rank, world = env_ranks()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    n = world
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if n > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from vibetensor_b200 import fabric, ops

    peak_gbs, peak_kind = measured_peak()
    if args.suite_only:
        if rank == 0:
            suite = op_suite(torch, peak_gbs, args.suite_scale, tuple(args.suite_ops.split(',')))
            emit({"metric": "per-op HBM GB/s", "n_gpus": 1, "suite_scale": args.suite_scale,
                  "peak_gbs": peak_gbs, "peak_source": peak_kind, "ops": suite})
        return
    shard_elems = TOTAL_ELEMS // n
    # per-rank stream of the seed: shards are reproducible without one host holding 16 GiB
    g = torch.Generator(device=dev)
    g.manual_seed(4 * 1000 + rank)
    shard = torch.empty(shard_elems, device=dev, dtype=torch.float32)
    step_fill = 1 << 28
    for o in range(0, shard_elems, step_fill):
        shard[o:o + step_fill].normal_(generator=g)
    mesh = fabric.FabricMesh.from_world()
    ft = fabric.FabricTensor.sharded_1d_row(mesh, shard)
    assert ft.global_shape == (TOTAL_ELEMS,)

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the step, set up once: plan, descriptors, partial buffer and workspace are built here, so a
    # step is the local kernel launch plus (N > 1) the 4-byte all-reduce on the same stream
    prep = fabric.prepare_reduce("sum", ft, fused=False if args.no_fused else None)
    fused = prep.fused is not None
    result = None
    for _ in range(max(args.warmup, 3)):
        result = prep.run()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    kern_events = []
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        result = prep.run(kernel_events=ev)   # local kernel (timed by ev) + 4-byte combine
        kern_events.append(ev)
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    kern_all = sorted(a.elapsed_time(b) for a, b in kern_events)
    kern_ms = sum(kern_all) / len(kern_all)
    kern_stats = {"mean": kern_ms, "median": kern_all[len(kern_all) // 2], "min": kern_all[0], "max": kern_all[-1]}
    clocks = sampler.stop() if rank == 0 else None

    # correctness of what was timed: against an fp64 fold of the same shards, on the scale
    # max(|truth|, sigma * sqrt(N)) (sigma * sqrt(N) as sqrt(sum x^2))
    truth = torch.zeros((), device=dev, dtype=torch.float64)
    sq = torch.zeros((), device=dev, dtype=torch.float64)
    for o in range(0, shard_elems, step_fill):
        d = shard[o:o + step_fill].double()
        truth += d.sum()
        sq += d.pow(2).sum()
        del d
    if n > 1:
        dist.all_reduce(truth)
        dist.all_reduce(sq)
    scale = max(abs(truth.item()), sq.item() ** 0.5)
    rel = abs(result.double().item() - truth.item()) / scale
    assert rel <= 1e-5, f"sharded sum off by {rel:.3e} of max(|truth|, sigma*sqrt(N))"
    if fused:
        prep.comm.check()  # no exchange on this rank gave up waiting for a peer

    # ---- the other sharded reductions of the configuration: amax over the same tensor and
    # mean(dim=0) over a [1,048,576 x 4096] bf16 tensor split by rows (fp32 column partials,
    # one 16 KiB all-reduce, divide by the global row count, cast)
    sharded = []

    def timed(fn, steps):
        for _ in range(3):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        tt = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
        if n > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tt.item()

    prep_amax = None
    if not args.no_sharded_extras:
        k = max(1, min(args.steps, 10))
        prep_amax = fabric.prepare_reduce("max", ft, fused=False if args.no_fused else None)
        ms = timed(prep_amax.run, k)
        gmax = shard.max()
        if n > 1:
            dist.all_reduce(gmax, op=dist.ReduceOp.MAX)
        assert fabric.amax(ft).item() == gmax.item(), "sharded amax mismatch"
        assert prep_amax.run().item() == gmax.item(), "prepared sharded amax mismatch"
        sharded.append({"op": "amax", "tensor": f"[{TOTAL_ELEMS}] fp32", "ms_per_step": ms,
                        "fused_exchange": prep_amax.fused is not None,
                        "elements_per_s": TOTAL_ELEMS / (ms * 1e-3), "gb_per_s_whole_job": TOTAL_ELEMS * 4 / (ms * 1e-3) / 1e9})
        rows_total, cols = (1 << 20) * TOTAL_ELEMS // (1 << 32), 4096
        rows = rows_total // n
        xb = torch.empty((rows, cols), device=dev, dtype=torch.bfloat16)
        for o in range(0, rows, 1 << 14):
            xb[o:o + (1 << 14)].normal_(generator=g)
        fb = fabric.FabricTensor.sharded_1d_row(mesh, xb)
        prep_mean = fabric.prepare_reduce("mean", fb, dim=0, fused=False if args.no_fused else None)
        ms = timed(prep_mean.run, k)
        mcol = fabric.mean(fb, dim=0)
        assert torch.equal(prep_mean.run(), mcol), "prepared and one-off sharded mean differ"
        ref_col = xb.float().sum(0)
        if n > 1:
            dist.all_reduce(ref_col)
        ref_col = ref_col / (rows * n)
        assert torch.allclose(mcol.float(), ref_col, rtol=1e-2, atol=1e-2), "sharded bf16 mean(dim=0) off"
        ne = rows * n * cols
        sharded.append({"op": "mean(dim=0)", "tensor": f"[{rows * n},{cols}] bf16", "ms_per_step": ms,
                        "fused_exchange": prep_mean.fused is not None,
                        "elements_per_s": ne / (ms * 1e-3), "gb_per_s_whole_job": ne * 2 / (ms * 1e-3) / 1e9})
        del xb, fb, prep_mean

    # ---- vt::fabric_add with one operand on a peer GPU (rank 0 drives GPUs 0 and 1; the other
    # ranks wait on the rendezvous store, not on a device-side barrier)
    fabric_bin = None
    if n > 1 and not args.no_sharded_extras:
        store = dist.distributed_c10d._get_default_store()
        if rank == 0:
            try:
                fabric_bin = fabric_binary_leg(torch, ops, dev)
            except Exception as ex:
                fabric_bin = [{"op": "fabric_add", "error": str(ex)[:200]}]
            store.set("vbt_b200_fabric_leg_done", "1")
        else:
            store.wait(["vbt_b200_fabric_leg_done"])

    # ---- e2e: the shard starts in pinned host memory every step
    e2e = None
    if not args.no_e2e:
        try:
            e2e = run_e2e(torch, dist, ops, shard, n, args)
        except Exception as ex:  # host memory for the pinned copy may be unavailable
            e2e = {"value": None, "unit": "elements/s", "error": str(ex)[:200]}

    suite = None
    cpu = None
    prep = prep_amax = None
    if n == 1 and rank == 0:
        del shard, ft
        torch.cuda.empty_cache()
        if not args.no_suite:
            suite = op_suite(torch, peak_gbs, args.suite_scale, tuple(args.suite_ops.split(',')))
    ref_parity = None
    if n == 1 and rank == 0 and not args.no_cpu:
        v, kind, secs, sample, ref_sum = cpu_reference_sum(1 << 28, 8)
        cpu = {"value": v, "unit": "elements/s", "cores": 1, "kind": kind,
               "sample": f"8 passes over {1 << 28} of {TOTAL_ELEMS} fp32 elements ({secs:.1f} s), single thread "
                         f"(the reference CPU path is single-threaded); host has {os.cpu_count()} cores"}
        # the same sample through the GPU path: the kernel's and the reference loop's distance
        # from the fp64 truth, both on the scale max(|truth|, sigma * sqrt(N))
        ts = torch.from_numpy(sample).to(dev)
        ours = ops.sum(ts).item()
        t64 = ts.double().sum().item()
        sc = max(abs(t64), float(ts.double().pow(2).sum().sqrt().item()))
        ref_parity = {"sample_elements": int(sample.size), "kernel_vs_fp64": abs(ours - t64) / sc,
                      "reference_cpu_sum_vs_fp64": abs(ref_sum - t64) / sc,
                      "kernel_vs_reference_cpu_sum": abs(ours - ref_sum) / sc,
                      "note": "the reference adds left to right in fp32; its drift from the truth is its own"}
        del ts

    if rank == 0:
        shard_bytes = shard_elems * 4
        achieved = shard_bytes / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": "sharded fp32 sum throughput (elements/s; HBM GB/s in roofline)",
            "value": TOTAL_ELEMS / (ms_step * 1e-3), "unit": "elements/s", "n_gpus": n, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(n, fused),
            "gb_per_s_whole_job": TOTAL_ELEMS * 4 / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak_gbs, "unit": "GB/s",
                         "frac": round(achieved / peak_gbs, 4), "peak_source": peak_kind,
                         "frac_of_nominal_8tbs": round(achieved / NOMINAL_HBM_GBS, 4),
                         "kernel": "row_block_kernel<float, SumR<float>, 4>",
                         "bytes_per_launch": shard_bytes, "ms_per_launch": kern_ms,
                         "ms_per_launch_stats": kern_stats,
                         "traffic": (REDUCE_TRAFFIC_BYTES_PER_ELEM * shard_elems
                                     if REDUCE_TRAFFIC_BYTES_PER_ELEM is not None else None)},
            "e2e": e2e, "gpu_launches": args.steps * n, "clocks": clocks,
            "parity": {"err_vs_fp64_over_max_abs_truth_sigma_sqrt_n": rel, "bound": 1e-5,
                       "reference_sum_on_sample": ref_parity},
            "sharded_ops": sharded,
        }
        if fabric_bin is not None:
            line["fabric_elementwise"] = fabric_bin
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if suite is not None:
            line["ops"] = suite
        emit(line)
    if n > 1:
        dist.destroy_process_group()


def bind_to_gpu_numa_node(gpu_index: int):
    """Host-side only: run this process (and so first-touch its pinned buffer) on the CPUs of
    the NUMA node the GPU's PCIe slot hangs off.  Returns the node number, or None when the
    topology cannot be read (then nothing is changed)."""
    try:
        bdf = subprocess.run(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.strip().lower()
        if bdf.count(":") == 2 and len(bdf.split(":")[0]) == 8:
            bdf = bdf[4:]  # nvidia-smi prints an 8-digit PCI domain, sysfs a 4-digit one
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def fabric_binary_leg(torch, ops, dev):
    """vt::fabric_add on two GPUs of one process: a and the result on `dev`, b on the next GPU.
    Peer-load mode reads b in place over NVLink inside the elementwise kernel; copy-fallback
    copies it to local scratch first and then runs the local kernel."""
    d0 = dev.index
    d1 = (d0 + 1) % torch.cuda.device_count()
    nel = 1 << 28
    a = torch.randn(nel, device=dev)
    b = torch.randn(nel, device=torch.device("cuda", d1))
    out = torch.empty_like(a)
    want = a + b.to(dev)
    res = []
    for label, policy in (("peer_load", False), ("copy_fallback", "always")):
        _, mode = ops.fabric_binary("add", a, b, compute_device=d0, use_copy_fallback=policy, out=out)
        torch.cuda.synchronize(dev)
        ok = bool(torch.equal(out, want))
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(5)]
        for e0, e1 in evs:
            e0.record()
            ops.fabric_binary("add", a, b, compute_device=d0, use_copy_fallback=policy, out=out)
            e1.record()
        torch.cuda.synchronize(dev)
        ms = sorted(e0.elapsed_time(e1) for e0, e1 in evs)[2]
        res.append({"op": "fabric_add fp32", "config": f"[{nel}] a, out on GPU {d0}; b on GPU {d1}", "mode": mode,
                    "requested": label, "ms": ms, "link_gbs": nel * 4 / (ms * 1e-3) / 1e9,
                    "frac_of_measured_peer_copy_770gbs": nel * 4 / (ms * 1e-3) / 1e9 / 770.0, "matches_local_add": ok,
                    "note": "bound by NVLink: 4 bytes of b per element cross the link (measured peer copy on this pool: "
                            "770 GB/s per direction)"})
    return res


def run_e2e(torch, dist, ops, shard, n, args):
    """Host-resident input: per step, H2D of the whole shard from pinned memory in 64 MiB
    chunks alternating over two copy streams, per-chunk partial sums on the compute stream
    behind events, one combine, all-reduce, and a D2H read of the 4-byte result.  Also
    measures the same copies with no kernel behind them: the ceiling this leg can reach."""
    dev = shard.device
    steps = max(1, min(args.steps, 3))
    chunk = 1 << 24  # elements (64 MiB)
    nstage = 4
    nchunks = (shard.numel() + chunk - 1) // chunk
    node = bind_to_gpu_numa_node(dev.index or 0)
    host = torch.empty(shard.numel(), dtype=torch.float32, pin_memory=True)
    host.copy_(shard)  # the synthetic shard, now host-resident (first touched on the bound node)
    torch.cuda.synchronize()
    stage = [torch.empty(chunk, device=dev, dtype=torch.float32) for _ in range(nstage)]
    free_ev = [torch.cuda.Event() for _ in range(nstage)]
    copy_streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
    partials = torch.empty(nchunks, device=dev, dtype=torch.float32)
    out_host = torch.empty(1, dtype=torch.float32, pin_memory=True)
    compute = torch.cuda.current_stream(dev)
    chunk_sum = [ops.PreparedReduce("sum", stage[i], None, False, partial=True) for i in range(nstage)]
    final_sum = ops.PreparedReduce("sum", partials, None, False, partial=True)
    tail = shard.numel() - (nchunks - 1) * chunk  # elements of the last chunk

    def one_step(with_kernels=True):
        for c in range(nchunks):
            lo, hi = c * chunk, min((c + 1) * chunk, shard.numel())
            k = c % nstage
            cs = copy_streams[c % 2]
            with torch.cuda.stream(cs):
                cs.wait_event(free_ev[k])
                stage[k][: hi - lo].copy_(host[lo:hi], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(cs)
            compute.wait_event(ready)
            if with_kernels:
                if hi - lo == chunk:
                    p = chunk_sum[k].run()
                else:
                    p = ops.reduce("sum", stage[k][:tail], None, False, partial=True)
                partials[c:c + 1].copy_(p.reshape(1))
            free_ev[k].record(compute)
        if not with_kernels:
            compute.synchronize()
            return 0.0
        total = final_sum.run()
        if n > 1:
            dist.all_reduce(total)
        out_host.copy_(total.reshape(1), non_blocking=True)
        compute.synchronize()
        return float(out_host[0])

    def timed(with_kernels):
        for ev in free_ev:
            ev.record(compute)
        one_step(with_kernels)
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            val = one_step(with_kernels)
        torch.cuda.synchronize()
        dt = torch.tensor([(time.perf_counter() - t0) / steps], device=dev, dtype=torch.float64)
        if n > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return dt.item(), val

    dt, val = timed(True)
    dt_copy, _ = timed(False)
    del host
    return {"value": TOTAL_ELEMS / dt, "unit": "elements/s", "ms_per_step": dt * 1e3,
            "h2d_bytes_per_step": shard.numel() * 4 * n, "d2h_bytes_per_step": 4 * n, "steps": steps,
            "launches_per_step": (nchunks + 1) * n, "result": val,
            "h2d_ceiling": {"value": TOTAL_ELEMS / dt_copy, "unit": "elements/s", "ms_per_step": dt_copy * 1e3,
                            "gb_per_s_all_ranks": shard.numel() * 4 * n / dt_copy / 1e9,
                            "note": "the same pinned-memory copies with no kernel behind them"},
            "frac_of_h2d_ceiling": dt_copy / dt, "numa_node": node, "chunk_bytes": chunk * 4, "copy_streams": 2}


_JSON_OUT = sys.stdout


def emit(line: dict) -> None:
    """The one JSON line, on the process's original stdout."""
    print(json.dumps(line), file=_JSON_OUT, flush=True)


def main():
    global TOTAL_ELEMS, _JSON_OUT
    # Libraries (NCCL's version banner, for one) write to file descriptor 1.  Keep the real
    # stdout for the JSON line only and send everything else to stderr.
    sys.stdout.flush()
    _JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-suite", action="store_true", help="skip the per-op table (N = 1)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-resident end-to-end leg")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sharded-extras", action="store_true", help="skip the sharded amax / bf16 mean(dim=0) legs")
    ap.add_argument("--no-fused", action="store_true",
                    help="N > 1: combine with an NCCL all-reduce after the kernel instead of inside it")
    ap.add_argument("--suite-only", action="store_true", help="run only the per-op table")
    ap.add_argument("--suite-scale", default="full", choices=["full", "small"],
                    help="small: reduced C2/C3/C4 shapes (a few GB on the device) for profiler captures")
    ap.add_argument("--suite-ops", default="c1,c2,c3,c4,ew", help="which configurations the per-op table runs")
    ap.add_argument("--elems", type=int, default=TOTAL_ELEMS,
                    help="elements of the headline tensor (default 2^32; smaller only for profiler captures)")
    args = ap.parse_args()
    TOTAL_ELEMS = args.elems
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
