"""Benchmark of the `bits` top-k selection hot path (and its CPU baseline).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--k 256] [--impl reference]

Workload (the reference's selection sweep shape): a float32 distance matrix of q=1024 rows
by n=2^20 columns (4 GiB) per GPU, Uniform[0,1) from a seeded device generator (synthetic:
the reference itself only ever measures generated data), k=256 by default.  One step = one
pass of the selection over the whole matrix.  With N GPUs the matrix is database-sharded:
every rank holds its own q x n column block of a q x (N*n) matrix (weak scaling), selects
its local top-k, the candidates are all-gathered over NCCL and merged on every rank; the K timed
searches run as a stream (`ShardedSearch.submit_select` / `drain`): the all-gather of one search
is in flight while the next local selection runs, and all K are complete inside the timed region.

The JSON line carries: `value` (distances/s with the matrix resident in HBM), `e2e` (same
metric through the C ABI with HOST buffers: pinned host -> device copy of the matrix, the
selection, and the device -> host copy of the result, all inside the timed region),
`e2e_knn` (the reference binary's own flow: host points and queries -> device, distance matrix
made on the device, selection, result -> host),
`roofline` (algorithmic bytes / CUDA-event kernel time against the measured HBM peak),
`cpu_baseline` (the CPU port of the reference's OpenMP heap selection, timed on this host)
and `sweep` (other k and the adversarial descending-row input, kernel time only).

`--impl reference` times the reference's CPU selection alone (oracle/_ref when it was
compiled, else the oracle port) and prints the same line shape with "impl": "reference".
"""
import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import threading
import time

ROOT = pathlib.Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

Q = 1024
N_COLS = 1 << 20
METRIC = "bits top-k selection throughput"
UNIT = "distances/s"
# the reference's published H100-PCIe numbers for this shape (q=1024, n=2^20), by k:
# plots/kselection-hopper01-108424.csv lines 13, 45, 61, 106
# ncu: (2.4831 GB read + 5.6 MB written) / 592 rows, k = 256
NCU_DRAM_BYTES_PER_ROW = (2.4831e9 + 5.6e6) / 592
PUBLISHED_H100 = {32: 4.781e11, 128: 4.637e11, 256: 4.674e11, 2048: 3.599e11}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def wait_first_sample(self, limit_s=3.0):
        t_end = time.perf_counter() + limit_s
        while self.proc is not None and not self.lines and time.perf_counter() < t_end:
            time.sleep(0.02)
        self.lines.clear()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=5)
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) != 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_selection_baseline(host_matrix, k, budget_s=20.0):
    """Times the CPU port of the reference's OpenMP heap selection on a bounded row sample."""
    import numpy as np
    from oracle import oracle
    oracle.build()
    cores = oracle.num_threads()
    rows = min(host_matrix.shape[0], max(cores, 64))
    sample = np.ascontiguousarray(host_matrix[:rows])
    kind, what = "port", "port of parallel_knn::selection"
    run = lambda m: (oracle.select_heap(m, k), None)[1]
    try:
        # the reference's own parallel_knn::selection when it was compiled (it reports the time of
        # selection() alone, like the reference's main loop)
        from oracle import ref_select
        if ref_select.available():
            ref_select.select("parallel", sample[:cores], k)
            kind, what = "reference", "the reference's parallel_knn::selection compiled from its sources"
            run = lambda m: ref_select.select("parallel", m, k)[2]
    except Exception:
        kind, what = "port", "port of parallel_knn::selection"
        run = lambda m: (oracle.select_heap(m, k), None)[1]
    run(sample[:cores])  # warm the thread pool and the pages
    times = []
    spent = 0.0
    while len(times) < 5 and spent < budget_s:
        t0 = time.perf_counter()
        inner = run(sample)
        dt = time.perf_counter() - t0
        times.append(inner if inner is not None else dt)
        spent += dt
    best = statistics.median(times)
    return {"value": rows * host_matrix.shape[1] / best, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"first {rows} of {host_matrix.shape[0]} rows x {host_matrix.shape[1]} columns of the same "
                      f"matrix, k={k}, OpenMP heap selection ({what}), median of {len(times)} runs"}


def knn_section(bk, dev):
    """Fused k-NN (the other hot path): n = 2^20 points, q = 2^14 queries, Uniform[0,1), kernel
    time by CUDA events.  FP32 is the bit-exact mode; tf32 / bf16 run on tcgen05.  For the
    largest case the unfused pipelines (distance GEMM + bits selection, in query batches) and,
    where it was compiled, the reference's own fused-cache kernel are timed beside it."""
    import torch

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    n, q = 1 << 20, 1 << 14
    gen = torch.Generator(device=dev).manual_seed(42)
    result = {"n": n, "q": q, "data": "Uniform[0,1) coordinates, seed 42", "cases": {}}
    modes = (("fp32", bk.L2_PARTIAL), ("tf32", bk.L2_TF32), ("bf16", bk.L2_BF16))
    for dim, k in ((16, 32), (64, 128)):
        points = torch.rand((n, dim), generator=gen, device=dev)
        queries = torch.rand((q, dim), generator=gen, device=dev)
        out = (torch.empty((q, k), device=dev), torch.empty((q, k), dtype=torch.int32, device=dev))
        for name, mode in modes:
            ws = torch.empty(max(bk.fused_workspace_bytes(n, q, dim, k, mode), 256), dtype=torch.uint8, device=dev)
            ms = timed(lambda: bk.fused(points, queries, k, mode=mode, out=out, workspace=ws), 1 if name == "fp32" else 3)
            result["cases"][f"fused_{name}_dim{dim}_k{k}"] = {"ms": ms, "queries_per_s": q / (ms * 1e-3),
                                                             "distances_per_s": q * n / (ms * 1e-3)}
            del ws
        # unfused: distance matrix for 2048 queries at a time (8 GiB), then the bits selection
        qb = 2048
        dist = torch.empty((qb, n), device=dev)
        sel = (torch.empty((qb, k), device=dev), torch.empty((qb, k), dtype=torch.int32, device=dev))
        for name, mode in (("fp32", bk.L2_PARTIAL), ("bf16", bk.L2_BF16)):
            ws = torch.empty(max(bk.l2_workspace_bytes(n, qb, dim, mode), 256), dtype=torch.uint8, device=dev)

            def unfused():
                for b in range(0, q, qb):
                    bk.l2(points, queries[b:b + qb], mode=mode, out=dist, workspace=ws)
                    bk.select(dist, k, out=sel)

            ms = timed(unfused, 1)
            result["cases"][f"unfused_{name}_gemm_plus_bits_dim{dim}_k{k}"] = {"ms": ms, "queries_per_s": q / (ms * 1e-3)}
            del ws
        del dist
        try:
            from oracle import ref_select
            if ref_select.available():
                sub = 4096  # a quarter of the queries; the kernel is linear in q
                _, _, sec = ref_select.fused_cache(points.cpu().numpy(), queries[:sub].cpu().numpy(), k,
                                                   block_query_dim=1, dim_mult=1, repeats=1)
                result["cases"][f"reference_fused_cache_dim{dim}_k{k}"] = {
                    "ms": sec * 1e3 * (q / sub), "queries_per_s": sub / sec,
                    "note": "the reference's fused-cache kernel (8,4,2 / block-query-dim 1 / dim-mult 1) compiled "
                            f"from its sources, timed on {sub} queries and scaled to {q}"}
        except Exception as err:
            result["cases"][f"reference_fused_cache_dim{dim}_k{k}"] = {"unavailable": str(err)}
        torch.cuda.empty_cache()
    return result


def sharded_knn_section(bk, search, dev, rank, world, barrier, max_over_ranks):
    """The sharded search of the largest configuration, one shard per GPU: every rank holds 2^24
    points of dimension 64 (4 GiB; 8 ranks = the 2^27-point database), all 16384 queries, k = 128;
    fused tensor-core search of the shard (bf16 split images), one all-gather of the candidates,
    merge.  Queries per second of the whole job, device time, max over ranks."""
    import torch
    n_shard, q, dim, k = 1 << 24, 1 << 14, 64, 128
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    points = torch.rand((n_shard, dim), generator=gen, device=dev)
    gen_q = torch.Generator(device=dev).manual_seed(7)          # the same queries on every rank
    queries = torch.rand((q, dim), generator=gen_q, device=dev)
    mode = bk.L2_BF16
    ws = torch.empty(max(bk.fused_workspace_bytes(n_shard, q, dim, k, mode), 256), dtype=torch.uint8, device=dev)
    fin = (torch.empty((q, k), device=dev), torch.empty((q, k), dtype=torch.int32, device=dev))

    def step():
        search.knn(points, queries, k, rank * n_shard, out=None if world == 1 else fin, mode=mode, workspace=ws)

    step()
    barrier()
    steps = 3
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    bk.device_status()
    del points, ws
    torch.cuda.empty_cache()
    return {"n_total": n_shard * world, "n_per_gpu": n_shard, "q": q, "dim": dim, "k": k, "mode": "bf16 (tcgen05)",
            "ms_per_step": ms, "queries_per_s": q / (ms * 1e-3), "distances_per_s": q * n_shard * world / (ms * 1e-3),
            "steps": steps}


def run_profile_case(name):
    """Small cases of the k-NN kernels for profiler captures: a few hundred MB on the device,
    three launches each (inputs larger than L2 where the kernel streams them)."""
    import torch
    import __graft_entry__ as entry
    bk = entry.load_package()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(42)
    dim, k = 64, 128
    if name == "fused_tc_small":
        dim, k = 16, 16                                 # the consumer-bound end: few MMAs, few candidates
    if name in ("fused_tc", "fused_tc_small", "fused_fp32"):
        n, q = 1 << 18, 148 * 128                       # one query tile per SM
        mode = bk.L2_PARTIAL if name == "fused_fp32" else bk.L2_BF16
        if name == "fused_fp32":
            q = 148 * 2 * 128                           # two 128-query blocks per SM
        points = torch.rand((n, dim), generator=gen, device=dev)
        queries = torch.rand((q, dim), generator=gen, device=dev)
        ws = torch.empty(max(bk.fused_workspace_bytes(n, q, dim, k, mode), 256), dtype=torch.uint8, device=dev)
        out = (torch.empty((q, k), device=dev), torch.empty((q, k), dtype=torch.int32, device=dev))
        for _ in range(3):
            bk.fused(points, queries, k, mode=mode, out=out, workspace=ws)
    else:
        n, q = 1 << 18, 2048                            # 2 GiB distance matrix
        mode = bk.L2_BF16 if name == "l2_tc" else bk.L2_PARTIAL
        points = torch.rand((n, dim), generator=gen, device=dev)
        queries = torch.rand((q, dim), generator=gen, device=dev)
        ws = torch.empty(max(bk.l2_workspace_bytes(n, q, dim, mode), 256), dtype=torch.uint8, device=dev)
        out = torch.empty((q, n), device=dev)
        for _ in range(3):
            bk.l2(points, queries, mode=mode, out=out, workspace=ws)
    torch.cuda.synchronize()
    bk.device_status()
    print(json.dumps({"profile_case": name, "n": n, "q": q, "dim": dim, "k": k}))


def run_reference_arm(args):
    """The reference's own CPU implementation of the path, timed on the host cores."""
    import numpy as np
    from oracle import oracle
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle.build()
    cores = oracle.num_threads()
    rows = max(cores, 64)
    rng = np.random.default_rng(42)
    sample = rng.random((rows, N_COLS), dtype=np.float32)
    kind = "port"
    times = []

    def select():
        t0 = time.perf_counter()
        oracle.select_heap(sample, args.k)
        times.append(time.perf_counter() - t0)

    try:
        # the reference's own parallel_knn::selection (OpenMP heap), compiled from its sources;
        # it reports the time of selection() alone, as the reference's main loop measures it
        from oracle import ref_select
        if ref_select.available():
            ref_select.select("parallel", sample[:cores], args.k)
            kind = "reference"

            def select():
                times.append(ref_select.select("parallel", sample, args.k)[2])
    except Exception:
        kind = "port"
    for _ in range(max(args.warmup, 1)):
        select()
    times.clear()
    for _ in range(args.steps):
        select()
    dt = sum(times) / len(times)
    value = rows * N_COLS / dt
    sample_text = (f"each step = {rows} of {Q} rows x {N_COLS} columns, Uniform[0,1) seed 42, k={args.k}, "
                   f"OpenMP heap selection on {cores} threads "
                   f"({'the reference parallel_knn::selection compiled from its sources' if kind == 'reference' else 'CPU port of parallel_knn::selection'})")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"k-selection q={Q} n=2^20 uniform k={args.k} (bounded sample per step)",
                       "q": Q, "n": N_COLS, "k": args.k},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample_text},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--k", type=int, default=256)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the k / input-order sweep")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--rows", type=int, default=Q, help="rows of the matrix (smaller = profiling case)")
    ap.add_argument("--profile-case", default=None, choices=["fused_tc", "fused_tc_small", "l2_tc", "fused_fp32", "l2_fp32"],
                    help="run a few launches of one small case of that kernel and exit (for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.profile_case is not None:
        run_profile_case(args.profile_case)
        return

    import torch
    import __graft_entry__ as entry
    bk = entry.load_package()
    bk.lib()  # fails loudly when the CUDA library is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if args.gpus == 1 and world == 1:
            pass
        else:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist_pg = None
    if world > 1:
        import torch.distributed as dist_pg_mod
        dist_pg_mod.init_process_group("nccl", device_id=dev)
        dist_pg = dist_pg_mod

    q, n, k = args.rows, N_COLS, args.k
    gen = torch.Generator(device=dev).manual_seed(42 + rank)
    matrix = torch.rand((q, n), generator=gen, device=dev, dtype=torch.float32)
    offsets = torch.full((q,), rank * n, dtype=torch.int32, device=dev)  # global column index of the shard
    if world > 1:
        fin_d = torch.empty((q, k), dtype=torch.float32, device=dev)
        fin_i = torch.empty((q, k), dtype=torch.int32, device=dev)

    launches_per_step = 1 if world == 1 else 2
    from importlib import import_module
    search = import_module(entry.PKG_NAME + ".sharded").ShardedSearch(bk, rank, world)

    out_d, out_i = search.local_views(q, k, dev)  # the local candidates live in the exchange buffer

    def step(src=matrix):
        # local selection with global labels, then (N > 1) ONE NCCL all-gather + merge kernel
        search.select(src, k, rank * n, offsets=offsets, out=None if world == 1 else (fin_d, fin_i))

    def stream_step(events=None):
        # the same search as one of a stream of searches: with N > 1 its all-gather stays in flight
        # while the next local selection runs (two buffer sets), and the previous search is merged
        search.submit_select(matrix, k, rank * n, offsets=offsets, out=None if world == 1 else (fin_d, fin_i),
                             events=events)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist_pg.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist_pg.all_reduce(t, op=dist_pg.ReduceOp.MAX)
        return float(t.item())

    # ---- resident-input throughput (`value`) and the kernel time for the roofline ----------
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_first_sample()
    for _ in range(args.warmup):
        stream_step()
    search.drain()
    barrier()
    # keep the GPU under the same load a little longer so that the clock sampler (20 ms period)
    # sees the clocks this workload settles at; still untimed
    # (a fixed count, identical on every rank: each step holds collectives when N > 1)
    for _ in range(300):
        stream_step()
    search.drain()
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 2)]
    barrier()
    ev[-2].record()
    for s in range(args.steps):
        stream_step(events=(ev[2 * s], ev[2 * s + 1]))
    search.drain()  # the K-th search is complete inside the timed region too
    ev[-1].record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    bk.device_status()
    total_ms = max_over_ranks(ev[-2].elapsed_time(ev[-1]))
    kernel_ms = statistics.mean(ev[2 * s].elapsed_time(ev[2 * s + 1]) for s in range(args.steps))
    ms_per_step = total_ms / args.steps
    value = q * n * world / (ms_per_step * 1e-3)

    peak_gbs, peak_kind = measured_peaks()
    algo_bytes = 4.0 * q * n + 8.0 * q * k
    achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "select_kernel", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                "frac": achieved / peak_gbs, "peak_source": f"{peak_kind} (copy bandwidth, burst)",
                "algorithmic_bytes_per_launch": algo_bytes, "kernel_ms": kernel_ms,
                "traffic": None}
    # DRAM traffic of the same kernel from one ncu capture of a 592-row case (one full wave), per
    # row; traffic is proportional to the rows, so a full launch is rows x that.
    roofline["traffic"] = NCU_DRAM_BYTES_PER_ROW * q
    roofline["traffic_source"] = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of select_kernel<256,1>, "
                                  "592 x 2^20 capture, scaled by rows")

    # ---- sweep: other k, and the adversarial descending rows (kernel time only) -------------
    sweep = None
    desc_host = None
    if not args.no_sweep and world == 1:
        sweep = {}
        desc = None
        for order in ("uniform", "descending"):
            src = matrix
            if order == "descending":
                desc = torch.sort(matrix, dim=1, descending=True).values
                src = desc
            for kk in (16, 64, 256, 1024, 2048):
                od = torch.empty((q, kk), dtype=torch.float32, device=dev)
                oi = torch.empty((q, kk), dtype=torch.int32, device=dev)
                reps = 5 if order == "uniform" else 2
                for _ in range(2 if order == "uniform" else 1):
                    bk.select(src, kk, out=(od, oi))
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    bk.select(src, kk, out=(od, oi))
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / reps
                sweep[f"{order}_k{kk}"] = {"ms": ms, "distances_per_s": q * n / (ms * 1e-3),
                                           "frac_of_hbm_peak": (4.0 * q * n + 8.0 * q * kk) / (ms * 1e-3) / 1e9 / peak_gbs}
            del src
        # kept on the host for the same-box run of the reference's kernel on the adversarial rows
        desc_host = desc.cpu().numpy() if (desc is not None and not args.no_cpu and not args.no_e2e) else None
        del desc
        torch.cuda.empty_cache()
        # ablation: the same kernel without its radius filter (the reference's partial-bitonic-regs):
        # what the buffer + filter buy on uniform rows
        bk.set_tuning("select.filter", 0)
        try:
            od = torch.empty((q, 32), dtype=torch.float32, device=dev)
            oi = torch.empty((q, 32), dtype=torch.int32, device=dev)
            bk.select(matrix, 32, out=(od, oi))
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            bk.select(matrix, 32, out=(od, oi))
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            sweep["uniform_k32_without_filter"] = {"ms": ms, "distances_per_s": q * n / (ms * 1e-3),
                                                   "frac_of_hbm_peak": (4.0 * q * n + 8.0 * q * 32) / (ms * 1e-3) / 1e9 / peak_gbs}
        finally:
            bk.set_tuning("select.filter", 1)

    # ---- end to end through the C ABI from host buffers (`e2e`) ----------------------------
    e2e = None
    e2e_knn = None
    host = None
    if not args.no_e2e:
        host = torch.empty((q, n), dtype=torch.float32).pin_memory()
        host.copy_(matrix)
        host_d = torch.empty((q, k), dtype=torch.float32).pin_memory()
        host_i = torch.empty((q, k), dtype=torch.int32).pin_memory()
        staging = torch.empty_like(matrix)
        res_d, res_i = (out_d, out_i) if world == 1 else (fin_d, fin_i)

        def e2e_step():
            staging.copy_(host, non_blocking=True)
            step(staging)
            host_d.copy_(res_d, non_blocking=True)
            host_i.copy_(res_i, non_blocking=True)

        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
        e2e = {"value": q * n * world / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "steps": e2e_steps,
               "h2d_bytes_per_step": 4 * q * n, "d2h_bytes_per_step": 8 * q * k,
               "what": "pinned host distance matrix -> device, selection, result -> host (PCIe-bound: the matrix "
                       "is 4 GiB per step)"}

        # The flow of the reference's `knn` binary (prepare / distances / selection / finish,
        # src/main.cpp): the VECTORS come from the host every step, the distance matrix is made on
        # the device (exact FP32 kernel) and never crosses PCIe.
        e2e_dim = 32
        hp = torch.rand((n, e2e_dim), dtype=torch.float32).pin_memory()
        hq = torch.rand((q, e2e_dim), dtype=torch.float32).pin_memory()
        dp = torch.empty((n, e2e_dim), dtype=torch.float32, device=dev)
        dq = torch.empty((q, e2e_dim), dtype=torch.float32, device=dev)

        # the points travel in four pieces on a copy stream; the distance kernel of a piece (its
        # columns of the matrix) starts as soon as the piece is on the device
        pieces = 4
        bounds = [(i * n // pieces, (i + 1) * n // pieces) for i in range(pieces)]
        copy_stream = torch.cuda.Stream(device=dev)
        arrived = [torch.cuda.Event() for _ in range(pieces)]
        consumed = torch.cuda.Event()

        def knn_step():
            main = torch.cuda.current_stream()
            copy_stream.wait_event(consumed)       # the previous step no longer reads dp / dq
            with torch.cuda.stream(copy_stream):
                dq.copy_(hq, non_blocking=True)
                for i, (b, e) in enumerate(bounds):
                    dp[b:e].copy_(hp[b:e], non_blocking=True)
                    arrived[i].record(copy_stream)
            for i, (b, e) in enumerate(bounds):
                main.wait_event(arrived[i])
                bk.l2(dp[b:e], dq, mode=bk.L2_EXACT, out=staging[:, b:e])
            consumed.record(main)
            step(staging)
            host_d.copy_(res_d, non_blocking=True)
            host_i.copy_(res_i, non_blocking=True)

        consumed.record(torch.cuda.current_stream())

        for _ in range(2):
            knn_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            knn_step()
        e1.record()
        barrier()
        knn_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
        e2e_knn = {"value": q * n * world / (knn_ms * 1e-3), "unit": UNIT, "ms_per_step": knn_ms, "steps": e2e_steps,
                   "h2d_bytes_per_step": 4 * e2e_dim * (n + q), "d2h_bytes_per_step": 8 * q * k, "dim": e2e_dim,
                   "what": "pinned host points and queries -> device (four pieces on a copy stream, the distance "
                           "kernel of a piece starts when it has arrived), exact FP32 distance matrix on the device, "
                           "selection, result -> host: the reference's own end-to-end flow"}
        del staging, dp, dq, hp, hq

    # ---- same-box comparator: the reference's own `bits-prefetch` kernel, recompiled ---------
    reference_gpu = None
    if rank == 0 and world == 1 and not args.no_cpu and host is not None:
        try:
            from oracle import ref_select
            if ref_select.available():
                host_np = host.numpy()
                ref_sel = {}
                for kk in sorted({32, k, 2048}):
                    _, _, sec = ref_select.select("bits-prefetch", host_np, kk, block_size=256, batch=13, repeats=3)
                    ref_sel[f"k{kk}"] = {"ms": sec * 1e3, "distances_per_s": q * n / sec}
                reference_gpu = {"what": "the reference's bits-prefetch kernel compiled from its sources for sm_100a "
                                         "(block 256, batch 13: its tuned H100 shape), same matrix, host-timed "
                                         "selection() like its main loop, fastest of 3",
                                 "uniform": ref_sel}
                if desc_host is not None:
                    _, _, sec = ref_select.select("bits-prefetch", desc_host, k, block_size=256, batch=13, repeats=2)
                    reference_gpu["descending"] = {f"k{k}": {"ms": sec * 1e3, "distances_per_s": q * n / sec}}
                    desc_host = None
        except Exception as err:  # the comparator is optional
            reference_gpu = {"unavailable": str(err)}

    knn = None
    if rank == 0 and world == 1 and not args.no_sweep:
        del matrix
        torch.cuda.empty_cache()
        knn = knn_section(bk, dev)

    # ---- database-sharded fused k-NN: 2^24 points of dim 64 per GPU, 16384 queries, k = 128 ----
    knn_sharded = None
    if not args.no_sweep:
        if "matrix" in dir():
            del matrix
        torch.cuda.empty_cache()
        knn_sharded = sharded_knn_section(bk, search, dev, rank, world, barrier, max_over_ranks)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        if host is None:
            gen2 = torch.Generator(device=dev).manual_seed(42)
            host = torch.rand((64, n), generator=gen2, device=dev, dtype=torch.float32).cpu()
        cpu = cpu_selection_baseline(host.numpy(), k)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": (value / world / PUBLISHED_H100[k]) if (k in PUBLISHED_H100 and q == Q) else None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"k-selection sweep shape: q={q} x n=2^20 float32 Uniform[0,1) per GPU, k={k}",
                           "q": q, "n": n, "k": k, "sharding": "database columns" if world > 1 else "none",
                           "l2_policy": "input (4 GiB per GPU) is larger than L2; no flush needed"},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "e2e_knn": e2e_knn,
                "gpu_launches": launches_per_step * args.steps, "clocks": clocks}
        if sweep is not None:
            line["sweep"] = sweep
        if reference_gpu is not None:
            line["reference_gpu"] = reference_gpu
        if knn is not None:
            line["knn"] = knn
        if knn_sharded is not None:
            line["knn_sharded"] = knn_sharded
        print(json.dumps(line), flush=True)
    if world > 1:
        dist_pg.destroy_process_group()


if __name__ == "__main__":
    main()
