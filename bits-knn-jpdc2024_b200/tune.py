"""Regenerates csrc/tuning_table.inc: the launch shapes the library picks per problem shape.

    python bits-knn-jpdc2024_b200/tune.py [--quick] [--dry-run]

Runs on the GPU the library will be used on (a few minutes; --quick: fewer repetitions).  For
every bucket of k and of row-slice count it times the `bits` selection over candidate shapes
(block size x pairs per thread x stage ring x fold threshold) on seeded Uniform[0,1) rows and on
per-row descending rows, and keeps, among the shapes within 2 % of the best uniform time, the one
with the best descending time; for the FP32 fused search it times both kernels per (dim, k) at
q = 2^14, n = 2^20.  The table is compiled into the library: rebuild it afterwards (build.py).

Role of the reference's parameter sweeps and tables (scripts/run-parameters.sh ->
scripts/optima.csv, looked up by `config_algorithm` in scripts/config.sh:98-214).
"""
import argparse
import importlib.util
import itertools
import pathlib
import sys

PKG = pathlib.Path(__file__).resolve().parent
ROOT = PKG.parent
TABLE = PKG / "csrc" / "tuning_table.inc"
KNOBS = ("select.threads", "select.ipt", "select.stage_bytes", "select.stages", "select.merge_at", "select.unroll")


def load_package():
    spec = importlib.util.spec_from_file_location("bits_knn_jpdc2024_b200", PKG / "__init__.py",
                                                  submodule_search_locations=[str(PKG)])
    module = importlib.util.module_from_spec(spec)
    sys.modules["bits_knn_jpdc2024_b200"] = module
    spec.loader.exec_module(module)
    return module


def time_ms(fn, reps):
    import torch
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def select_candidates(k):
    """(threads, ipt, stage_bytes, stages, merge_pct, unroll) worth trying for a list of k pairs."""
    shapes = [(t, i) for t, i in ((256, 1), (256, 2), (256, 4), (512, 1), (512, 2), (512, 4), (1024, 1), (1024, 2))
              if t * i >= k and t * i <= max(256, 2 * k)]
    out = []
    for (t, i) in shapes:
        for stage_bytes, stages in ((16384, 3), (16384, 4), (32768, 2), (32768, 3), (65536, 2)):
            if stage_bytes < 16 * t:            # a stage is at least one 4-vector per thread
                continue
            smem = stage_bytes * stages + 2 * t * i * 8 + 512
            blocks = max(1, 1024 // t)
            if smem * blocks > 226 * 1024:      # keep the block count the register budget allows
                continue
            # (lists of 1024 pairs and more are folded by selection, which takes the whole buffer: later folds)
            for merge_pct in ((50, 75) if t * i <= 256 else ((75, 100) if t * i < 1024 else (100, 140))):
                out.append((t, i, stage_bytes, stages, merge_pct, 2))
    return out


def tune_select(bk, quick):
    import torch
    rows = []
    n = 1 << 20
    gen = torch.Generator(device="cuda").manual_seed(42)
    matrix = torch.rand((1024, n), generator=gen, device="cuda")
    descending = torch.sort(matrix[:296], dim=1, descending=True).values.contiguous()
    for k in (64, 256, 512, 1024, 2048):
        for rows_max, q in ((296, 148), (1 << 62, 1024)):
            src = matrix[:q]
            out = (torch.empty((q, k), device="cuda"), torch.empty((q, k), dtype=torch.int32, device="cuda"))
            out_d = (torch.empty((296, k), device="cuda"), torch.empty((296, k), dtype=torch.int32, device="cuda"))
            measured = []
            for cand in select_candidates(k):
                for key, value in zip(KNOBS, cand):
                    bk.set_tuning(key, value)
                try:
                    uni = time_ms(lambda: bk.select(src, k, out=out), 2 if quick else 5)
                    desc = time_ms(lambda: bk.select(descending, k, out=out_d), 1 if quick else 2)
                except bk.BitsKnnError:
                    continue
                measured.append((uni, desc, cand))
            bk.device_status()
            best_uni = min(m[0] for m in measured)
            uni, desc, cand = min((m for m in measured if m[0] <= 1.02 * best_uni), key=lambda m: m[1])
            print(f"select k<={k} rows<={rows_max if rows_max < 1 << 40 else 'any'}: {cand} uniform {uni:.3f} ms, "
                  f"descending(296 rows) {desc:.3f} ms", flush=True)
            rows.append((k, rows_max, cand))
    for key in KNOBS:
        bk.set_tuning(key, 0)
    return rows


def tune_splits(bk, quick):
    """Row slices per launch the automatic split should aim at (few long rows), per k bucket."""
    import torch
    gen = torch.Generator(device="cuda").manual_seed(7)
    matrix = torch.rand((8, 1 << 24), generator=gen, device="cuda")
    wanted = {}
    for k in (64, 256, 1024, 2048):
        out = (torch.empty((8, k), device="cuda"), torch.empty((8, k), dtype=torch.int32, device="cuda"))
        best = None
        for splits in (8, 16, 24, 32, 48, 64):
            if splits * k > 65536:
                continue
            ws = torch.empty(bk.select_split_workspace_bytes(8, k, splits), dtype=torch.uint8, device="cuda")
            ms = time_ms(lambda: bk.select_split(matrix, k, splits=splits, workspace=ws, out=out), 2 if quick else 4)
            if best is None or ms < best[0]:
                best = (ms, splits)
        wanted[k] = 8 * best[1]
        print(f"splits k<={k}: {best[1]} slices per row for 8 rows ({best[0]:.3f} ms) -> {wanted[k]} blocks", flush=True)
    return wanted


def tune_fused(bk, quick):
    import torch
    rows = []
    n, q = 1 << 20, 1 << 14
    gen = torch.Generator(device="cuda").manual_seed(3)
    for dim in (4, 8, 12, 16, 24):
        points = torch.rand((n, dim), generator=gen, device="cuda")
        queries = torch.rand((q, dim), generator=gen, device="cuda")
        for k in (16, 64, 128, 256):
            out = (torch.empty((q, k), device="cuda"), torch.empty((q, k), dtype=torch.int32, device="cuda"))
            ws = torch.empty(max(bk.fused_workspace_bytes(n, q, dim, k, bk.L2_PARTIAL), 256), dtype=torch.uint8, device="cuda")
            times = []
            for variant in (0, 1):
                bk.set_tuning("fused.variant", variant)
                times.append(time_ms(lambda: bk.fused(points, queries, k, mode=bk.L2_PARTIAL, out=out, workspace=ws), 1))
            bk.set_tuning("fused.variant", 2)
            rows.append((dim, k, 1 if times[1] <= times[0] else 0))
            print(f"fused dim<={dim} k<={k}: 8-query {times[0]:.2f} ms, tiled {times[1]:.2f} ms", flush=True)
    rows.append((320, 256, 1))  # beyond the sweep the tiled kernel always won
    return rows


def write_table(select_rows, wanted, fused_rows, device_name):
    lines = [f"// Launch shapes measured on {device_name}; regenerate with bits-knn-jpdc2024_b200/tune.py.",
             "// BITSKNN_SELECT_ROW(k_max, rows_max, threads, ipt, stage_bytes, stages, merge_pct, unroll, blocks_wanted)"]
    for k, rows_max, cand in select_rows:
        blocks = wanted.get(k, wanted.get(64 if k <= 64 else (256 if k <= 256 else (1024 if k <= 1024 else 2048)), 0))
        rows_text = "1LL << 62" if rows_max >= 1 << 40 else str(rows_max)
        lines.append(f"BITSKNN_SELECT_ROW({k}, {rows_text}, {cand[0]}, {cand[1]}, {cand[2]}, {cand[3]}, {cand[4]}, {cand[5]}, {blocks})")
    lines.append("// BITSKNN_FUSED_ROW(dim_max, k_max, tiled)")
    for dim, k, tiled in fused_rows:
        lines.append(f"BITSKNN_FUSED_ROW({dim}, {k}, {tiled})")
    return "\n".join(lines) + "\n"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--dry-run", action="store_true", help="print the table instead of writing it")
    ap.add_argument("--out", default=str(TABLE))
    args = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("tune.py needs the GPU the library will run on")
    torch.cuda.set_device(0)
    bk = load_package()
    bk.lib()
    select_rows = tune_select(bk, args.quick)
    wanted = tune_splits(bk, args.quick)
    fused_rows = tune_fused(bk, args.quick)
    text = write_table(select_rows, wanted, fused_rows, torch.cuda.get_device_name(0))
    if args.dry_run:
        print(text)
    else:
        pathlib.Path(args.out).write_text(text)
        print(f"wrote {args.out}; rebuild the library (bits-knn-jpdc2024_b200/build.py)")


if __name__ == "__main__":
    main()
