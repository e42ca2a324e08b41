"""Extracts the published known-answer checksums of the reference's selection runs.

Reads the stderr capture the reference ships for `scripts/run-kselection.sh`
(`data/kselection-hopper01-108424.err`) and writes `kselection_checksums.json` beside this
script.  Run it where the reference checkout is available:

    python tests/golden/make_kselection_golden.py /path/to/reference

How the capture is decoded.  The run script (scripts/run-kselection.sh:58-113) loops over
q = 2^6, 2^8, 2^10, 2^12 with n = 2^30 / q and k = 2^5 .. 2^11, and for each (q, k) starts
the `knn` binary ten times (algorithms bits, bits-prefetch, air-topk, grid-select, warpsort,
radik, warp-select, block-select, block-select-tunable, warp-select-tunable), every time
with `-r 20 --seed 24 -g uniform -p identity` and the default dimension 1
(src/main.cpp:180-181).  Each successful start prints 20 lines `Checksum: <uint32>`
(src/main.cpp:410-417: the sum of the k indices of query 0); a start that throws prints an
`exception occurred!` block or a `cudaError...` / `CUDA error.` block instead.  So the capture is a sequence of invocations, ten per
configuration, in loop order.
"""
import json
import pathlib
import os
import sys

ALGORITHMS = ["bits", "bits-prefetch", "air-topk", "grid-select", "warpsort", "radik",
              "warp-select", "block-select", "block-select-tunable", "warp-select-tunable"]


def invocations(lines):
    """Yield one list of checksums per `knn` start (empty list for a failed start)."""
    current = []
    in_exception = False
    for line in lines:
        line = line.rstrip("\n")
        if line.startswith("Checksum: "):
            in_exception = False
            current.append(int(line.split()[1]))
            if len(current) == 20:
                yield current
                current = []
        elif line.startswith("exception occurred!") or "cudaError" in line:
            # two kinds of failed start appear in the capture: a RAFT exception with a
            # stack trace, and the reference's own CUDA error report (three lines)
            assert not current, "failure in the middle of a run"
            in_exception = True
            yield []
        else:
            assert in_exception or line == "", f"unexpected line: {line!r}"


def main():
    ref = pathlib.Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BITSKNN_REFERENCE_DIR", str(pathlib.Path(__file__).resolve().parents[3] / "reference")))
    src = ref / "data" / "kselection-hopper01-108424.err"
    runs = list(invocations(src.read_text().splitlines()))
    configs = [(2 ** qp, 2 ** (30 - qp), 2 ** kp) for qp in (6, 8, 10, 12) for kp in range(5, 12)]
    assert len(runs) == len(configs) * len(ALGORITHMS), (len(runs), len(configs))
    out = []
    for ci, (q, n, k) in enumerate(configs):
        per_alg = {}
        for ai, alg in enumerate(ALGORITHMS):
            per_alg[alg] = sorted(set(runs[ci * len(ALGORITHMS) + ai]))
        every = sorted({v for vals in per_alg.values() for v in vals})
        out.append({"seed": 24, "generator": "uniform", "preprocessor": "identity", "dim": 1,
                    "q": q, "n": n, "k": k, "unanimous": len(every) == 1,
                    "bits": per_alg["bits"], "bits-prefetch": per_alg["bits-prefetch"],
                    "all": every})
    dst = pathlib.Path(__file__).with_name("kselection_checksums.json")
    dst.write_text(json.dumps({"source": "data/kselection-hopper01-108424.err",
                               "configs": out}, indent=1) + "\n")
    print(f"wrote {dst} ({len(out)} configurations, "
          f"{sum(c['unanimous'] for c in out)} unanimous)")


if __name__ == "__main__":
    main()
