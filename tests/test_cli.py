"""The `knn` command line keeps the reference's surface (src/main.cpp:168-269, docs/knn.md)."""
import pathlib
import subprocess

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
KNN = ROOT / "bits-knn-jpdc2024_b200" / "bin" / "knn"
HEADER = ("algorithm,generator,preprocessor,iteration,point_count,query_count,dim,block_size,k,"
          "items_per_thread,deg,phase,time")


@pytest.fixture(scope="module")
def knn(bk):
    if not KNN.exists():
        subprocess.run(["make", "-C", str(KNN.parents[1] / "host")], check=True)
    return KNN


def run(knn, *args):
    return subprocess.run([str(knn), *args], capture_output=True, text=True, timeout=600)


def test_header_and_help(knn):
    r = run(knn, "--header")
    assert r.returncode == 0 and r.stdout.strip() == HEADER
    r = run(knn, "--help")
    assert r.returncode == 0
    for name in ("serial", "parallel", "partial-bitonic-regs", "partial-bitonic-buffered-static", "bits", "bits-prefetch", "bits-sq", "fused-cache", "magma-dist",
                 "magma-part-dist", "bits-sharded"):
        assert f"- {name}\n" in r.stderr
    for flag in ("--algorithm", "--repeat", "--knn", "--number", "--query", "--dimension", "--generator",
                 "--preprocessor", "--seed", "--block-size", "--items-per-thread", "--verify", "--point-layout",
                 "--query-layout", "--deg", "--no-output", "--header"):
        assert flag in r.stderr


@pytest.mark.parametrize("args,message", [
    (["-d", "0"], "Dimension must be greater than 0"),
    (["-n", "0"], "Number of objects in the database must be greater than 0"),
    (["-q", "0"], "Number of query objects must be greater than 0"),
    (["-k", "0"], "Number of nearest neighbors must be greater than 0"),
    (["--block-size", "0"], "Block size must be greater than 0"),
    (["-g", "nope"], "Unknown generator: 'nope'"),
    (["-p", "nope"], "Unknown preprocessor: 'nope'"),
    (["-a", "nope"], "Unknown algorithm: 'nope'"),
])
def test_validation_messages(knn, args, message):
    r = run(knn, *args)
    assert r.returncode == 1 and message in r.stderr


@pytest.mark.gpu
def test_published_checksum_end_to_end(knn, cuda):
    # the reference's published run (scripts/run-kselection.sh): seed 24, uniform, dim 1;
    # n = 2^20, k = 32 printed `Checksum: 16556617` for every algorithm.  q is reduced to 64
    # (queries are drawn after the points, so query 0 is the same).
    r = run(knn, "-a", "bits", "-n", "1M", "-q", "64", "-k", "32", "--seed", "24", "-r", "2",
            "--items-per-thread", "13", "--block-size", "256")
    assert r.returncode == 0, r.stderr
    assert r.stderr.splitlines() == ["Checksum: 16556617"] * 2
    rows = r.stdout.strip().splitlines()
    assert len(rows) == 14
    phases = [row.split(",")[-2] for row in rows[:7]]
    assert phases == ["prepare", "transfer-in", "distances", "selection", "postprocessing", "finish", "transfer-out"]
    assert rows[0].startswith('bits,uniform,identity,0,1048576,64,1,256,32,"13,1,1",1,prepare,')


@pytest.mark.gpu
@pytest.mark.parametrize("args", [
    ["-a", "bits-prefetch", "-n", "64k", "-q", "128", "-k", "100", "-d", "10", "--seed", "7"],
    ["-a", "partial-bitonic-regs", "-n", "64k", "-q", "16", "-k", "32", "--seed", "7"],
    ["-a", "partial-bitonic-buffered-static", "-n", "64k", "-q", "16", "-k", "32", "--seed", "7"],
    ["-a", "partial-bitonic-buffered-static", "-n", "100000", "-q", "4", "-k", "300", "--seed", "24", "-p", "descending"],
    ["-a", "bits-sq", "--deg", "8", "-n", "256k", "-q", "4", "-k", "64", "--seed", "7"],
    ["-a", "bits", "-n", "100000", "-q", "8", "-k", "256", "--seed", "24", "-p", "descending"],
    ["-a", "bits", "-n", "2M", "-q", "4", "-k", "64", "--seed", "7"],          # few long rows: sliced automatically
    ["-a", "bits", "-n", "3000", "-q", "16", "-k", "8", "-d", "6", "--seed", "3", "--point-layout", "column",
     "--query-layout", "column"],
    ["-a", "parallel", "-n", "3000", "-q", "16", "-k", "8", "-d", "6", "--seed", "3"],
    ["-a", "bits", "-n", "4096", "-q", "16", "-k", "8", "-d", "4", "--seed", "3", "-g", "clustered:16,0.05"],
])
def test_verify_against_serial(knn, cuda, args):
    r = run(knn, *args, "--verify", "serial")
    assert r.returncode == 0, r.stderr
    assert "Difference" not in r.stderr
    assert r.stderr.count("Checksum:") == 1


@pytest.mark.gpu
@pytest.mark.parametrize("args", [
    ["-n", "20000", "-q", "100", "-k", "32", "-d", "8", "--seed", "7", "--items-per-thread", "8,4,2",
     "--block-size", "4", "--deg", "2"],
    ["-n", "5000", "-q", "33", "-k", "16", "-d", "37", "--seed", "9", "-g", "normal:0,2"],
])
def test_fused_labels_equal_serial_labels(knn, cuda, args):
    # the fused kernel reports partial distances (no query norm), like the reference's, so the
    # tolerant --verify (relative distance test) does not apply; the labels must still agree,
    # which the checksum of query 0 shows
    sums = []
    for alg in ("fused-cache", "bits-fused", "serial"):
        r = run(knn, "-a", alg, *args)
        assert r.returncode == 0, r.stderr
        sums.append(r.stderr.strip())
    assert sums[0] == sums[1] == sums[2] and sums[0].startswith("Checksum: ")


@pytest.mark.gpu
def test_expired_device_wait_makes_the_next_phase_throw(knn, cuda):
    # host/selftest.cpp: for several registry entries, selection() after the library's diagnostic
    # kernel gave up its bounded wait must throw, and the next selection() gives the old result
    exe = KNN.parent / "host_selftest"
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().splitlines()[-1] == "ok", r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("alg", ["bits-sharded", "bits-sharded-bf16"])
def test_sharded_id_verifies_against_serial(knn, cuda, alg):
    # uses every visible GPU (one on a single-GPU box: the same code path without the exchange)
    r = run(knn, "-a", alg, "-n", "100000", "-q", "64", "-k", "32", "-d", "8", "--seed", "11", "--verify", "serial")
    assert r.returncode == 0, r.stderr
    assert "Difference" not in r.stderr
    assert r.stderr.count("Checksum:") == 1


@pytest.mark.gpu
def test_unsupported_k_message(knn, cuda):
    r = run(knn, "-a", "bits", "-n", "8192", "-q", "4", "-k", "4096")
    assert r.returncode == 1 and "Unsupported k value: 4096" in r.stderr
    r = run(knn, "-a", "magma-part-dist", "-n", "4096", "-q", "64", "-d", "16", "--seed", "1", "--no-output")
    assert r.returncode == 0 and "distances" in r.stdout
