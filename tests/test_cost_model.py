"""The B200 cost model of the host layer (include/catccos_host/cost_model.h; counterpart of the
reference's tests/dynamic_tiling cost model), through `catccos_run --estimate`.  No device needed."""
import subprocess

import pytest


@pytest.fixture(scope="module")
def driver():
    from catccos_b200 import build as b
    b.build()
    return b.DRIVER


def _estimate(driver, *args):
    r = subprocess.run([driver, "--estimate", *[str(a) for a in args]], capture_output=True, text=True)
    out = r.stdout.split()
    if r.returncode != 0:
        return r.returncode, out
    return 0, dict(m0=int(out[0]), block_num=int(out[1]), cost=float(out[2]), compute=float(out[3]), comm=float(out[4]))


# kernel, ranks, m, n, k, measured microseconds per launch (max over ranks, sustained clocks; the MXFP8
# rows are the GEMM launch without the activation quantiser that the benchmark step also times)
MEASURED = [
    ("agmm", 1, 8192, 4096, 8192, 461), ("agmm", 2, 4096, 4096, 8192, 491), ("agmm", 4, 2048, 4096, 8192, 544),
    ("agmm", 8, 1024, 4096, 8192, 594), ("mmrs", 1, 8192, 8192, 2048, 222), ("mmrs", 4, 8192, 8192, 2048, 329),
    ("mmrs", 8, 8192, 8192, 2048, 357), ("mmar", 2, 512, 2048, 1024, 55), ("a5fp8mxagmm", 1, 16384, 4096, 7168, 440),
    ("a5fp8mxagmm", 8, 2048, 4096, 7168, 540),
]


@pytest.mark.parametrize("kernel,ranks,m,n,k,measured_us", MEASURED)
def test_model_is_within_15_percent_of_the_measured_launch_times(driver, kernel, ranks, m, n, k, measured_us):
    rc, e = _estimate(driver, kernel, ranks, m, n, k)
    assert rc == 0
    assert abs(e["cost"] - measured_us) <= 0.15 * measured_us, e


def test_selection_prefers_pairs_for_large_and_single_ctas_for_tiny_problems(driver):
    _, big = _estimate(driver, "agmm", 8, 1024, 4096, 8192)
    assert big["m0"] == 256 and big["block_num"] == 148
    _, tiny = _estimate(driver, "mmar", 2, 512, 2048, 1024)       # 32 tiles of 128 x 256: one wave either way
    assert tiny["m0"] == 128
    _, mx = _estimate(driver, "a5fp8mxagmm", 8, 2048, 4096, 7168)
    assert mx["m0"] == 256                                         # the MXFP8 operators exist as pair kernels only


def test_model_scales_like_a_roofline(driver):
    _, a = _estimate(driver, "agmm", 1, 8192, 4096, 4096, 256, 148)
    _, b = _estimate(driver, "agmm", 1, 8192, 4096, 8192, 256, 148)
    assert 1.9 < b["compute"] / a["compute"] < 2.05                # twice the K, twice the main loop
    _, half = _estimate(driver, "agmm", 1, 8192, 4096, 8192, 256, 74)
    assert half["compute"] > 1.9 * b["compute"]                    # half the SMs
    costs = [_estimate(driver, "agmm", r, 8192 // r, 4096, 8192)[1]["cost"] for r in (1, 2, 4, 8)]
    assert costs == sorted(costs)                                  # same work per GPU, more peers: never cheaper
    _, rs = _estimate(driver, "mmrs", 8, 8192, 8192, 2048)
    assert abs(rs["comm"] - 7 / 8 * 8192 * 8192 * 2 / 770e3) < 0.5  # bytes over the measured peer bandwidth
    # wave quantisation: 75 pair tiles on 74 pairs cost two waves
    _, w1 = _estimate(driver, "agmm", 1, 256 * 74, 256, 4096, 256, 148)
    _, w2 = _estimate(driver, "agmm", 1, 256 * 75, 256, 4096, 256, 148)
    assert w2["compute"] > 1.8 * w1["compute"]


def test_unsupported_and_invalid_requests(driver):
    assert _estimate(driver, "a5moe", 8, 4096, 4096, 7168) == (2, ["unsupported"])
    assert _estimate(driver, "nope", 8, 4096, 4096, 7168) == (2, ["unsupported"])
    assert _estimate(driver, "agmm", 0, 4096, 4096, 7168) == (2, ["invalid"])
    assert _estimate(driver, "agmm", 2, 4096, 4096, 7168, 192, 148) == (2, ["invalid"])      # no such tile


def test_tiling_candidates_csv(driver, tmp_path):
    """GetTilings / CreateTilingFile / WriteTilingInfos of include/catccos_host/tiling.h (the reference's
    tests/dynamic_tiling/include/tiling.h): candidates the operator accepts, one CSV row each."""
    path = tmp_path / "tilings.csv"
    r = subprocess.run([driver, "--tilings", "agmm", "8", "1024", "4096", "8192", str(path)], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.split() == ["6"]
    rows = path.read_text().strip().splitlines()
    assert rows[0] == "Op,M,K,N,Transpose A,Transpose B,M0,N0,K0,blockNum,Model(us),Time(us)"
    body = [x.split(",") for x in rows[1:]]
    assert len(body) == 6 and all(b[0] == "AllGatherMatmul" and b[1:4] == ["1024", "8192", "4096"] for b in body)
    assert {(b[6], b[9]) for b in body} == {("128", "148"), ("128", "74"), ("128", "37"), ("256", "148"), ("256", "74"), ("256", "36")}
    best = min(body, key=lambda b: float(b[10]))
    assert (best[6], best[9]) == ("256", "148") and all(b[11] == "" for b in body)      # the measured column is left open
    # the MXFP8 operator has pair kernels only; a shape the operator rejects yields no candidates
    r = subprocess.run([driver, "--tilings", "a5fp8mxagmm", "8", "2048", "4096", "7168", str(path)], capture_output=True, text=True)
    assert r.stdout.split() == ["3"]
    r = subprocess.run([driver, "--tilings", "mmrs", "8", "8190", "8192", "2048", str(path)], capture_output=True, text=True)
    assert r.stdout.split() == ["0"]
