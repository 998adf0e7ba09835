"""The C++ host layer (operator registry, operator classes, launch map, driver binary)."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def driver():
    from catccos_b200 import build as b
    b.build()
    return b.DRIVER


def test_registry_lists_every_operator_on_the_path(driver):
    out = subprocess.run([driver, "--list"], capture_output=True, text=True, check=True).stdout.split()
    assert set(out) == {"MatmulAllReduce", "AllGatherMatmul", "MatmulReduceScatter", "Ascend950AllGatherMatmul",
                        "Ascend950MatmulReduceScatter", "Ascend950Fp8MxAllGatherMatmul", "Ascend950DispatchFFNCombine",
                        "Ascend950MxFp8MatmulReduceScatter", "MxQuantAllGather",
                        "Ascend950Fp8MxAllToAllVGroupedMatmul", "Ascend950Fp8MxGroupedMatmulAllToAllV",
                        "AllGatherMatmulWithGatherResult", "AllGatherMatmulRemoteRead", "Ascend950Fp4MxAllGatherMatmul", "Ascend950AllToAllMatmul", "Ascend950MatmulAllToAll", "Ascend950MxFp8MatmulAllToAll", "Ascend950Fp4MxMatmulReduceScatter",
                        "Ascend950Fp4MxAllToAllVGroupedMatmul", "Ascend950Fp4MxGroupedMatmulAllToAllV"}


def test_argument_and_init_errors_return_nonzero(driver, tmp_path):
    assert subprocess.run([driver], capture_output=True).returncode == 1
    assert subprocess.run([driver, "nope", "27", "1", "0", "tcp://127.0.0.1:1", "8", "8", "8", str(tmp_path)],
                          capture_output=True).returncode == 1
    if not torch.cuda.is_available():
        r = subprocess.run([driver, "mmar", "1", "1", "0", "tcp://127.0.0.1:1", "128", "256", "64", str(tmp_path)],
                           capture_output=True, text=True)
        assert r.returncode != 0 and "shmem init failed" in r.stderr


@pytest.mark.gpu
def test_single_rank_mx_quant_allgather_driver_run(driver, tmp_path):
    """`mxqtag` through the host path with the reference's file names
    (examples/ascend950_mx_quant_allgather/mx_quant_allgather_host.h:48-74): codes and scales byte for byte."""
    from oracle import mxquant
    m, n = 200, 1024
    x = (torch.randn((m, n), generator=torch.Generator().manual_seed(3)) * 2).to(torch.bfloat16)
    x.view(torch.uint16).numpy().tofile(os.path.join(tmp_path, "rank_0_input.bin"))
    r = subprocess.run([driver, "mxqtag", "36", "1", "0", "tcp://127.0.0.1:8789", str(m), str(n), "1", str(tmp_path),
                        "0", "0", "1", "0", "0", "1", "1"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    codes, scales, _ = mxquant.quantize_mx_e4m3(x.to(torch.float32).numpy(), "rne")
    assert np.array_equal(np.fromfile(os.path.join(tmp_path, "rank_0_output.bin"), dtype=np.uint8).reshape(m, n), codes)
    assert np.array_equal(np.fromfile(os.path.join(tmp_path, "rank_0_mxscale.bin"), dtype=np.uint8).reshape(m, -1), scales)


def _write_dense_files(tmp_path, world, a, b, trans_b=False):
    for r in range(world):
        av = a[r].view(torch.uint16) if a[r].dtype == torch.bfloat16 else a[r]
        bm = b[r].t().contiguous() if trans_b else b[r]
        bv = bm.view(torch.uint16) if bm.dtype == torch.bfloat16 else bm
        av.numpy().tofile(os.path.join(tmp_path, f"rank_{r}_a.bin"))
        bv.numpy().tofile(os.path.join(tmp_path, f"rank_{r}_b.bin"))


@pytest.mark.gpu
@pytest.mark.parametrize("kernel,dtype", [("mmar", torch.float16), ("agmm", torch.bfloat16), ("mmrs", torch.bfloat16)])
def test_single_rank_driver_run(driver, tmp_path, kernel, dtype):
    """rank_size 1 through the whole host path: files -> operator class -> launch map -> result file -> verifier."""
    from oracle import dense, inputs, verify
    m, n, k = 384, 520, 256
    a, b = inputs.allgather_matmul_inputs(1, m, k, n, dtype)
    _write_dense_files(str(tmp_path), 1, a, b)
    code = "1" if dtype == torch.float16 else "27"
    r = subprocess.run([driver, kernel, code, "1", "0", "tcp://127.0.0.1:8788", str(m), str(n), str(k), str(tmp_path),
                        "0", "0", "1", "0", "0", "2", "3"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    name = "output_0.bin" if kernel == "agmm" else "output.bin"
    raw = np.fromfile(os.path.join(tmp_path, name), dtype=np.uint16 if dtype == torch.bfloat16 else np.float16)
    out = torch.from_numpy(raw.reshape(m, n))
    out = out.view(torch.bfloat16) if dtype == torch.bfloat16 else out
    gold = dense.matmul_fp32(a[0], b[0])
    ok, precision, eb = verify.reference_check(out, gold, k)
    assert ok, (precision, eb)


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", ["agmmwg", "agmmrr", "a5atamm", "a5mmata"])
def test_single_rank_driver_run_of_the_data_flow_variants(driver, tmp_path, kernel):
    """The variants' operator classes through the driver at rank_size 1 (every one is then the plain product); the
    gather-result operator also writes the gathered A, which must be the input bit for bit."""
    from oracle import dense, inputs, verify
    m, n, k = 384, 520, 256
    a, b = inputs.allgather_matmul_inputs(1, m, k, n, torch.bfloat16)
    _write_dense_files(str(tmp_path), 1, a, b)
    r = subprocess.run([driver, kernel, "27", "1", "0", "tcp://127.0.0.1:8788", str(m), str(n), str(k), str(tmp_path),
                        "0", "0", "1", "0", "0", "2", "3"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = np.fromfile(os.path.join(tmp_path, "output_0.bin"), dtype=np.uint16)
    out = torch.from_numpy(raw.reshape(m, n)).view(torch.bfloat16)
    ok, precision, eb = verify.reference_check(out, dense.matmul_fp32(a[0], b[0]), k)
    assert ok, (precision, eb)
    if kernel == "agmmwg":
        got = np.fromfile(os.path.join(tmp_path, "output_gather_a.bin"), dtype=np.uint16).reshape(m, k)
        assert np.array_equal(got, a[0].view(torch.uint16).numpy())


@pytest.mark.gpu
def test_two_rank_driver_run(driver, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from oracle import dense, inputs, verify
    world, m, n, k = 2, 256, 512, 256
    a, b = inputs.allgather_matmul_inputs(world, m, k, n, torch.bfloat16)
    _write_dense_files(str(tmp_path), world, a, b)
    port = f"tcp://127.0.0.1:{24000 + os.getpid() % 1000}"
    procs = [subprocess.Popen([driver, "agmm", "27", "2", str(r), port, str(m), str(n), str(k), str(tmp_path)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    for p in procs:
        out, _ = p.communicate(timeout=300)
        assert p.returncode == 0, out
    gold = dense.golden_allgather_matmul(a, b)
    for r in range(world):
        raw = np.fromfile(os.path.join(tmp_path, f"output_{r}.bin"), dtype=np.uint16).reshape(world * m, n)
        ok, precision, eb = verify.reference_check(torch.from_numpy(raw).view(torch.bfloat16), gold[r], k)
        assert ok, (r, precision, eb)


def _check(driver, *args):
    r = subprocess.run([driver, "--check", *[str(a) for a in args]], capture_output=True, text=True)
    return r.returncode, r.stdout.split()


@pytest.mark.parametrize("args", [
    ("mmar", 2, 512, 2048, 1024),                      # benchmark configuration 1
    ("agmm", 8, 1024, 4096, 8192),                     # 2
    ("mmrs", 8, 8192, 8192, 2048),                     # 3
    ("a5fp8mxagmm", 8, 2048, 4096, 7168),              # 4
    ("a5moe", 8, 4096, 4096, 7168, 8, 256),            # 5 (n = 2 x intermediate)
    ("a5mxfp8mmrs", 8, 8192, 8192, 2048),
    ("a5agmm", 1, 8, 8, 8),
    ("agmmwg", 8, 1024, 4096, 8192),                   # data-flow variants and further operators on configuration-sized shapes
    ("agmmrr", 8, 1024, 4096, 8192),
    ("a5atamm", 8, 8192, 4096, 8192),
    ("a5mmata", 8, 8192, 8192, 2048),
    ("a5mxfp8mmata", 8, 8192, 8192, 2048),
    ("a5fp4mxagmm", 8, 2048, 4096, 7168),
    ("a5fp4mmrs", 8, 8192, 8192, 2048),
    ("mxqtag", 8, 2048, 7168, 0),
    ("a5fp8mxatavgmm", 8, 4096, 4096, 7168, 1, 256),
    ("a5fp8gmmata", 8, 4096, 7168, 2048, 1, 256),
    ("a5fp4mxatavgmm", 8, 4096, 4096, 7168, 1, 256),
    ("a5fp4gmmata", 8, 4096, 7168, 2048, 1, 256),
])
def test_operator_classes_accept_the_benchmark_configurations(driver, args):
    """CheckCocTilingParams of every operator class, and the buffers fit the reference's 1004 MiB symmetric buffer."""
    rc, out = _check(driver, *args)
    assert rc == 0 and out[0] == "ok", out
    assert int(out[1]) <= 1004 * 1024 * 1024


@pytest.mark.parametrize("args", [
    ("mmrs", 8, 8190, 8192, 2048),                     # rows not divisible by the ranks
    ("agmm", 8, 1024, 4100, 8192),                     # n not a multiple of 8 (16-byte rows)
    ("agmm", 8, 65536, 4096, 8192),                    # gathered A would not fit the symmetric buffer
    ("a5fp8mxagmm", 8, 2048, 4096, 7170),              # k not a multiple of the 32-element scale block
    ("a5mxfp8mmrs", 2, 192, 256, 128),                 # rows per rank not a multiple of 128
    ("a5moe", 8, 4096, 4096, 7000, 8, 256),            # k % 256, as the reference operator demands
    ("a5moe", 8, 4096, 4096, 7168, 8, 250),            # experts not divisible by the ranks
    ("mmar", 0, 512, 2048, 1024),                      # no ranks
    ("a5atamm", 8, 8190, 4096, 8192),                  # rows not divisible by the ranks
    ("a5mmata", 8, 8190, 8192, 2048),
    ("a5fp4mxagmm", 8, 2048, 4096, 7200),              # k not a multiple of 64
    ("a5fp8mxatavgmm", 8, 4096, 4096, 7168, 1, 250),   # experts not divisible by the ranks
])
def test_operator_classes_reject_unusable_tilings(driver, args):
    rc, out = _check(driver, *args)
    assert rc == 2 and out == ["rejected"], out


def test_check_mode_reports_unknown_kernels(driver):
    rc, _ = _check(driver, "nope", 2, 8, 8, 8)
    assert rc == 1
