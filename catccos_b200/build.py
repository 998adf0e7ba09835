"""In-tree build of libcatccos_b200.so with nvcc for sm_100a (no JIT cache, no pip install)."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcatccos_b200.so")
DRIVER = os.path.join(HERE, "catccos_run")
SOURCES = ["symm_heap.cu", "dense_ops.cu", "c_api.cu", "no_alloc.cu", "mx_quant.cu", "mx_ops.cu", "moe_aux.cu", "moe_ops.cu", "mxq_allgather.cu", "fp4_gemm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def _newer(a, b):
    return (not os.path.exists(b)) or os.path.getmtime(a) > os.path.getmtime(b)


def build(force=False, verbose=False):
    """Compiles every .cu under csrc/ and links the shared library next to this file."""
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "catccos_b200.h"))
    newest_header = max(os.path.getmtime(h) for h in headers)
    objs, procs = [], []
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(s, o) or newest_header > os.path.getmtime(o):
            cmd = [nvcc] + NVCC_FLAGS + ["-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed for {src}:\n{out}\n")
        elif verbose:
            print(out)
    if failed:
        raise RuntimeError("CUDA build failed")
    if force or procs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-cudart", "static", "-Xcompiler", "-fPIC", "-lpthread", "-ldl", "-lrt"]
        subprocess.check_call(cmd)
    build_driver(force)
    return LIB


def build_driver(force=False):
    """The C++ host driver (operator registry, file I/O, launch map) on top of the shared library."""
    src = os.path.join(CSRC, "host", "catccos_run.cpp")
    inc = os.path.join(os.path.dirname(HERE), "include")
    deps = [src, LIB] + [os.path.join(inc, "catccos_host", f) for f in os.listdir(os.path.join(inc, "catccos_host"))]
    deps.append(os.path.join(inc, "catccos_b200.h"))
    if force or not os.path.exists(DRIVER) or any(os.path.getmtime(d) > os.path.getmtime(DRIVER) for d in deps):
        cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-I", inc, "-I", os.path.join(cuda, "include"), src, "-o", DRIVER,
                               "-L", HERE, "-lcatccos_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart",
                               "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda, "lib64")])
    return DRIVER


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
