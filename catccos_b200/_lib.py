"""ctypes binding of libcatccos_b200.so (the C-ABI in include/catccos_b200.h).

There is no CPU or PyTorch fallback: if the shared library has not been built the import fails
with the build command to run.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcatccos_b200.so")


class CatccosError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"catccos error {code}: {message}")
        self.code = code


class CocTilingParams(ctypes.Structure):
    """utils/info.h:95-114 of the reference: 17 uint32 fields in the same order."""
    _fields_ = [(n, ctypes.c_uint32) for n in (
        "m", "k", "n", "transA", "transB", "m0", "k0", "n0", "commTileM", "commInterval", "commNpuSplit",
        "commDataSplit", "commBlockM", "rankSize", "epSize", "expertNum", "topK")]


class KernelParams(ctypes.Structure):
    """utils/info.h:123-167 of the reference (KernelParams) as a plain struct."""
    _fields_ = [("ptrA", ctypes.c_void_p), ("ptrB", ctypes.c_void_p), ("ptrC", ctypes.c_void_p),
                ("customPtrs", ctypes.POINTER(ctypes.c_void_p)), ("customCount", ctypes.c_uint32)]


LAUNCH_ARGS = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.POINTER(KernelParams), ctypes.c_void_p,
               ctypes.c_void_p, ctypes.POINTER(CocTilingParams), ctypes.c_uint32, ctypes.c_uint32]

# name -> (restype, argtypes); every symbol include/catccos_b200.h declares
SIGNATURES = {
    "catccos_shmem_init": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64, ctypes.c_char_p]),
    "catccos_shmem_init_emulated": (ctypes.c_int, [ctypes.c_int32, ctypes.c_uint64]),
    "catccos_shmem_finalize": (ctypes.c_int, []),
    "catccos_shmem_malloc": (ctypes.c_void_p, [ctypes.c_size_t]),
    "catccos_shmem_free": (None, [ctypes.c_void_p]),
    "catccos_shmem_ptr": (ctypes.c_void_p, [ctypes.c_void_p, ctypes.c_int32]),
    "catccos_shmem_get_host": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_size_t]),
    "catccos_shmem_put_host": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t]),
    "catccos_shmem_my_pe": (ctypes.c_int32, []),
    "catccos_shmem_n_pes": (ctypes.c_int32, []),
    "catccos_shmem_barrier_all": (ctypes.c_int, []),
    "catccos_last_error": (ctypes.c_char_p, []),
    "catccos_last_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int32)]),
    "catccos_reset_status": (ctypes.c_int, []),
    "catccos_debug_wait_unset_flag": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint32]),
    "catccos_debug_set_flags": (ctypes.c_int, [ctypes.c_uint32]),
    "catccos_debug_set_trace": (ctypes.c_int, [ctypes.c_void_p]),
    "catccos_debug_rs_tile_order": (ctypes.c_int, [ctypes.c_int32] * 5 + [ctypes.POINTER(ctypes.c_int32), ctypes.c_int32,
                                                                        ctypes.POINTER(ctypes.c_int32)]),
    "catccos_debug_ag_group_rows": (ctypes.c_int, [ctypes.c_int64, ctypes.c_int32, ctypes.c_int64]),
    "catccos_debug_ag_tile_order": (ctypes.c_int, [ctypes.c_int32] * 5 + [ctypes.POINTER(ctypes.c_int32), ctypes.c_int32]),
    "catccos_debug_ag_push_order": (ctypes.c_int, [ctypes.c_int32] * 3 + [ctypes.POINTER(ctypes.c_int32), ctypes.c_int32]),
    "catccos_fp4_gemm_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32]),
    "catccos_fp4_gemm": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_uint32,
                                        ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32]),
    "catccos_debug_slot_sequence": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint8), ctypes.c_int32,
                                                   ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
    "catccos_symmetric_bytes": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(CocTilingParams)]),
    "catccos_workspace_bytes": (ctypes.c_size_t, [ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(CocTilingParams)]),
    "catccos_launch": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32] + LAUNCH_ARGS),
    "catccos_launch_emulated": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_uint32,
                                               ctypes.POINTER(KernelParams), ctypes.POINTER(ctypes.c_void_p),
                                               ctypes.c_void_p, ctypes.POINTER(CocTilingParams), ctypes.c_uint32,
                                               ctypes.c_uint32]),
    "catccos_run_host": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_uint32, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                        ctypes.c_uint32, ctypes.POINTER(CocTilingParams), ctypes.c_uint32,
                                        ctypes.c_uint32]),
    "catccos_run_host_resident": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_uint32, ctypes.c_void_p,
                                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                                 ctypes.c_uint32, ctypes.POINTER(CocTilingParams), ctypes.c_uint32,
                                                 ctypes.c_uint32, ctypes.c_uint32]),
    "catccos_debug_moe_stage_ms": (ctypes.c_int, [ctypes.POINTER(ctypes.c_float), ctypes.c_int32]),
    "catccos_mx_quant": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32]),
    "catccos_sf_atoms_bytes": (ctypes.c_size_t, [ctypes.c_uint32, ctypes.c_uint32]),
    "catccos_gemm_no_alloc": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int32,
                                             ctypes.c_uint32, ctypes.c_uint32]),
    "catccos_gemm_no_alloc_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_uint64),
                                                    ctypes.c_uint32]),
}
for _op in ("MatmulAllReduce", "AllGatherMatmul", "MatmulReduceScatter", "Ascend950AllGatherMatmul",
            "Ascend950MatmulReduceScatter"):
    for _dt in ("FP16", "BF16"):
        SIGNATURES[f"Launch{_op}{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)


for _dt in ("FP16", "BF16"):
    SIGNATURES[f"LaunchAscend950Fp8MxAllGatherMatmul{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950Fp4MxAllGatherMatmul{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950Fp4MxMatmulReduceScatter{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)


for _dt in ("FP16", "BF16"):
    SIGNATURES[f"LaunchAllGatherMatmulWithGatherResult{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAllGatherMatmulRemoteRead{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950AllToAllMatmul{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950MatmulAllToAll{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950MxFp8MatmulAllToAll{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
SIGNATURES["LaunchAscend950DispatchFFNCombineBF16"] = (ctypes.c_int, LAUNCH_ARGS)
SIGNATURES["LaunchAscend950BF16QuantAllGatherFP8E4M3FN"] = (ctypes.c_int, LAUNCH_ARGS)
for _dt in ("FP16", "BF16"):
    SIGNATURES[f"LaunchAscend950Fp8MxAllToAllVGroupedMatmul{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950Fp4MxAllToAllVGroupedMatmul{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950Fp4MxGroupedMatmulAllToAllV{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950Fp8MxGroupedMatmulAllToAllV{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
for _dt in ("FP16", "BF16"):
    SIGNATURES[f"LaunchAscend950MxFp8MatmulReduceScatter{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)
    SIGNATURES[f"LaunchAscend950MxFp8E4M3MatmulReduceScatter{_dt}"] = (ctypes.c_int, LAUNCH_ARGS)


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m catccos_b200.build` (needs nvcc); "
            "there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)     # AttributeError if the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args
    return lib


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = load()
    return _LIB


def check(rc):
    if rc != 0:
        raise CatccosError(rc, lib().catccos_last_error().decode(errors="replace"))
