"""ctypes binding of libq27b200.so: `lib()` loads it, `call(name, *args)` invokes a C-ABI entry point with torch
tensors passed by device pointer and raises on a non-zero return code (the protocol of the reference's
engine/python/q27lib.py:120-149). There is no fallback: if the library is missing or was not built, loading raises.
"""

import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
LIB_PATH = os.environ.get("Q27B200_LIB", os.path.join(HERE, "libq27b200.so"))

P, I, I64, F, SZ = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t
U32P = ctypes.POINTER(ctypes.c_uint32)

# name -> (argument types, result type); mirrors include/q27b200/capi.h line by line
SIGNATURES = {
    "q27_last_error": ([], ctypes.c_char_p),
    "q27b_sf_bytes": ([I64, I64], I64),
    "q27b_sf_offset": ([I64, I64, I64], I64),
    "q27b_glu_row": ([I64, I], I64),
    "q27b_swizzle_sf": ([P, I, I, P, I, P], I),
    "q27b_copy_glu": ([P, SZ, P, SZ, SZ, I, P], I),
    "q27b_ckpt_open": ([ctypes.c_char_p, ctypes.POINTER(P)], I),
    "q27b_ckpt_close": ([P], None),
    "q27b_ckpt_count": ([P], I),
    "q27b_ckpt_tensor": ([P, ctypes.c_char_p, ctypes.c_char_p, I, ctypes.POINTER(I64), I, ctypes.POINTER(I), ctypes.POINTER(I64)], I),
    "q27b_ckpt_read": ([P, ctypes.c_char_p, I64, I64, P], I),
    "q27b_ckpt_fp4_layer": ([P, ctypes.c_char_p, P], I),
    "q27b_ckpt_load_fp4": ([P, ctypes.c_char_p, I, P, P, P, SZ, P], I),
    "q27b_quant_fp4": ([P, I, I, F, P, P, P], I),
    "q27b_quant_fp4_bf16": ([P, I, I, F, P, P, P], I),
    "q27b_quant_fp4_batch": ([P, P, I, P], I),
    "q27b_rmsnorm_quant_fp4": ([P, P, I, I, F, P, F, P, P, P, I, P, P], I),
    "q27b_trace_set": ([P], I),
    "q27b_probe_wait_timeout": ([I, P], I),
    "q27b_quant_fp4_weight": ([P, I, I, F, P, P, P], I),
    "q27b_quant_fp4_dynamic": ([P, I, I, P, P, P, P], I),
    "q27b_quant_fp4_dynamic_bf16": ([P, I, I, P, P, P, P], I),
    "q27b_skinny_fp4_scaled": ([I, I, I, P, P, P, P, P, P, P, P, SZ, P], I),
    "q27b_silu_mul_quant_fp4": ([P, P, I64, I, I, F, P, P, P], I),
    "q27b_silu_mul_quant_fp4_bf16": ([P, P, I64, I, I, F, P, P, P], I),
    "q27b_silu_mul_quant_fp4_glu": ([P, I, I, F, F, F, P, P, P], I),
    "q27b_silu_mul_quant_fp4_glu_bf16": ([P, I, I, F, F, F, P, P, P], I),
    "q27b_skinny_fp4": ([I, I, I, P, P, P, P, I, P, P, P, F, P, P, SZ, P], I),
    "q27b_skinny_fp4_bf16": ([I, I, I, P, P, P, P, I, P, P, P, P, SZ, P], I),
    "q27b_skinny_fp4_glu_bf16": ([I, I, I, P, P, P, P, F, F, P, P, SZ, P], I),
    "q27b_skinny_fp4_static": ([I, I, I, P, P, P, P, I, P, P, P, F, P, P], I),
    "q27b_skinny_workspace_bytes": ([I, I, I], I64),
    "q27b_skinny_group_build": ([I, I, P, I, P, SZ, P, P], I),
    "q27b_skinny_fp4_group": ([P, P, P, SZ, P], I),
    "q27t_skinny_fp4_group": ([P, P, P, SZ], I),
    "q27b_skinny_fp4_group_gather": ([P, P, P, SZ, P, P], I),
    "q27b_group_gather_wait": ([P, I, P, P], I),
    "q27b_gemm_fp4_glu_bf16_gather": ([I, I, I, P, P, P, P, F, F, P, P, P], I),
    "q27b_gemm_fp4": ([I, I, I, P, P, P, P, F, P, F, P, P], I),
    "q27b_gemm_fp4_bf16": ([I, I, I, P, P, P, P, F, P, P], I),
    "q27b_gemm_fp4_glu_bf16": ([I, I, I, P, P, P, P, F, F, P, P], I),
    "q27b_gemm_fp4_glu": ([I, I, I, P, P, P, P, F, F, F, P, P, P], I),
    "q27b_device_status": ([U32P], I),
    "q27b_quad_available": ([], I),
    "q27t_last_us": ([], F),
    "q27t_sf_bytes": ([I64, I64], I64),
    "q27t_quant_fp4": ([P, I, I, F, P, P], I),
    "q27t_quant_fp4_bf16": ([P, I, I, F, P, P], I),
    "q27t_rmsnorm_quant": ([P, P, I, F, P, I, F, P, P], I),
    "q27t_quant_fp4_weight": ([P, I, I, F, P, P], I),
    "q27t_quant_fp4_dynamic": ([P, I, I, P, P, P], I),
    "q27t_skinny_fp4_scaled": ([I, I, I, P, P, P, P, P, P, P, P, SZ], I),
    "q27t_silu_mul_quant_fp4": ([P, P, I64, I, I, F, P, P], I),
    "q27t_silu_mul_quant_fp4_bf16": ([P, P, I64, I, I, F, P, P], I),
    "q27t_silu_mul_quant_fp4_glu": ([P, I, I, F, F, F, P, P], I),
    "q27t_silu_mul_quant_fp4_glu_bf16": ([P, I, I, F, F, F, P, P], I),
    "q27t_swizzle_sf": ([P, I, I, P], I),
    "q27t_swizzle_sf_glu": ([P, I, I, P, I], I),
    "q27t_gemm_fp4": ([I, I, I, P, P, P, P, F, P, F, P], I),
    "q27t_gemm_fp4_bf16": ([I, I, I, P, P, P, P, F, P], I),
    "q27t_gemm_fp4_glu_bf16": ([I, I, I, P, P, P, P, F, F, P], I),
    "q27t_gemm_fp4_glu": ([I, I, I, P, P, P, P, F, F, F, P, P], I),
    "q27t_skinny_fp4": ([I, I, I, P, P, P, P, F, P, F, P, P, SZ], I),
    "q27t_skinny_fp4_segments": ([I, I, I, P, P, P, P, I, P, P, P, F, P, P, SZ], I),
    "q27t_skinny_fp4_bf16": ([I, I, I, P, P, P, P, F, P, P, SZ], I),
    "q27t_skinny_fp4_glu_bf16": ([I, I, I, P, P, P, P, F, F, P, P, SZ], I),
    "q27t_skinny_fp4_static": ([I, I, I, P, P, P, P, F, P, F, P], I),
    "q27t_bench_gemm": ([I, I, I, I, P, P, P, P, I64, I64, I, I, P, P, SZ, P], I),
}

# the test-scaffolding library (include/q27b200/testing.h); only the test suite loads it
TEST_LIB_PATH = os.path.join(HERE, "libq27b200_test.so")
TEST_SIGNATURES = {
    "q27b_skinny_plan": ([I, I, I, I, P, I, P, P, P], I),
    "q27b_skinny_tile_parts": ([I, I, I, I, P, I], I),
    "q27b_skinny_group_plan": ([I, P, P, I, I, I, P, I, P, P, P], I),
    "q27t_ref_gemm_fp4": ([I, I, I, P, P, P, P, F, P], I),
    "q27t_cxx_launchers": ([P, I, I, F, P, P, I, P, P, I, P, P, P, P, SZ, I, P, P, F, F, F, P, P], I),
    "q27t_cxx_throws": ([], I),
}

_lib = None
_test_lib = None


def build(verbose: bool = False) -> str:
    """Compiles the CUDA sources for sm_100a into libq27b200.so (nvcc cross-compiles without a GPU)."""
    r = subprocess.run(["make", "-C", CSRC, "-j8"], capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode:
        raise RuntimeError("building libq27b200.so failed")
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `make -C {CSRC}` (there is no fallback path)")
        _lib = ctypes.CDLL(LIB_PATH)
        for name, (args, res) in SIGNATURES.items():
            fn = getattr(_lib, name)  # a missing symbol is an error: the header and the library must agree
            fn.argtypes, fn.restype = args, res
    return _lib


def scaffold_lib():
    """The scaffolding library of the test suite; it resolves its references to the product library, loaded first."""
    global _test_lib
    if _test_lib is None:
        lib()
        if not os.path.exists(TEST_LIB_PATH):
            raise RuntimeError(f"{TEST_LIB_PATH} is missing: build it with `make -C {CSRC}`")
        _test_lib = ctypes.CDLL(TEST_LIB_PATH)
        for name, (args, res) in TEST_SIGNATURES.items():
            fn = getattr(_test_lib, name)
            fn.argtypes, fn.restype = args, res
    return _test_lib


def _arg(x):
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes") and hasattr(x, "dtype"):  # numpy array (host-side arguments)
        return x.ctypes.data
    return x


def last_error() -> str:
    return lib().q27_last_error().decode()


def call(name, *args):
    """Calls an entry point that returns a status; raises RuntimeError with the library's message on failure."""
    rc = getattr(scaffold_lib() if name in TEST_SIGNATURES else lib(), name)(*map(_arg, args))
    if rc != 0:
        raise RuntimeError(f"{name}: {last_error()}")


def device_status() -> int:
    s = ctypes.c_uint32()
    call("q27b_device_status", ctypes.byref(s))
    return s.value
