"""ctypes binding of the CPU oracle (oracle/libnvfp4_oracle.so) and, when present, of the
reference bridge (oracle/_ref/libref_fp4.so).  TEST INFRASTRUCTURE ONLY: imported by
tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs, never by the library.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(_HERE, "libnvfp4_oracle.so")
REF_LIB = os.path.join(_HERE, "_ref", "libref_fp4.so")
REF_DENSE_LIB = os.path.join(_HERE, "_ref", "libref_dense.so")

AUTO, GEMV, GEMM = 0, 1, 2

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

_lib = None


def build():
    subprocess.run(["make", "-C", _HERE, "oracle"], check=True, stdout=subprocess.DEVNULL)


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_LIB):
            build()
        lib = ctypes.CDLL(ORACLE_LIB)
        lib.nvfp4_oracle_e2m1.restype = c_float
        lib.nvfp4_oracle_e2m1.argtypes = [ctypes.c_uint]
        lib.nvfp4_oracle_ue4m3.restype = c_float
        lib.nvfp4_oracle_ue4m3.argtypes = [ctypes.c_uint8]
        lib.nvfp4_oracle_f2bf.restype = ctypes.c_uint16
        lib.nvfp4_oracle_f2bf.argtypes = [c_float]
        lib.nvfp4_oracle_bf2f.restype = c_float
        lib.nvfp4_oracle_bf2f.argtypes = [ctypes.c_uint16]
        lib.nvfp4_oracle_f2e4m3.restype = ctypes.c_uint8
        lib.nvfp4_oracle_f2e4m3.argtypes = [c_float]
        lib.nvfp4_oracle_dequant_bf16.restype = None
        lib.nvfp4_oracle_dequant_bf16.argtypes = [_u8p, _u8p, c_float, c_int, c_int, _u16p]
        lib.nvfp4_oracle_linear_mt.restype = None
        lib.nvfp4_oracle_linear_mt.argtypes = [_u16p, c_int, _u8p, _u8p, c_float, c_int, c_int, c_void_p, _u16p,
                                               c_int, c_int]
        lib.nvfp4_oracle_linear_rows.restype = None
        lib.nvfp4_oracle_linear_rows.argtypes = [_u16p, c_int, _u8p, _u8p, c_float, c_int, c_int, c_void_p, _u16p,
                                                 c_int, c_int, c_int]
        lib.nvfp4_oracle_swiglu.restype = None
        lib.nvfp4_oracle_swiglu.argtypes = [_u16p, _u16p, ctypes.c_size_t, _u16p]
        lib.nvfp4_oracle_swiglu_merged.restype = None
        lib.nvfp4_oracle_swiglu_merged.argtypes = [_u16p, c_int, c_int, _u16p]
        lib.nvfp4_oracle_dense_linear.restype = None
        lib.nvfp4_oracle_dense_linear.argtypes = [_u16p, c_int, _u16p, c_int, c_int, c_void_p, _u16p]
        lib.nvfp4_oracle_dense_gemv_ref.restype = None
        lib.nvfp4_oracle_dense_gemv_ref.argtypes = [_u16p, _u16p, c_int, c_int, c_void_p, _u16p]
        lib.nvfp4_oracle_rmsnorm.restype = None
        lib.nvfp4_oracle_rmsnorm.argtypes = [_u16p, c_void_p, _u16p, c_float, c_int, c_int, _u16p, c_void_p]
        lib.nvfp4_oracle_mlp.restype = None
        lib.nvfp4_oracle_mlp.argtypes = [_u16p, c_int, c_int, c_int, _u8p, _u8p, c_float, _u8p, _u8p, c_float,
                                         c_void_p, _u16p, c_int, c_int]
        lib.nvfp4_oracle_tp_mlp.restype = None
        lib.nvfp4_oracle_tp_mlp.argtypes = [_u16p, c_int, c_int, c_int, c_int, _u8p, _u8p, c_float, _u8p, _u8p,
                                            c_float, c_void_p, _u16p, c_int, c_int, c_int]
        lib.nvfp4_oracle_rel_frobenius.restype = ctypes.c_double
        lib.nvfp4_oracle_rel_frobenius.argtypes = [_u16p, _u16p, ctypes.c_size_t]
        _lib = lib
    return _lib


def _res_ptr(residual):
    if residual is None:
        return None
    assert residual.dtype == np.uint16 and residual.flags["C_CONTIGUOUS"]
    return residual.ctypes.data


def dequant(packed, scale, gs):
    N, K = packed.shape[0], packed.shape[1] * 2
    out = np.empty((N, K), np.uint16)
    load().nvfp4_oracle_dequant_bf16(packed, scale, gs, N, K, out)
    return out


def linear(A, packed, scale, gs, residual=None, mode=AUTO, threads=1):
    """A: uint16 [M,K] BF16 bits; returns uint16 [M,N]."""
    M, K = A.shape
    N = packed.shape[0]
    assert packed.shape[1] * 2 == K and scale.shape == (N, K // 16)
    C = np.empty((M, N), np.uint16)
    load().nvfp4_oracle_linear_mt(A, M, packed, scale, gs, N, K, _res_ptr(residual), C, mode, threads)
    return C


def linear_rows(A, packed, scale, gs, n0, n1, residual=None, mode=AUTO):
    """Rows [n0,n1) only; the returned [M,N] array is valid in those columns."""
    M, K = A.shape
    N = packed.shape[0]
    C = np.zeros((M, N), np.uint16)
    load().nvfp4_oracle_linear_rows(A, M, packed, scale, gs, N, K, _res_ptr(residual), C, mode, n0, n1)
    return C


def swiglu(gate, up):
    out = np.empty_like(gate)
    load().nvfp4_oracle_swiglu(gate.reshape(-1), up.reshape(-1), gate.size, out.reshape(-1))
    return out


def swiglu_merged(merged):
    T, I2 = merged.shape
    out = np.empty((T, I2 // 2), np.uint16)
    load().nvfp4_oracle_swiglu_merged(merged, T, I2 // 2, out)
    return out


def dense_linear(A, W, residual=None):
    """A [M,K], W [N,K]: uint16 BF16 bits; returns uint16 [M,N]."""
    M, K = A.shape
    N = W.shape[0]
    assert W.shape[1] == K
    C = np.empty((M, N), np.uint16)
    load().nvfp4_oracle_dense_linear(np.ascontiguousarray(A), M, np.ascontiguousarray(W), N, K, _res_ptr(residual), C)
    return C


def dense_gemv_ref(A, W, residual=None):
    """One token (A [1,K] or [K]) through the reference's BF16 GEMV summation order; returns uint16 [1,N]."""
    A = np.ascontiguousarray(A).reshape(-1)
    N, K = W.shape
    assert A.shape[0] == K
    C = np.empty((1, N), np.uint16)
    res = None if residual is None else np.ascontiguousarray(residual).reshape(-1)
    load().nvfp4_oracle_dense_gemv_ref(A, np.ascontiguousarray(W), N, K, _res_ptr(res), C.reshape(-1))
    return C


def rmsnorm(x, weight, eps, bias=None):
    """x, bias: uint16 [M,K] BF16 bits; weight [K].  Returns the normalised rows; with `bias`
    (x + bias normalised) also the updated residual."""
    M, K = x.shape
    out = np.empty((M, K), np.uint16)
    if bias is None:
        load().nvfp4_oracle_rmsnorm(np.ascontiguousarray(x), None, np.ascontiguousarray(weight), eps, M, K, out, None)
        return out
    bias = np.ascontiguousarray(bias)
    res = np.empty((M, K), np.uint16)
    load().nvfp4_oracle_rmsnorm(np.ascontiguousarray(x), bias.ctypes.data, np.ascontiguousarray(weight), eps, M, K, out,
                                res.ctypes.data)
    return out, res


def mlp(X, gu_packed, gu_scale, gu_gs, dn_packed, dn_scale, dn_gs, residual=None, mode=AUTO, threads=1):
    M, H = X.shape
    I = dn_packed.shape[1] * 2
    out = np.empty((M, H), np.uint16)
    load().nvfp4_oracle_mlp(X, M, H, I, gu_packed, gu_scale, gu_gs, dn_packed, dn_scale, dn_gs,
                            _res_ptr(residual), out, mode, threads)
    return out


def tp_mlp(X, P, gu_packed, gu_scale, gu_gs, dn_packed, dn_scale, dn_gs, residual=None, mode=AUTO,
           partial_bf16=True, threads=1):
    M, H = X.shape
    I = dn_packed.shape[1] * 2
    out = np.empty((M, H), np.uint16)
    load().nvfp4_oracle_tp_mlp(X, M, H, I, P, gu_packed, gu_scale, gu_gs, dn_packed, dn_scale, dn_gs,
                               _res_ptr(residual), out, mode, int(partial_bf16), threads)
    return out


def rel_frobenius(a, b):
    a = np.ascontiguousarray(a).reshape(-1)
    b = np.ascontiguousarray(b).reshape(-1)
    return load().nvfp4_oracle_rel_frobenius(a, b, a.size)


def bf16_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x):
    """Round-to-nearest-even FP32 -> BF16 bits (numpy)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = u + 0x7FFF + ((u >> 16) & 1)
    return (r >> 16).astype(np.uint16)


def encode_e4m3(x):
    """float -> unsigned E4M3 byte, round to nearest even, subnormals kept, saturating at 448:
    the numpy twin of nvfp4_oracle_f2e4m3 (tests check the two against each other)."""
    a = np.abs(np.ascontiguousarray(x, np.float32))
    sub = np.rint(a * np.float32(512.0))                      # 2^-9 grid below 2^-6; 8 is the first normal
    m, e = np.frexp(a)                                         # a = m * 2^e, m in [0.5, 1)
    q = np.rint(m * np.float32(16.0))
    carry = q == 16.0
    q = np.where(carry, 8.0, q)
    e = e + carry
    code = ((e - 1 + 7).astype(np.int64) << 3) | (q.astype(np.int64) - 8)
    code = np.where(a < np.float32(0.015625), sub.astype(np.int64), code)
    code = np.where((a >= 448.0) | (code > 0x7E) | np.isnan(a), 0x7E, code)
    return code.astype(np.uint8)


def encode_e4m3_scalar(x):
    """The same through the oracle's C encoder, element by element (small arrays only)."""
    lib = load()
    flat = np.ascontiguousarray(x, np.float32).reshape(-1)
    return np.fromiter((lib.nvfp4_oracle_f2e4m3(float(v)) for v in flat), np.uint8, flat.size).reshape(np.shape(x))


def ref_available():
    return os.path.exists(REF_LIB)


def ref_dense_available():
    return os.path.exists(REF_LIB) and os.path.exists(REF_DENSE_LIB)


_ref = None


def load_ref():
    """The reference engine's own kernels (device pointers, needs a GPU)."""
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(REF_LIB)
        vp = c_void_p
        lib.ref_fp4_gemv.argtypes = [vp, vp, vp, c_float, c_int, c_int, vp, vp]
        lib.ref_fp4_gemv_add.argtypes = [vp, vp, vp, c_float, c_int, c_int, vp, vp, vp]
        lib.ref_fp4_dual_gemv.argtypes = [vp, vp, vp, c_float, vp, vp, c_float, c_int, c_int, vp, vp, vp]
        lib.ref_fp4_gemm.argtypes = [vp, vp, vp, c_float, c_int, c_int, vp, c_int, vp]
        lib.ref_fp4_gemm_add.argtypes = [vp, vp, vp, c_float, c_int, c_int, vp, vp, c_int, vp]
        lib.ref_swiglu.argtypes = [vp, vp, vp, c_int, c_int, vp]
        lib.ref_swiglu_merged.argtypes = [vp, vp, c_int, c_int, vp]
        for n in ("ref_fp4_gemv", "ref_fp4_gemv_add", "ref_fp4_dual_gemv", "ref_fp4_gemm", "ref_fp4_gemm_add",
                  "ref_swiglu", "ref_swiglu_merged"):
            getattr(lib, n).restype = None
        if os.path.exists(REF_DENSE_LIB):
            dl = ctypes.CDLL(REF_DENSE_LIB)
            dl.ref_dense_gemv.argtypes = [vp, vp, vp, c_int, c_int, vp]
            dl.ref_dense_gemv_add.argtypes = [vp, vp, vp, vp, c_int, c_int, vp]
            dl.ref_dense_gemv.restype = dl.ref_dense_gemv_add.restype = None
            lib.dense = dl
        if hasattr(lib, "ref_rmsnorm"):
            lib.ref_rmsnorm.argtypes = [vp, vp, vp, c_float, c_int, c_int, vp]
            lib.ref_fused_add_rmsnorm.argtypes = [vp, vp, vp, vp, c_float, c_int, c_int, vp]
            lib.ref_rmsnorm.restype = lib.ref_fused_add_rmsnorm.restype = None
        _ref = lib
    return _ref
