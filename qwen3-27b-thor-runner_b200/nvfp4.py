"""ctypes binding of libnvfp4_b200.so (the C ABI declared in include/nvfp4_b200.h).

Host-side helper for tests and benchmarks: it adds nothing to the data path -- every
method forwards raw device pointers to the C entry point of the same name.  There is
no CPU fallback: loading fails loudly when the CUDA library has not been built.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libnvfp4_b200.so")

c_void_p, c_int, c_float, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t


class PeerExchange(ctypes.Structure):
    """nvfp4_peer_exchange (include/nvfp4_b200.h)."""
    _fields_ = [("peer", ctypes.c_void_p * 8), ("rank", ctypes.c_int), ("world", ctypes.c_int), ("slot_pairs", ctypes.c_int)]


class LinearDesc(ctypes.Structure):
    """nvfp4_linear_desc (include/nvfp4_b200.h)."""
    _fields_ = [("A", ctypes.c_void_p), ("swiglu_up", ctypes.c_void_p), ("a_row_stride", ctypes.c_longlong),
                ("k_valid", ctypes.c_int), ("M", ctypes.c_int), ("packed", ctypes.c_void_p), ("scale", ctypes.c_void_p),
                ("global_scale", ctypes.c_float), ("N", ctypes.c_int), ("K", ctypes.c_int), ("residual", ctypes.c_void_p),
                ("C", ctypes.c_void_p), ("px", ctypes.c_void_p), ("norm_weight", ctypes.c_void_p),
                ("norm_eps", ctypes.c_float), ("swiglu_epilogue", ctypes.c_int)]


class PeerExchange(ctypes.Structure):
    """nvfp4_peer_exchange of include/nvfp4_b200.h."""
    _fields_ = [("peer", c_void_p * 8), ("rank", c_int), ("world", c_int), ("slot_pairs", c_int)]


class QuantizedWeight(ctypes.Structure):
    """Layout of qwen_thor::core::QuantizedWeight (reference src/engine/layer.h:197-204)."""
    _fields_ = [("packed", c_void_p), ("scale", c_void_p), ("global_scale", c_float),
                ("input_scale", c_float), ("N", c_int), ("K", c_int)]


# name -> (restype, argtypes); every symbol include/nvfp4_b200.h declares.
SIGNATURES = {
    "nvfp4_create": (c_int, [c_int, c_size_t, ctypes.POINTER(c_void_p)]),
    "nvfp4_destroy": (c_int, [c_void_p]),
    "nvfp4_workspace_bytes": (c_int, [c_int, c_int, c_int, ctypes.POINTER(c_size_t)]),
    "nvfp4_status_string": (ctypes.c_char_p, [c_int]),
    "nvfp4_set_option": (c_int, [c_void_p, ctypes.c_char_p, c_int]),
    "nvfp4_get_option": (c_int, [c_void_p, ctypes.c_char_p, ctypes.POINTER(c_int)]),
    "nvfp4_linear": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int,
                             c_void_p, c_void_p, c_void_p]),
    "nvfp4_linear_decode_noalloc": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p,
                                            c_void_p, c_void_p]),
    "nvfp4_noalloc_status": (c_int, [ctypes.POINTER(ctypes.c_uint), c_int]),
    "nvfp4_linear_f32": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p]),
    "nvfp4_linear_reduce_peers": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p,
                                          c_void_p, c_void_p]),
    "nvfp4_linear_ex": (c_int, [c_void_p, c_void_p, c_void_p]),
    "nvfp4_chain_create": (c_int, [c_void_p, c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "nvfp4_chain_run": (c_int, [c_void_p, c_void_p]),
    "nvfp4_chain_destroy": (c_int, [c_void_p]),
    "nvfp4_linear_dual": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p,
                                  c_void_p, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "nvfp4_dequant_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p]),
    "nvfp4_scan_scales": (c_int, [c_void_p, c_void_p, c_int, c_int, ctypes.POINTER(ctypes.c_longlong), c_void_p]),
    "nvfp4_swiglu": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "nvfp4_swiglu_strided": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, ctypes.c_longlong, c_void_p,
                                     ctypes.c_longlong, c_void_p]),
    "nvfp4_linear_bf16": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "nvfp4_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p]),
    "nvfp4_add_rmsnorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_void_p]),
    "nvfp4_swiglu_interleaved": (c_int, [c_void_p, c_void_p, c_int, c_int, ctypes.c_longlong, c_void_p, ctypes.c_longlong,
                                         c_void_p]),
    "nvfp4_invoke_fp4_gemv": (None, [c_void_p, ctypes.POINTER(QuantizedWeight), c_void_p, c_void_p]),
    "nvfp4_invoke_fp4_gemv_add": (None, [c_void_p, ctypes.POINTER(QuantizedWeight), c_void_p, c_void_p,
                                         c_void_p]),
    "nvfp4_invoke_fp4_dual_gemv": (None, [c_void_p, ctypes.POINTER(QuantizedWeight),
                                          ctypes.POINTER(QuantizedWeight), c_void_p, c_void_p, c_void_p]),
    "nvfp4_invoke_fp4_gemm": (None, [c_void_p, ctypes.POINTER(QuantizedWeight), c_void_p, c_int, c_void_p]),
    "nvfp4_invoke_fp4_gemm_add": (None, [c_void_p, ctypes.POINTER(QuantizedWeight), c_void_p, c_void_p, c_int,
                                         c_void_p]),
    "nvfp4_init_fp4_cublaslt": (None, []),
    "nvfp4_cleanup_fp4_cublaslt": (None, []),
    "nvfp4_last_status": (c_int, []),
    "nvfp4_default_handle_workspace": (c_int, [c_size_t]),
    "nvfp4_linear_host": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int,
                                  c_void_p, c_void_p, c_void_p]),
    "nvfp4_launch_count": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_ulonglong)]),
    "nvfp4_device_status": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_uint)]),
}

_lib = None


def load():
    """Load the shared library and attach signatures.  Raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C {_HERE}` "
                "(or __graft_entry__.build()); there is no fallback path")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class Nvfp4Error(RuntimeError):
    def __init__(self, status):
        self.status = status
        super().__init__(f"nvfp4 status {status}: {load().nvfp4_status_string(status).decode()}")


def _ptr(t):
    """Device/host address of a torch tensor, an int, or None."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(stream):
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class Handle:
    """One library handle on one device (nvfp4_create / nvfp4_destroy)."""

    def __init__(self, device=0, workspace_bytes=64 << 20):
        self.lib = load()
        h = c_void_p()
        st = self.lib.nvfp4_create(device, workspace_bytes, ctypes.byref(h))
        if st:
            raise Nvfp4Error(st)
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.lib.nvfp4_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        if st:
            raise Nvfp4Error(st)

    def set_option(self, name, value):
        self._check(self.lib.nvfp4_set_option(self.h, name.encode(), value))

    def get_option(self, name):
        v = c_int()
        self._check(self.lib.nvfp4_get_option(self.h, name.encode(), ctypes.byref(v)))
        return v.value

    def launch_count(self):
        v = ctypes.c_ulonglong()
        self._check(self.lib.nvfp4_launch_count(self.h, ctypes.byref(v)))
        return v.value

    def device_status(self):
        v = ctypes.c_uint()
        self._check(self.lib.nvfp4_device_status(self.h, ctypes.byref(v)))
        return v.value

    def linear_ex(self, A, M, packed, scale, global_scale, N, K, C, residual=None, swiglu_up=None, a_row_stride=0,
                  k_valid=0, px=None, norm_weight=None, norm_eps=0.0, swiglu_epilogue=False, stream=None):
        """nvfp4_linear_ex: the linear layer with SwiGLU (A = gate half, swiglu_up = up half) or
        RMSNorm (norm_weight) formed while staging, a row stride, a zero-padded K, and an
        optional peer exchange."""
        d = LinearDesc(_ptr(A), _ptr(swiglu_up), a_row_stride, k_valid, M, _ptr(packed), _ptr(scale), global_scale, N, K,
                       _ptr(residual), _ptr(C), None if px is None else ctypes.addressof(px), _ptr(norm_weight), norm_eps, int(bool(swiglu_epilogue)))
        self._check(self.lib.nvfp4_linear_ex(self.h, ctypes.byref(d), _stream(stream)))

    def linear_f32(self, A, M, packed, scale, global_scale, N, K, C_f32, stream=None):
        self._check(self.lib.nvfp4_linear_f32(self.h, _ptr(A), M, _ptr(packed), _ptr(scale), global_scale, N, K,
                                              _ptr(C_f32), _stream(stream)))

    def linear_reduce_peers(self, A, M, packed, scale, global_scale, N, K, C, peers, rank, slot_pairs, residual=None,
                            stream=None, check=True):
        """nvfp4_linear_reduce_peers: `peers` = the world's exchange buffers as mapped into this process
        (device tensors or raw pointers), `rank` = this rank's place among them."""
        px = PeerExchange()
        for q, b in enumerate(peers):
            px.peer[q] = _ptr(b)
        px.rank, px.world, px.slot_pairs = rank, len(peers), slot_pairs
        st = self.lib.nvfp4_linear_reduce_peers(self.h, _ptr(A), M, _ptr(packed), _ptr(scale), global_scale, N, K,
                                                _ptr(residual), _ptr(C), ctypes.byref(px), _stream(stream))
        if check:
            self._check(st)
        return st

    def linear(self, A, M, packed, scale, global_scale, N, K, C, residual=None, stream=None, check=True):
        st = self.lib.nvfp4_linear(self.h, _ptr(A), M, _ptr(packed), _ptr(scale), global_scale, N, K,
                                   _ptr(residual), _ptr(C), _stream(stream))
        if check:
            self._check(st)
        return st

    def linear_dual(self, A, M, p1, s1, gs1, p2, s2, gs2, N, K, C1, C2, stream=None):
        self._check(self.lib.nvfp4_linear_dual(self.h, _ptr(A), M, _ptr(p1), _ptr(s1), gs1, _ptr(p2), _ptr(s2),
                                               gs2, N, K, _ptr(C1), _ptr(C2), _stream(stream)))

    def dequant(self, packed, scale, global_scale, N, K, out, stream=None):
        self._check(self.lib.nvfp4_dequant_bf16(self.h, _ptr(packed), _ptr(scale), global_scale, N, K,
                                                _ptr(out), _stream(stream)))

    def scan_scales(self, scale, N, K, stream=None):
        """Block-scale bytes 0x7F / 0xFF in a weight (480 to the reference, NaN to the tensor core); a weight
        that holds any stays off the tensor-core GEMV from here on.  Synchronises."""
        n = ctypes.c_longlong(0)
        self._check(self.lib.nvfp4_scan_scales(self.h, _ptr(scale), N, K, ctypes.byref(n), _stream(stream)))
        return n.value

    def swiglu(self, gate, up, M, I, out, stream=None):
        self._check(self.lib.nvfp4_swiglu(self.h, _ptr(gate), _ptr(up), M, I, _ptr(out), _stream(stream)))

    def swiglu_strided(self, gate, up, M, I, row_stride_in, out, row_stride_out, stream=None):
        self._check(self.lib.nvfp4_swiglu_strided(self.h, _ptr(gate), _ptr(up), M, I, row_stride_in, _ptr(out),
                                                  row_stride_out, _stream(stream)))

    def linear_bf16(self, A, M, W, N, K, C, residual=None, stream=None):
        self._check(self.lib.nvfp4_linear_bf16(self.h, _ptr(A), M, _ptr(W), N, K, _ptr(residual), _ptr(C), _stream(stream)))

    def rmsnorm(self, x, weight, eps, M, K, out, stream=None):
        self._check(self.lib.nvfp4_rmsnorm(self.h, _ptr(x), _ptr(weight), eps, M, K, _ptr(out), _stream(stream)))

    def add_rmsnorm(self, residual, bias, weight, eps, M, K, norm_out, stream=None):
        self._check(self.lib.nvfp4_add_rmsnorm(self.h, _ptr(residual), _ptr(bias), _ptr(weight), eps, M, K, _ptr(norm_out),
                                               _stream(stream)))

    def swiglu_interleaved(self, gate_up, M, I, row_stride_in, out, row_stride_out, stream=None):
        self._check(self.lib.nvfp4_swiglu_interleaved(self.h, _ptr(gate_up), M, I, row_stride_in, _ptr(out), row_stride_out,
                                                      _stream(stream)))

    def linear_host(self, A_host, M, packed, scale, global_scale, N, K, C_host, residual_host=None, stream=None):
        self._check(self.lib.nvfp4_linear_host(self.h, _ptr(A_host), M, _ptr(packed), _ptr(scale), global_scale,
                                               N, K, _ptr(residual_host), _ptr(C_host), _stream(stream)))


class Chain:
    """nvfp4_chain: a fixed sequence of linears (up to 8 tokens each) run by one launch.  `linears` is a list
    of dicts with the fields of nvfp4_linear_desc (A, M, packed, scale, global_scale, N, K, C and the
    optional residual, swiglu_up, a_row_stride, k_valid, px, norm_weight, norm_eps, swiglu_epilogue);
    tensors are given as torch tensors or raw addresses and must stay alive while the chain exists."""

    def __init__(self, handle, linears):
        self.handle = handle
        self.keep = linears
        arr = (LinearDesc * len(linears))()
        for d, l in zip(arr, linears):
            px = l.get("px")
            d.A, d.swiglu_up = _ptr(l["A"]), _ptr(l.get("swiglu_up"))
            d.a_row_stride, d.k_valid, d.M = l.get("a_row_stride", 0), l.get("k_valid", 0), l["M"]
            d.packed, d.scale, d.global_scale = _ptr(l["packed"]), _ptr(l["scale"]), l.get("global_scale", 1.0)
            d.N, d.K = l["N"], l["K"]
            d.residual, d.C = _ptr(l.get("residual")), _ptr(l["C"])
            d.px = None if px is None else ctypes.addressof(px)
            d.norm_weight, d.norm_eps = _ptr(l.get("norm_weight")), l.get("norm_eps", 0.0)
            d.swiglu_epilogue = int(bool(l.get("swiglu_epilogue", False)))
        c = c_void_p()
        st = handle.lib.nvfp4_chain_create(handle.h, arr, len(linears), ctypes.byref(c))
        if st:
            raise Nvfp4Error(st)
        self.c = c

    def run(self, stream=None):
        st = self.handle.lib.nvfp4_chain_run(self.c, _stream(stream))
        if st:
            raise Nvfp4Error(st)

    def close(self):
        if getattr(self, "c", None):
            self.handle.lib.nvfp4_chain_destroy(self.c)
            self.c = None
