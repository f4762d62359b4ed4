"""ctypes binding of libnvfp4_ckpt.so (include/nvfp4_checkpoint.h): NVFP4 checkpoint ingestion on
the host -- safetensors reader/writer, the reference's row merges, the tensor-parallel shard rule."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
CKPT_LIB_PATH = os.path.join(_HERE, "lib", "libnvfp4_ckpt.so")
SHARD_TOOL_PATH = os.path.join(_HERE, "lib", "nvfp4_shard")

c_void_p, c_int, c_char_p = ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p


class CkptTensor(ctypes.Structure):
    _fields_ = [("data", c_void_p), ("nbytes", ctypes.c_size_t), ("dtype", ctypes.c_char * 16), ("rank", c_int),
                ("shape", ctypes.c_longlong * 8)]


class HostWeight(ctypes.Structure):
    _fields_ = [("packed", c_void_p), ("scale", c_void_p), ("global_scale", ctypes.c_float), ("input_scale", ctypes.c_float),
                ("N", c_int), ("K", c_int)]


CKPT_SIGNATURES = {
    "nvfp4_ckpt_open": (c_int, [c_char_p, ctypes.POINTER(c_void_p)]),
    "nvfp4_ckpt_close": (c_int, [c_void_p]),
    "nvfp4_ckpt_count": (c_int, [c_void_p]),
    "nvfp4_ckpt_name": (c_char_p, [c_void_p, c_int]),
    "nvfp4_ckpt_get": (c_int, [c_void_p, c_char_p, ctypes.POINTER(CkptTensor)]),
    "nvfp4_ckpt_linear": (c_int, [c_void_p, c_char_p, ctypes.POINTER(HostWeight)]),
    "nvfp4_merge_rows": (c_int, [ctypes.POINTER(HostWeight), c_int, c_void_p, c_void_p, ctypes.POINTER(HostWeight)]),
    "nvfp4_merge_rows_ex": (c_int, [ctypes.POINTER(HostWeight), c_int, c_void_p, c_void_p, ctypes.POINTER(HostWeight), c_int]),
    "nvfp4_tp_shard_gate_up": (c_int, [ctypes.POINTER(HostWeight), c_int, c_int, c_void_p, c_void_p, ctypes.POINTER(HostWeight)]),
    "nvfp4_tp_shard_down": (c_int, [ctypes.POINTER(HostWeight), c_int, c_int, c_void_p, c_void_p, ctypes.POINTER(HostWeight)]),
    "nvfp4_tp_shard_down_k": (c_int, [c_int, c_int]),
    "nvfp4_interleave_gate_up": (c_int, [ctypes.POINTER(HostWeight), c_void_p, c_void_p, ctypes.POINTER(HostWeight)]),
    "nvfp4_tp_shard_qkv": (c_int, [ctypes.POINTER(HostWeight), c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                   ctypes.POINTER(HostWeight)]),
    "nvfp4_tp_shard_qkv_rows": (c_int, [c_int, c_int, c_int, c_int]),
    "nvfp4_ckpt_write": (c_int, [c_char_p, ctypes.POINTER(c_char_p), ctypes.POINTER(CkptTensor), c_int]),
    "nvfp4_ckpt_status_string": (c_char_p, [c_int]),
}

_lib = None


class CkptError(RuntimeError):
    def __init__(self, status):
        self.status = status
        super().__init__(f"nvfp4_ckpt status {status}: {load().nvfp4_ckpt_status_string(status).decode()}")


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(CKPT_LIB_PATH):
            raise RuntimeError(f"{CKPT_LIB_PATH} is missing: build it with `make -C {_HERE}`")
        lib = ctypes.CDLL(CKPT_LIB_PATH)
        for name, (res, args) in CKPT_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def _check(st):
    if st:
        raise CkptError(st)


_NP = {"U8": np.uint8, "F8_E4M3": np.uint8, "F8_E5M2": np.uint8, "I8": np.int8, "BF16": np.uint16, "F16": np.float16,
       "F32": np.float32, "I32": np.int32, "I64": np.int64}


class Checkpoint:
    """A read-only mapped safetensors file; arrays returned by tensor()/linear() are copies."""

    def __init__(self, path):
        self.lib = load()
        c = c_void_p()
        _check(self.lib.nvfp4_ckpt_open(os.fsencode(path), ctypes.byref(c)))
        self.c = c

    def names(self):
        return [self.lib.nvfp4_ckpt_name(self.c, i).decode() for i in range(self.lib.nvfp4_ckpt_count(self.c))]

    def tensor(self, name):
        t = CkptTensor()
        _check(self.lib.nvfp4_ckpt_get(self.c, name.encode(), ctypes.byref(t)))
        dt = t.dtype.decode()
        shape = tuple(t.shape[i] for i in range(t.rank))
        raw = ctypes.string_at(t.data, t.nbytes)
        return np.frombuffer(raw, dtype=_NP.get(dt, np.uint8)).reshape(shape).copy(), dt

    def linear(self, prefix):
        """(packed [N, K/2] u8, scale [N, K/16] u8, global_scale, input_scale)"""
        w = HostWeight()
        _check(self.lib.nvfp4_ckpt_linear(self.c, prefix.encode(), ctypes.byref(w)))
        packed = np.frombuffer(ctypes.string_at(w.packed, w.N * w.K // 2), np.uint8).reshape(w.N, w.K // 2).copy()
        scale = np.frombuffer(ctypes.string_at(w.scale, w.N * w.K // 16), np.uint8).reshape(w.N, w.K // 16).copy()
        return packed, scale, float(w.global_scale), float(w.input_scale)

    def close(self):
        if getattr(self, "c", None):
            self.lib.nvfp4_ckpt_close(self.c)
            self.c = None


def _host_weight(packed, scale, gs):
    w = HostWeight()
    w.packed, w.scale = packed.ctypes.data, scale.ctypes.data
    w.global_scale, w.input_scale = gs, 0.0
    w.N, w.K = packed.shape[0], packed.shape[1] * 2
    return w


def merge_rows(parts, take_first_scale=False):
    """parts: [(packed, scale, global_scale), ...] with equal K -> merged triple.  Different global scales
    are an error unless take_first_scale (the reference's rule: the first part's scale for all rows)."""
    lib = load()
    arr = (HostWeight * len(parts))(*[_host_weight(np.ascontiguousarray(p), np.ascontiguousarray(s), g) for p, s, g in parts])
    keep = [(np.ascontiguousarray(p), np.ascontiguousarray(s)) for p, s, _ in parts]
    for i, (p, s) in enumerate(keep):
        arr[i].packed, arr[i].scale = p.ctypes.data, s.ctypes.data
    rows = sum(p.shape[0] for p, _ in keep)
    K = keep[0][0].shape[1] * 2
    po, so = np.empty((rows, K // 2), np.uint8), np.empty((rows, K // 16), np.uint8)
    m = HostWeight()
    _check(lib.nvfp4_merge_rows_ex(arr, len(parts), po.ctypes.data, so.ctypes.data, ctypes.byref(m), int(take_first_scale)))
    return po, so, float(m.global_scale)


def shard_gate_up(packed, scale, gs, rank, world):
    lib = load()
    packed, scale = np.ascontiguousarray(packed), np.ascontiguousarray(scale)
    w = _host_weight(packed, scale, gs)
    rows, K = packed.shape[0] // world, packed.shape[1] * 2
    po, so = np.empty((rows, K // 2), np.uint8), np.empty((rows, K // 16), np.uint8)
    out = HostWeight()
    _check(lib.nvfp4_tp_shard_gate_up(ctypes.byref(w), rank, world, po.ctypes.data, so.ctypes.data, ctypes.byref(out)))
    return po, so


def interleave_gate_up(packed, scale, gs):
    """Merged gate/up rows -> slabs of 8 gate rows + their 8 up rows (the swiglu_epilogue layout)."""
    lib = load()
    packed, scale = np.ascontiguousarray(packed), np.ascontiguousarray(scale)
    w = _host_weight(packed, scale, gs)
    po, so = np.empty_like(packed), np.empty_like(scale)
    out = HostWeight()
    _check(lib.nvfp4_interleave_gate_up(ctypes.byref(w), po.ctypes.data, so.ctypes.data, ctypes.byref(out)))
    return po, so


def shard_qkv(packed, scale, gs, q_rows, kv_rows, n_kv_heads, rank, world):
    lib = load()
    packed, scale = np.ascontiguousarray(packed), np.ascontiguousarray(scale)
    w = _host_weight(packed, scale, gs)
    rows = lib.nvfp4_tp_shard_qkv_rows(q_rows, kv_rows, n_kv_heads, world)
    _check(rows if rows < 0 else 0)
    K = packed.shape[1] * 2
    po, so = np.empty((rows, K // 2), np.uint8), np.empty((rows, K // 16), np.uint8)
    out = HostWeight()
    _check(lib.nvfp4_tp_shard_qkv(ctypes.byref(w), q_rows, kv_rows, n_kv_heads, rank, world, po.ctypes.data, so.ctypes.data,
                                  ctypes.byref(out)))
    return po, so


def shard_down(packed, scale, gs, rank, world):
    lib = load()
    packed, scale = np.ascontiguousarray(packed), np.ascontiguousarray(scale)
    w = _host_weight(packed, scale, gs)
    kp = lib.nvfp4_tp_shard_down_k(w.K, world)
    _check(kp if kp < 0 else 0)
    po, so = np.empty((w.N, kp // 2), np.uint8), np.empty((w.N, kp // 16), np.uint8)
    out = HostWeight()
    _check(lib.nvfp4_tp_shard_down(ctypes.byref(w), rank, world, po.ctypes.data, so.ctypes.data, ctypes.byref(out)))
    return po, so


def write(path, tensors):
    """tensors: {name: (array, dtype string)}; arrays are written as their raw bytes."""
    lib = load()
    names = (c_char_p * len(tensors))(*[n.encode() for n in tensors])
    keep = [np.ascontiguousarray(a) for a, _ in tensors.values()]
    arr = (CkptTensor * len(tensors))()
    for i, ((a, dt), k) in enumerate(zip(tensors.values(), keep)):
        arr[i].data, arr[i].nbytes, arr[i].dtype, arr[i].rank = k.ctypes.data, k.nbytes, dt.encode(), k.ndim
        for d in range(k.ndim):
            arr[i].shape[d] = k.shape[d]
    _check(lib.nvfp4_ckpt_write(os.fsencode(path), names, arr, len(tensors)))
