"""Host side of the tensor-parallel NVFP4 blocks (MLP, attention projections): ctypes binding of libnvfp4_b200_tp.so
(include/nvfp4_b200_tp.h) and the numpy statement of its sharding rule, which the CPU
(gloo) tests run against the oracle.  One process per GPU; the communicator id travels over
whatever channel the caller has (the benchmark broadcasts it with torch.distributed)."""
import ctypes
import os

import numpy as np

import nvfp4

_HERE = os.path.dirname(os.path.abspath(__file__))
TP_LIB_PATH = os.path.join(_HERE, "lib", "libnvfp4_b200_tp.so")
UNIQUE_ID_BYTES = 128
P2P_HANDLE_BYTES = 64

c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

TP_SIGNATURES = {
    "nvfp4_tp_unique_id": (c_int, [c_void_p]),
    "nvfp4_tp_comm_create": (c_int, [c_void_p, c_int, c_int, ctypes.POINTER(c_void_p)]),
    "nvfp4_tp_comm_destroy": (c_int, [c_void_p]),
    "nvfp4_tp_comm_set_bf16_partials": (c_int, [c_void_p, c_int]),
    "nvfp4_tp_comm_set_deadline_ms": (c_int, [c_void_p, c_int]),
    "nvfp4_tp_comm_state": (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    "nvfp4_tp_comm_abort": (c_int, [c_void_p]),
    "nvfp4_tp_mlp_create": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                    c_float, c_int, ctypes.POINTER(c_void_p)]),
    "nvfp4_tp_mlp_destroy": (c_int, [c_void_p]),
    "nvfp4_tp_mlp_forward": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "nvfp4_tp_mlp_shard_bytes": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_size_t)]),
    "nvfp4_tp_mlp_p2p_handle": (c_int, [c_void_p, c_void_p]),
    "nvfp4_tp_mlp_p2p_attach": (c_int, [c_void_p, c_void_p]),
    "nvfp4_tp_mlp_set_fused": (c_int, [c_void_p, c_int]),
    "nvfp4_tp_mlp_status": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_uint)]),
    "nvfp4_tp_mlp_use_exchange": (c_int, [c_void_p, c_void_p]),
    "nvfp4_tp_exchange_create": (c_int, [c_void_p, c_int, ctypes.POINTER(c_void_p)]),
    "nvfp4_tp_exchange_destroy": (c_int, [c_void_p]),
    "nvfp4_tp_exchange_handle": (c_int, [c_void_p, c_void_p]),
    "nvfp4_tp_exchange_attach": (c_int, [c_void_p, c_void_p]),
    "nvfp4_tp_exchange_status": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_uint)]),
    "nvfp4_tp_attn_create": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float,
                                     c_void_p, c_void_p, c_float, c_int, ctypes.POINTER(c_void_p)]),
    "nvfp4_tp_attn_destroy": (c_int, [c_void_p]),
    "nvfp4_tp_attn_dims": (c_int, [c_void_p, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "nvfp4_tp_attn_shard_bytes": (c_int, [c_void_p, ctypes.POINTER(ctypes.c_size_t)]),
    "nvfp4_tp_attn_use_exchange": (c_int, [c_void_p, c_void_p]),
    "nvfp4_tp_attn_set_fused": (c_int, [c_void_p, c_int]),
    "nvfp4_tp_attn_qkv": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "nvfp4_tp_attn_out": (c_int, [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_void_p, c_void_p, c_void_p]),
}

_lib = None


def load():
    global _lib
    if _lib is None:
        nvfp4.load()
        if not os.path.exists(TP_LIB_PATH):
            raise RuntimeError(f"{TP_LIB_PATH} is missing: build it with `make -C {_HERE}`")
        lib = ctypes.CDLL(TP_LIB_PATH)
        for name, (res, args) in TP_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


# ------------------------------------------------------------------ sharding rule (numpy, host)

def shard_gate_up(packed, scale, rank, world):
    """Merged gate/up [2I, H]: rank r keeps gate rows and up rows [r*I/P, (r+1)*I/P), merged again."""
    I = packed.shape[0] // 2
    assert I % (16 * world) == 0
    ip = I // world
    rows = np.r_[rank * ip:(rank + 1) * ip, I + rank * ip:I + (rank + 1) * ip]
    return np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scale[rows])


def shard_down(packed, scale, rank, world):
    """Down [H, I]: rank r keeps K columns [r*I/P, (r+1)*I/P), K zero-padded to a multiple of 256
    (zero codes and zero scales: the padding contributes exactly nothing)."""
    H, I = packed.shape[0], packed.shape[1] * 2
    assert I % (16 * world) == 0
    ip = I // world
    kp = (ip + 255) // 256 * 256
    p = np.zeros((H, kp // 2), np.uint8)
    s = np.zeros((H, kp // 16), np.uint8)
    p[:, :ip // 2] = packed[:, rank * ip // 2:(rank + 1) * ip // 2]
    s[:, :ip // 16] = scale[:, rank * ip // 16:(rank + 1) * ip // 16]
    return p, s


def qkv_rows(q_rows, kv_rows, n_kv_heads, rank, world):
    """Row indices of the merged [q_rows + 2*kv_rows, H] tensor (q, k, v) that rank r keeps: its share
    of the q rows and the k and v rows of its KV heads (of KV head r // (P // n_kv) when the ranks
    outnumber the KV heads)."""
    assert q_rows % (8 * world) == 0 and kv_rows % n_kv_heads == 0
    ql = q_rows // world
    head = kv_rows // n_kv_heads
    if world <= n_kv_heads:
        assert n_kv_heads % world == 0
        kvl, kv0 = kv_rows // world, rank * (kv_rows // world)
    else:
        assert world % n_kv_heads == 0
        kvl, kv0 = head, (rank // (world // n_kv_heads)) * head
    return np.r_[rank * ql:(rank + 1) * ql, q_rows + kv0:q_rows + kv0 + kvl,
                 q_rows + kv_rows + kv0:q_rows + kv_rows + kv0 + kvl]


def shard_qkv(packed, scale, q_rows, kv_rows, n_kv_heads, rank, world):
    rows = qkv_rows(q_rows, kv_rows, n_kv_heads, rank, world)
    return np.ascontiguousarray(packed[rows]), np.ascontiguousarray(scale[rows])


def interleave_rows(I):
    """Row order of the swiglu_epilogue layout for a merged gate/up tensor of 2I rows."""
    assert I % 8 == 0
    s = np.arange(I // 8)[:, None] * 8 + np.arange(8)[None, :]
    return np.concatenate([s, I + s], axis=1).reshape(-1)


def pad_activation(act, kp):
    """[M, I/P] BF16 bits -> [M, kp] with zero padding."""
    out = np.zeros((act.shape[0], kp), act.dtype)
    out[:, :act.shape[1]] = act
    return out


# ------------------------------------------------------------------ host-side pre-flight of a step

class TpStepError(RuntimeError):
    """A tensor-parallel step was called off before anything was enqueued."""


class StepGuard:
    """Pre-flight of a tensor-parallel step, on the host, before any kernel or collective is enqueued.

    A collective that one rank never joins, or joins with another token count, leaves the other
    ranks waiting on the device; so every rank first posts the token count it is about to enqueue
    (or the failure it hit) in a key-value store all ranks reach -- the torch.distributed store of
    the process group, or any object with set / get / wait(keys, timeout) -- and reads the others'.
    A rank that posts another count, posts a failure, or posts nothing within the deadline makes
    every rank raise TpStepError; the caller then skips the step (and, for a rank that is gone for
    good, aborts the communicator: Comm.abort).  Failures are found out between steps only, with
    nothing in flight on the GPUs.
    (The reference's single-GPU analogue: the bounded polling of sync_stream_with_timeout,
    src/engine/engine.cpp:38-61, and the request-level error codes of :332-337.)"""

    def __init__(self, store, rank, world, deadline_s=5.0, prefix="nvfp4_tp_step"):
        self.store, self.rank, self.world = store, rank, world
        self.deadline_s, self.prefix = float(deadline_s), prefix
        self.step = 0

    def _key(self, rank):
        return f"{self.prefix}/{self.step}/{rank}"

    def fail(self, reason):
        """Call instead of check() when this rank cannot take part in the step: the others learn of it at once."""
        self.store.set(self._key(self.rank), "fail:" + str(reason))
        self.step += 1

    def check(self, M):
        """Every rank calls this with its token count before it enqueues the step."""
        import datetime
        self.store.set(self._key(self.rank), str(int(M)))
        others = [r for r in range(self.world) if r != self.rank]
        step = self.step
        self.step += 1
        try:
            if others:
                self.store.wait([f"{self.prefix}/{step}/{r}" for r in others], datetime.timedelta(seconds=self.deadline_s))
        except Exception as e:      # the store's timeout error type depends on the store
            raise TpStepError(f"step {step}: a rank did not report within {self.deadline_s} s ({type(e).__name__})") from None
        for r in others:
            v = self.store.get(f"{self.prefix}/{step}/{r}")
            v = v.decode() if isinstance(v, (bytes, bytearray)) else str(v)
            if v.startswith("fail:"):
                raise TpStepError(f"step {step}: rank {r} failed before the step: {v[5:]}")
            if int(v) != int(M):
                raise TpStepError(f"step {step}: rank {r} is about to enqueue {v} tokens, this rank {int(M)}")
        return True


# ------------------------------------------------------------------ device objects

class Comm:
    def __init__(self, unique_id, rank, world):
        self.lib = load()
        c = c_void_p()
        buf = None if unique_id is None else ctypes.create_string_buffer(bytes(unique_id), UNIQUE_ID_BYTES)
        st = self.lib.nvfp4_tp_comm_create(buf, rank, world, ctypes.byref(c))
        if st:
            raise nvfp4.Nvfp4Error(st)
        self.c, self.rank, self.world = c, rank, world

    def set_bf16_partials(self, on):
        """NCCL path of the row-split linears: False (default) = FP32 partials (reduce-scatter, finish on
        the rank's slice, all-gather), True = one all-reduce of BF16-rounded partials."""
        st = self.lib.nvfp4_tp_comm_set_bf16_partials(self.c, int(bool(on)))
        if st:
            raise nvfp4.Nvfp4Error(st)

    def set_deadline_ms(self, ms):
        """How long a call on the (non-blocking) communicator may stay "in progress" before it is aborted."""
        st = self.lib.nvfp4_tp_comm_set_deadline_ms(self.c, int(ms))
        if st:
            raise nvfp4.Nvfp4Error(st)

    def state(self):
        """0 = idle or healthy, 1 = a call is in progress, -1 = failed or aborted."""
        v = c_int()
        st = self.lib.nvfp4_tp_comm_state(self.c, ctypes.byref(v))
        if st:
            raise nvfp4.Nvfp4Error(st)
        return v.value

    def abort(self):
        st = self.lib.nvfp4_tp_comm_abort(self.c)
        if st:
            raise nvfp4.Nvfp4Error(st)

    def close(self):
        if getattr(self, "c", None):
            self.lib.nvfp4_tp_comm_destroy(self.c)
            self.c = None


def unique_id():
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    st = load().nvfp4_tp_unique_id(buf)
    if st:
        raise nvfp4.Nvfp4Error(st)
    return bytes(buf.raw)


class Exchange:
    """A rank's peer-exchange buffer for the fused small-M reduction, shared by any number of blocks."""

    def __init__(self, comm, H):
        self.lib = load()
        x = c_void_p()
        st = self.lib.nvfp4_tp_exchange_create(comm.c, H, ctypes.byref(x))
        if st:
            raise nvfp4.Nvfp4Error(st)
        self.x = x

    def handle(self):
        buf = ctypes.create_string_buffer(P2P_HANDLE_BYTES)
        st = self.lib.nvfp4_tp_exchange_handle(self.x, buf)
        if st:
            raise nvfp4.Nvfp4Error(st)
        return bytes(buf.raw)

    def attach(self, handles):
        buf = None if handles is None else ctypes.create_string_buffer(bytes(handles), len(handles))
        st = self.lib.nvfp4_tp_exchange_attach(self.x, buf)
        if st:
            raise nvfp4.Nvfp4Error(st)

    def enable(self, dist=None, device=None):
        """Collective: exchange the buffer handles over torch.distributed and attach."""
        if dist is None or dist.get_world_size() == 1:
            return self.attach(None)
        import torch
        mine = torch.tensor(list(self.handle()), dtype=torch.uint8, device=device)
        allh = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(allh, mine)
        self.attach(b"".join(bytes(t.cpu().tolist()) for t in allh))

    def status(self):
        v = ctypes.c_uint()
        st = self.lib.nvfp4_tp_exchange_status(self.x, ctypes.byref(v))
        if st:
            raise nvfp4.Nvfp4Error(st)
        return v.value

    def close(self):
        if getattr(self, "x", None):
            self.lib.nvfp4_tp_exchange_destroy(self.x)
            self.x = None


class TpAttn:
    """Tensor-parallel attention projections (QKV split by KV-head groups, output projection split by K)."""

    def __init__(self, handle, comm, H, q_rows, kv_rows, n_kv_heads, o_in, qkv_packed, qkv_scale, qkv_gs, o_packed,
                 o_scale, o_gs, max_M):
        self.lib = load()
        a = c_void_p()
        st = self.lib.nvfp4_tp_attn_create(handle.h, comm.c, H, q_rows, kv_rows, n_kv_heads, o_in, qkv_packed.data_ptr(),
                                           qkv_scale.data_ptr(), qkv_gs, o_packed.data_ptr(), o_scale.data_ptr(), o_gs,
                                           max_M, ctypes.byref(a))
        if st:
            raise nvfp4.Nvfp4Error(st)
        self.a, self.H = a, H
        q, kv, o = c_int(), c_int(), c_int()
        self.lib.nvfp4_tp_attn_dims(a, ctypes.byref(q), ctypes.byref(kv), ctypes.byref(o))
        self.q_local, self.kv_local, self.o_local = q.value, kv.value, o.value

    def qkv(self, X, M, qkv_out, stream=None):
        st = self.lib.nvfp4_tp_attn_qkv(self.a, X.data_ptr(), M, qkv_out.data_ptr(), nvfp4._stream(stream))
        if st:
            raise nvfp4.Nvfp4Error(st)

    def out(self, attn, M, out, residual=None, row_stride=0, stream=None):
        ptr = attn if isinstance(attn, int) else attn.data_ptr()
        st = self.lib.nvfp4_tp_attn_out(self.a, ptr, row_stride, M, None if residual is None else residual.data_ptr(),
                                        out.data_ptr(), nvfp4._stream(stream))
        if st:
            raise nvfp4.Nvfp4Error(st)

    def use_exchange(self, x):
        st = self.lib.nvfp4_tp_attn_use_exchange(self.a, None if x is None else x.x)
        if st:
            raise nvfp4.Nvfp4Error(st)

    def set_fused(self, mode):
        st = self.lib.nvfp4_tp_attn_set_fused(self.a, int(mode))
        if st:
            raise nvfp4.Nvfp4Error(st)

    def shard_bytes(self):
        v = ctypes.c_size_t()
        self.lib.nvfp4_tp_attn_shard_bytes(self.a, ctypes.byref(v))
        return v.value

    def close(self):
        if getattr(self, "a", None):
            self.lib.nvfp4_tp_attn_destroy(self.a)
            self.a = None


class TpMlp:
    def __init__(self, handle, comm, H, I, gu_packed, gu_scale, gu_gs, dn_packed, dn_scale, dn_gs, max_M):
        self.lib = load()
        m = c_void_p()
        st = self.lib.nvfp4_tp_mlp_create(handle.h, comm.c, H, I, gu_packed.data_ptr(), gu_scale.data_ptr(), gu_gs,
                                          dn_packed.data_ptr(), dn_scale.data_ptr(), dn_gs, max_M, ctypes.byref(m))
        if st:
            raise nvfp4.Nvfp4Error(st)
        self.m, self.H, self.I = m, H, I

    def forward(self, X, M, out, residual=None, stream=None):
        st = self.lib.nvfp4_tp_mlp_forward(self.m, X.data_ptr(), M, None if residual is None else residual.data_ptr(),
                                           out.data_ptr(), nvfp4._stream(stream))
        if st:
            raise nvfp4.Nvfp4Error(st)

    def p2p_handle(self):
        buf = ctypes.create_string_buffer(P2P_HANDLE_BYTES)
        st = self.lib.nvfp4_tp_mlp_p2p_handle(self.m, buf)
        if st:
            raise nvfp4.Nvfp4Error(st)
        return bytes(buf.raw)

    def p2p_attach(self, handles):
        """handles: the ranks' p2p_handle() bytes concatenated in rank order (None for world 1).
        Afterwards forward() sums up to 16 tokens with the fused peer-memory kernel."""
        buf = None if handles is None else ctypes.create_string_buffer(bytes(handles), len(handles))
        st = self.lib.nvfp4_tp_mlp_p2p_attach(self.m, buf)
        if st:
            raise nvfp4.Nvfp4Error(st)

    def enable_p2p(self, dist=None, device=None):
        """Collective: exchange the buffer handles over torch.distributed and attach."""
        if dist is None or dist.get_world_size() == 1:
            return self.p2p_attach(None)
        import torch
        mine = torch.tensor(list(self.p2p_handle()), dtype=torch.uint8, device=device)
        allh = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(allh, mine)
        self.p2p_attach(b"".join(bytes(t.cpu().tolist()) for t in allh))

    def use_exchange(self, x):
        st = self.lib.nvfp4_tp_mlp_use_exchange(self.m, None if x is None else x.x)
        if st:
            raise nvfp4.Nvfp4Error(st)

    def set_fused(self, mode):
        """0/False = NCCL all-reduce, 1/True = reduction fused into the down-projection kernel,
        2 = separate push-and-sum kernel."""
        st = self.lib.nvfp4_tp_mlp_set_fused(self.m, int(mode))
        if st:
            raise nvfp4.Nvfp4Error(st)

    def status(self):
        v = ctypes.c_uint()
        st = self.lib.nvfp4_tp_mlp_status(self.m, ctypes.byref(v))
        if st:
            raise nvfp4.Nvfp4Error(st)
        return v.value

    def shard_bytes(self):
        v = ctypes.c_size_t()
        self.lib.nvfp4_tp_mlp_shard_bytes(self.m, ctypes.byref(v))
        return v.value

    def close(self):
        if getattr(self, "m", None):
            self.lib.nvfp4_tp_mlp_destroy(self.m)
            self.m = None
