"""NVFP4 checkpoint ingestion on the host (include/nvfp4_checkpoint.h): the safetensors reader
against files written by an independent pure-Python writer, the reference's merges
(src/engine/model.cpp:296-350, 456-514: plain row concatenation), the tensor-parallel shard rule
against its numpy statement (nvfp4_tp.py), and the offline shard tool end to end.  No checkpoint
is available offline, so the files are synthetic with the reference's tensor names."""
import json
import struct
import subprocess

import numpy as np
import pytest

import nvfp4_ckpt
import nvfp4_tp
import util


def py_write_safetensors(path, tensors, metadata=None, pad_header=0):
    """Independent writer: {name: (array, dtype)} in the given order, optional nested metadata."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (arr, dt) in tensors.items():
        b = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header).encode() + b" " * pad_header
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def linear_tensors(prefix, N, K, seed, gs, input_scale=None):
    packed, scale = util.make_weight(N, K, seed=seed)
    t = {prefix + ".weight_packed": (packed, "U8"), prefix + ".weight_scale": (scale, "F8_E4M3"),
         prefix + ".weight_global_scale": (np.array([gs], np.float32), "F32")}
    if input_scale is not None:
        t[prefix + ".input_global_scale"] = (np.array([input_scale], np.float32), "F32")
    return t, packed, scale


def test_reader_matches_independent_writer(tmp_path):
    p = "model.language_model.layers.3.mlp."
    tg, gp, gsc = linear_tensors(p + "gate_proj", 96, 256, 1, 2.5, input_scale=0.75)
    tu, up, usc = linear_tensors(p + "up_proj", 96, 256, 2, 2.5)
    extra = {"model.norm.weight": (np.arange(256, dtype=np.uint16), "BF16")}
    path = tmp_path / "a.safetensors"
    py_write_safetensors(path, {**extra, **tg, **tu}, metadata={"format": "pt", "nested": {"a": [1, {"b": "}"}]}}, pad_header=5)
    c = nvfp4_ckpt.Checkpoint(str(path))
    try:
        assert c.names()[0] == "model.norm.weight" and len(c.names()) == 8        # metadata is not a tensor
        packed, scale, gs, ins = c.linear(p + "gate_proj")
        assert np.array_equal(packed, gp) and np.array_equal(scale, gsc) and gs == 2.5 and ins == 0.75
        packed, scale, gs, ins = c.linear(p + "up_proj")
        assert np.array_equal(packed, up) and np.array_equal(scale, usc) and ins == 0.0
        norm, dt = c.tensor("model.norm.weight")
        assert dt == "BF16" and np.array_equal(norm, np.arange(256, dtype=np.uint16))
        with pytest.raises(nvfp4_ckpt.CkptError) as e:
            c.linear(p + "down_proj")
        assert e.value.status == -4
        with pytest.raises(nvfp4_ckpt.CkptError) as e:                         # a BF16 tensor is not a packed weight
            c.lib.nvfp4_ckpt_linear  # noqa: B018  (binding present)
            c.tensor("nope")
        assert e.value.status == -4
    finally:
        c.close()


def test_malformed_files_are_refused(tmp_path):
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")                         # header longer than the file
    with pytest.raises(nvfp4_ckpt.CkptError) as e:
        nvfp4_ckpt.Checkpoint(str(bad))
    assert e.value.status == -3
    h = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()   # 4 x F32 is 16 bytes, not 8
    bad.write_bytes(struct.pack("<Q", len(h)) + h + b"\0" * 8)
    with pytest.raises(nvfp4_ckpt.CkptError) as e:
        nvfp4_ckpt.Checkpoint(str(bad))
    assert e.value.status == -3
    with pytest.raises(nvfp4_ckpt.CkptError) as e:
        nvfp4_ckpt.Checkpoint(str(tmp_path / "missing.safetensors"))
    assert e.value.status == -2


def test_wrong_shapes_and_types(tmp_path):
    packed, scale = util.make_weight(32, 256, seed=3)
    path = tmp_path / "w.safetensors"
    py_write_safetensors(path, {"a.weight_packed": (packed, "U8"), "a.weight_scale": (scale[:, :8], "F8_E4M3"),
                                "a.weight_global_scale": (np.array([1.0], np.float32), "F32"),
                                "b.weight_packed": (packed.astype(np.int8), "I8"), "b.weight_scale": (scale, "F8_E4M3"),
                                "b.weight_global_scale": (np.array([1.0], np.float32), "F32")})
    c = nvfp4_ckpt.Checkpoint(str(path))
    try:
        with pytest.raises(nvfp4_ckpt.CkptError) as e:
            c.linear("a")
        assert e.value.status == -6
        with pytest.raises(nvfp4_ckpt.CkptError) as e:
            c.linear("b")
        assert e.value.status == -5
    finally:
        c.close()


def test_merge_rows_is_row_concatenation():
    q = util.make_weight(64, 512, seed=1)
    k = util.make_weight(16, 512, seed=2)
    v = util.make_weight(16, 512, seed=3)
    p, s, gs = nvfp4_ckpt.merge_rows([(q[0], q[1], 3.0), (k[0], k[1], 3.0), (v[0], v[1], 3.0)])
    assert gs == 3.0
    assert np.array_equal(p, np.concatenate([q[0], k[0], v[0]])) and np.array_equal(s, np.concatenate([q[1], k[1], v[1]]))
    with pytest.raises(nvfp4_ckpt.CkptError) as e:                              # the reference would take 3.0 for all parts
        nvfp4_ckpt.merge_rows([(q[0], q[1], 3.0), (k[0], k[1], 4.0)])
    assert e.value.status == -7
    other_k = util.make_weight(16, 256, seed=4)
    with pytest.raises(nvfp4_ckpt.CkptError) as e:
        nvfp4_ckpt.merge_rows([(q[0], q[1], 3.0), (other_k[0], other_k[1], 3.0)])
    assert e.value.status == -6


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_rule_matches_numpy_statement(world):
    H, I = 256, 17408 // 8        # I/8 = 272: K padding to 512 at world 8, as for the real I = 17408
    gu_p, gu_s = util.make_weight(2 * I, H, seed=5)
    dn_p, dn_s = util.make_weight(H, I, seed=6)
    for r in range(world):
        p, s = nvfp4_ckpt.shard_gate_up(gu_p, gu_s, 1.0, r, world)
        wp, ws = nvfp4_tp.shard_gate_up(gu_p, gu_s, r, world)
        assert np.array_equal(p, wp) and np.array_equal(s, ws)
        p, s = nvfp4_ckpt.shard_down(dn_p, dn_s, 1.0, r, world)
        wp, ws = nvfp4_tp.shard_down(dn_p, dn_s, r, world)
        assert np.array_equal(p, wp) and np.array_equal(s, ws)
    with pytest.raises(nvfp4_ckpt.CkptError):
        nvfp4_ckpt.shard_down(dn_p, dn_s, 1.0, 0, 3)                             # I not divisible by 16 * 3... (2176 % 48)


def test_shard_tool_end_to_end(tmp_path):
    """The offline tool on a synthetic checkpoint: every rank file holds exactly the shards the
    numpy rule gives, and the sharded MLP of the CPU oracle equals the unsplit one up to the
    rounding of the partial sums."""
    import oracle_binding as ob
    H, I, world = 256, 512, 2
    p = "model.language_model.layers.0.mlp."
    tg, gp, gs_ = linear_tensors(p + "gate_proj", I, H, 11, 1.0)
    tu, up, us_ = linear_tensors(p + "up_proj", I, H, 12, 1.0)
    td, dp, ds_ = linear_tensors(p + "down_proj", H, I, 13, 1.0)
    src = tmp_path / "model.safetensors"
    py_write_safetensors(src, {**tg, **tu, **td}, metadata={"format": "pt"})
    out = subprocess.run([nvfp4_ckpt.SHARD_TOOL_PATH, str(src), str(tmp_path / "mlp0"), str(world), p + "gate_proj",
                          p + "up_proj", p + "down_proj"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    gu_p, gu_s = np.concatenate([gp, up]), np.concatenate([gs_, us_])
    for r in range(world):
        c = nvfp4_ckpt.Checkpoint(str(tmp_path / f"mlp0.rank{r}.safetensors"))
        try:
            packed, scale, g, _ = c.linear("gate_up")
            wp, ws = nvfp4_tp.shard_gate_up(gu_p, gu_s, r, world)
            assert np.array_equal(packed, wp) and np.array_equal(scale, ws) and g == 1.0
            packed, scale, g, _ = c.linear("down")
            wp, ws = nvfp4_tp.shard_down(dp, ds_, r, world)
            assert np.array_equal(packed, wp) and np.array_equal(scale, ws)
        finally:
            c.close()
    X = util.make_bf16((3, H), seed=14)
    whole = ob.mlp(X, gu_p, gu_s, 1.0, dp, ds_, 1.0)
    split = ob.tp_mlp(X, world, gu_p, gu_s, 1.0, dp, ds_, 1.0, partial_bf16=False)
    assert ob.rel_frobenius(split, whole) <= 1e-3
    bad = subprocess.run([nvfp4_ckpt.SHARD_TOOL_PATH, str(src), str(tmp_path / "x"), "2", p + "gate_proj", p + "up_proj", "nope"],
                         capture_output=True, text=True)
    assert bad.returncode == 1 and "no tensor of that name" in bad.stderr


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_qkv_shard_rule_matches_numpy_statement(world):
    H, q_rows, kv_rows, n_kv = 256, 768, 128, 2
    p, s = util.make_weight(q_rows + 2 * kv_rows, H, seed=7)
    for r in range(world):
        cp, cs = nvfp4_ckpt.shard_qkv(p, s, 1.0, q_rows, kv_rows, n_kv, r, world)
        wp, ws = nvfp4_tp.shard_qkv(p, s, q_rows, kv_rows, n_kv, r, world)
        assert np.array_equal(cp, wp) and np.array_equal(cs, ws)
    with pytest.raises(nvfp4_ckpt.CkptError):
        nvfp4_ckpt.shard_qkv(p, s, 1.0, q_rows, kv_rows, n_kv, 0, 3)             # 3 ranks and 2 KV heads do not divide


def test_shard_tool_attention_projections(tmp_path):
    """The tool's attn form: q, k, v merged by rows, then every rank file holds the QKV rows of its
    KV-head group and its K columns of the output projection."""
    H, q_rows, kv_rows, n_kv, world = 256, 512, 128, 2, 4
    p = "model.language_model.layers.3.self_attn."
    tq, qp, qs = linear_tensors(p + "q_proj", q_rows, H, 21, 2.0)
    tk, kp, ks = linear_tensors(p + "k_proj", kv_rows, H, 22, 2.0)
    tv, vp, vs = linear_tensors(p + "v_proj", kv_rows, H, 23, 2.0)
    to, op, os_ = linear_tensors(p + "o_proj", H, q_rows, 24, 1.0)
    src = tmp_path / "model.safetensors"
    py_write_safetensors(src, {**tq, **tk, **tv, **to}, metadata={"format": "pt"})
    out = subprocess.run([nvfp4_ckpt.SHARD_TOOL_PATH, "attn", str(src), str(tmp_path / "attn3"), str(world), str(n_kv),
                          p + "q_proj", p + "k_proj", p + "v_proj", p + "o_proj"], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    mp, ms = np.concatenate([qp, kp, vp]), np.concatenate([qs, ks, vs])
    for r in range(world):
        c = nvfp4_ckpt.Checkpoint(str(tmp_path / f"attn3.rank{r}.safetensors"))
        try:
            packed, scale, g, _ = c.linear("qkv")
            wp, ws = nvfp4_tp.shard_qkv(mp, ms, q_rows, kv_rows, n_kv, r, world)
            assert np.array_equal(packed, wp) and np.array_equal(scale, ws) and g == 2.0
            packed, scale, g, _ = c.linear("o")
            wp, ws = nvfp4_tp.shard_down(op, os_, r, world)
            assert np.array_equal(packed, wp) and np.array_equal(scale, ws) and g == 1.0
        finally:
            c.close()


def test_interleave_gate_up_matches_numpy_statement():
    """Slabs of 8 gate rows followed by their 8 up rows; a shard of the tensor-parallel split works the same."""
    H, I = 256, 272
    p, s = util.make_weight(2 * I, H, seed=9)
    order = nvfp4_tp.interleave_rows(I)
    assert sorted(order) == list(range(2 * I))
    assert list(order[:16]) == list(range(8)) + list(range(I, I + 8))
    cp, cs = nvfp4_ckpt.interleave_gate_up(p, s, 1.0)
    assert np.array_equal(cp, p[order]) and np.array_equal(cs, s[order])
    with pytest.raises(nvfp4_ckpt.CkptError):
        nvfp4_ckpt.interleave_gate_up(p[:2 * I - 8], s[:2 * I - 8], 1.0)          # 2I not a multiple of 16


def test_writer_roundtrip(tmp_path):
    a = np.arange(24, dtype=np.uint8).reshape(2, 12)
    b = np.array([1.5], np.float32)
    path = tmp_path / "w.safetensors"
    nvfp4_ckpt.write(str(path), {'we"ird\\name': (a, "U8"), "s": (b, "F32")})
    raw = path.read_bytes()
    hlen = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + hlen])                                        # a standard JSON parser accepts the header
    assert header['we"ird\\name']["shape"] == [2, 12] and (8 + hlen) % 8 == 0
    c = nvfp4_ckpt.Checkpoint(str(path))
    try:
        got, dt = c.tensor('we"ird\\name')
        assert dt == "U8" and np.array_equal(got, a)
        got, dt = c.tensor("s")
        assert got[0] == 1.5
    finally:
        c.close()
