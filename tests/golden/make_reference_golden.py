"""Generates tests/golden/reference_b200.npz: outputs of the REFERENCE engine's own NVFP4
kernels (its dense_gemm_fp4_sm110.cu compiled unmodified for sm_100a into
oracle/_ref/libref_fp4.so by oracle/Makefile) on seeded inputs, run on a B200.

    python tests/golden/make_reference_golden.py [out.npz]

Inputs are not stored: cases() rebuilds them from seeds, so the CPU tests can feed the same
inputs to the oracle and compare with the stored reference outputs.  The reference has no
golden vectors of its own for this path; these files are what pins the oracle.

The dequant cases go through invoke_fp4_gemm with M = K = 16 and an identity activation
matrix: M > 8 takes the reference's dequant-to-BF16 + library GEMM path, and with a one-hot
activation row the FP32 accumulation returns the dequantised BF16 weight exactly, so the
output is the transposed table of fp4_dequant_kernel.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import oracle_binding as ob  # noqa: E402
import util  # noqa: E402


def _table_weight():
    packed = np.tile(np.array([(2 * j) | ((2 * j + 1) << 4) for j in range(8)], np.uint8), (256, 1))
    scale = np.arange(256, dtype=np.uint8).reshape(256, 1)
    return packed, scale


def cases():
    out = {}
    ident = ob.f32_to_bf16(np.eye(16, dtype=np.float32))
    for gs in (1.0, 1.7):
        p, s = _table_weight()
        out[f"dequant_table_gs{gs}"] = dict(kind="dequant", A=ident, packed=p, scale=s, gs=gs, residual=None)
    for i, (N, K, M, gs, res, sigma) in enumerate([
            (64, 512, 1, 1.0, False, 0.02), (64, 512, 1, 1.0, True, 0.02), (40, 1024, 3, 1.0, False, 0.02),
            (40, 1024, 8, 2.5, True, 0.14), (72, 512, 16, 1.0, False, 0.14), (72, 512, 24, 3.0, True, 0.02)]):
        p, s = util.make_weight(N, K, seed=100 + i, sigma=sigma)
        A = util.make_bf16((M, K), seed=200 + i)
        R = util.make_bf16((M, N), seed=300 + i) if res else None
        out[f"linear_{i}_N{N}_K{K}_M{M}"] = dict(kind="linear", A=A, packed=p, scale=s, gs=gs, residual=R)
    p1, s1 = util.make_weight(48, 256, seed=401)
    p2, s2 = util.make_weight(48, 256, seed=402)
    out["dual_N48_K256"] = dict(kind="dual", A=util.make_bf16((1, 256), seed=403), packed=p1, scale=s1, gs=1.0,
                                packed2=p2, scale2=s2, gs2=2.0, residual=None)
    out["swiglu_merged_T3_I136"] = dict(kind="swiglu", merged=util.make_bf16((3, 272), seed=501, std=2.0))
    return out


def oracle_output(c):
    if c["kind"] == "dequant":
        return np.ascontiguousarray(ob.dequant(c["packed"], c["scale"], c["gs"]).T)
    if c["kind"] == "linear":
        return ob.linear(c["A"], c["packed"], c["scale"], c["gs"], residual=c["residual"])
    if c["kind"] == "dual":
        return np.concatenate([ob.linear(c["A"], c["packed"], c["scale"], c["gs"]),
                               ob.linear(c["A"], c["packed2"], c["scale2"], c["gs2"])], axis=1)
    if c["kind"] == "swiglu":
        return ob.swiglu_merged(c["merged"])
    raise ValueError(c["kind"])


def reference_output(c):
    """Runs the reference's kernels; needs a GPU and oracle/_ref."""
    import torch
    ref = ob.load_ref()
    s = torch.cuda.current_stream().cuda_stream
    if c["kind"] == "swiglu":
        T, I = c["merged"].shape[0], c["merged"].shape[1] // 2
        x = util.to_dev(c["merged"])
        o = torch.zeros(T, I, dtype=torch.int16, device="cuda")
        ref.ref_swiglu_merged(o.data_ptr(), x.data_ptr(), T, I, s)
        torch.cuda.synchronize()
        return util.to_host_u16(o)
    A, p, sc = util.to_dev(c["A"]), util.to_dev(c["packed"]), util.to_dev(c["scale"])
    M, K = c["A"].shape
    N = c["packed"].shape[0]
    if c["kind"] == "dual":
        p2, s2 = util.to_dev(c["packed2"]), util.to_dev(c["scale2"])
        o1 = torch.zeros(1, N, dtype=torch.int16, device="cuda")
        o2 = torch.zeros(1, N, dtype=torch.int16, device="cuda")
        ref.ref_fp4_dual_gemv(A.data_ptr(), p.data_ptr(), sc.data_ptr(), c["gs"], p2.data_ptr(), s2.data_ptr(),
                              c["gs2"], N, K, o1.data_ptr(), o2.data_ptr(), s)
        torch.cuda.synchronize()
        return np.concatenate([util.to_host_u16(o1), util.to_host_u16(o2)], axis=1)
    o = torch.zeros(M, N, dtype=torch.int16, device="cuda")
    if c["residual"] is not None:
        o.copy_(util.to_dev(c["residual"]))   # in place, as the reference's callers do (layer.cu:102-104)
        if M == 1:
            ref.ref_fp4_gemv_add(A.data_ptr(), p.data_ptr(), sc.data_ptr(), c["gs"], N, K, o.data_ptr(),
                                 o.data_ptr(), s)
        else:
            ref.ref_fp4_gemm_add(A.data_ptr(), p.data_ptr(), sc.data_ptr(), c["gs"], N, K, o.data_ptr(),
                                 o.data_ptr(), M, s)
    elif M == 1:
        ref.ref_fp4_gemv(A.data_ptr(), p.data_ptr(), sc.data_ptr(), c["gs"], N, K, o.data_ptr(), s)
    else:
        ref.ref_fp4_gemm(A.data_ptr(), p.data_ptr(), sc.data_ptr(), c["gs"], N, K, o.data_ptr(), M, s)
    torch.cuda.synchronize()
    return util.to_host_u16(o)


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_b200.npz")
    res = {}
    worst = 0.0
    for name, c in cases().items():
        res[name] = reference_output(c)
        want = oracle_output(c)
        err = ob.rel_frobenius(want, res[name])
        worst = max(worst, err)
        print(f"{name}: shape {res[name].shape} oracle-vs-reference relF {err:.3e} "
              f"bitwise_equal {bool(np.array_equal(want, res[name]))} max_ulp {util.bf16_ulp_diff(want, res[name])}")
    np.savez_compressed(out, **res)
    print(f"wrote {out} ({os.path.getsize(out)} bytes), worst relF {worst:.3e}")


if __name__ == "__main__":
    main()
