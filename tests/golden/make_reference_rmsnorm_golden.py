"""Generates tests/golden/reference_b200_rmsnorm.npz: outputs of the REFERENCE engine's own
RMSNorm kernels (rmsnorm_kernel and fused_add_rmsnorm_kernel of its light_ops.cu, compiled
unmodified for sm_100a into oracle/_ref/libref_fp4.so by oracle/Makefile) on seeded inputs,
run on a B200.

    python tests/golden/make_reference_rmsnorm_golden.py [out.npz]

Inputs are rebuilt from seeds by cases().  The reference is built with --use_fast_math
(approximate rsqrtf and division), so the CPU oracle, which uses 1/sqrtf, may differ from
these outputs in the last BF16 bit of a few elements; the tests bound how many.
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

EPS = 1e-6


def cases():
    out = {}
    for i, (T, hs, add) in enumerate([(3, 5120, False), (1, 1024, False), (2, 5120, True), (5, 2048, True)]):
        c = dict(x=util.make_bf16((T, hs), seed=600 + i, std=1.5), w=util.make_bf16((hs,), seed=700 + i, std=0.3), add=add)
        if add:
            c["bias"] = util.make_bf16((T, hs), seed=800 + i, std=0.7)
        out[f"{'add_' if add else ''}rmsnorm_T{T}_hs{hs}"] = c
    return out


def oracle_output(c):
    """{norm, residual}: the normalised rows and, for the fused add, the updated residual."""
    if c["add"]:
        norm, res = ob.rmsnorm(c["x"], c["w"], EPS, bias=c["bias"])
        return norm, res
    return ob.rmsnorm(c["x"], c["w"], EPS), None


def reference_output(c):
    import torch
    ref = ob.load_ref()
    s = torch.cuda.current_stream().cuda_stream
    T, hs = c["x"].shape
    x, w = util.to_dev(c["x"]), util.to_dev(c["w"])
    o = torch.zeros(T, hs, dtype=torch.int16, device="cuda")
    if c["add"]:
        b = util.to_dev(c["bias"])
        ref.ref_fused_add_rmsnorm(o.data_ptr(), x.data_ptr(), b.data_ptr(), w.data_ptr(), EPS, T, hs, s)
        torch.cuda.synchronize()
        return util.to_host_u16(o), util.to_host_u16(x)
    ref.ref_rmsnorm(o.data_ptr(), x.data_ptr(), w.data_ptr(), EPS, T, hs, s)
    torch.cuda.synchronize()
    return util.to_host_u16(o), None


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_b200_rmsnorm.npz")
    res = {}
    for name, c in cases().items():
        norm, resid = reference_output(c)
        want, want_res = oracle_output(c)
        res[name] = norm
        line = (f"{name}: oracle-vs-reference relF {ob.rel_frobenius(want, norm):.3e} differing "
                f"{int((want != norm).sum())}/{norm.size} max_ulp {util.bf16_ulp_diff(want, norm)}")
        if resid is not None:
            res[name + "_residual"] = resid
            line += f" residual bitwise_equal {bool(np.array_equal(want_res, resid))}"
        print(line)
    np.savez_compressed(out, **res)
    print(f"wrote {out} ({os.path.getsize(out)} bytes)")


if __name__ == "__main__":
    main()
