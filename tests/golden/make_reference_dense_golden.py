"""Generates tests/golden/reference_b200_dense.npz: outputs of the REFERENCE engine's own BF16
GEMV kernels (invoke_dense_gemv / invoke_dense_gemv_add of its dense_gemm_sm110.cu, compiled
unmodified for sm_100a into oracle/_ref/libref_dense.so by oracle/Makefile) on seeded inputs,
run on a B200.

    python tests/golden/make_reference_dense_golden.py [out.npz]

The cases reach every kernel of the family: the plain one (K*2 <= 48 KB, K <= 8192), the
scattered one (K > 8192) and the K-tiled one (K*2 > 48 KB), each with and without the residual,
and an N that leaves the last block of the untiled kernel partly empty.
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


def cases():
    out = {}
    # Two defects of the reference's kernels stay outside the cases (found by running it once, then by reading):
    # a K that is not a multiple of 8 misaligns its 16-byte row loads (cudaErrorMisalignedAddress), and in the
    # K-tiled kernels the warps without an output row leave the block before the cooperative load of the
    # activations, so a last block with fewer rows than warps computes on unloaded shared memory (N % 8 != 0).
    for i, (N, K, res) in enumerate([(640, 5120, False), (384, 1024, True), (300, 17408, True), (256, 17408, False),
                                     (136, 25600, True), (64, 25600, False), (37, 2048, True)]):
        out[f"gemv{'_add' if res else ''}_N{N}_K{K}"] = dict(
            A=util.make_bf16((1, K), seed=900 + i), W=util.make_bf16((N, K), seed=950 + i, std=0.05),
            residual=util.make_bf16((1, N), seed=980 + i) if res else None)
    return out


def oracle_output(c):
    return ob.dense_gemv_ref(c["A"], c["W"], residual=c["residual"])


def reference_output(c):
    import torch
    dense = ob.load_ref().dense
    s = torch.cuda.current_stream().cuda_stream
    N, K = c["W"].shape
    A, W = util.to_dev(c["A"]), util.to_dev(c["W"])
    o = torch.zeros(1, N, dtype=torch.int16, device="cuda")
    if c["residual"] is not None:
        r = util.to_dev(c["residual"])
        dense.ref_dense_gemv_add(A.data_ptr(), W.data_ptr(), o.data_ptr(), r.data_ptr(), N, K, s)
    else:
        dense.ref_dense_gemv(A.data_ptr(), W.data_ptr(), o.data_ptr(), N, K, s)
    torch.cuda.synchronize()
    return util.to_host_u16(o)


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_b200_dense.npz")
    res = {}
    for name, c in cases().items():
        got = reference_output(c)
        want = oracle_output(c)
        res[name] = got
        print(f"{name}: oracle-vs-reference bitwise_equal {bool(np.array_equal(got, want))} "
              f"relF {ob.rel_frobenius(want, got):.3e} differing {int((want != got).sum())}/{got.size}")
    np.savez_compressed(out, **res)
    print(f"wrote {out} ({os.path.getsize(out)} bytes)")


if __name__ == "__main__":
    main()
