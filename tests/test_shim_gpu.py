"""The C++ side of the boundary on a GPU: a program written against the reference's operator names
(qwen_thor::ops::invoke_fp4_gemv / _gemv_add / _gemm / _gemm_add, src/engine/dense_gemm_fp4.h:25-72)
runs the reference's MLP sequence (run_mlp, src/engine/layer.cu:62-110) through the shim header
and libnvfp4_b200.so, from C++, with no Python on the data path; its output is compared with the
CPU oracle.  When the reference tree is present the program is compiled against the reference's
own layer.h, so the descriptor it fills is the reference's struct."""
import os
import shutil
import struct
import subprocess

import numpy as np
import pytest

import nvfp4
import oracle_binding as ob
import util

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_ROOT = os.environ.get("REF_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    if not shutil.which("nvcc"):
        pytest.skip("nvcc not on PATH")
    out = tmp_path_factory.mktemp("shim") / "shim_mlp_driver"
    lib_dir = os.path.dirname(nvfp4.LIB_PATH)
    cmd = ["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(ROOT, "qwen3-27b-thor-runner_b200", "include")]
    ref_engine = os.path.join(REF_ROOT, "src", "engine")
    if os.path.exists(os.path.join(ref_engine, "layer.h")):
        cmd += ["-DNVFP4_TEST_REF_LAYER_H", "-I", ref_engine]
    cmd += ["-o", str(out), os.path.join(ROOT, "tests", "cpp", "shim_mlp_driver.cu"), "-L", lib_dir, "-lnvfp4_b200",
            "-Xlinker", "-rpath", "-Xlinker", lib_dir]
    subprocess.run(cmd, check=True, capture_output=True)
    return str(out)


@pytest.mark.parametrize("M,gs_gu,gs_dn", [(1, 1.0, 1.0), (1, 37.5, 2688.0), (4, 1.0, 1.0), (40, 1.0, 1.0)])
def test_run_mlp_sequence_from_cpp(driver, tmp_path, M, gs_gu, gs_dn):
    H, I = 1024, 2304
    gu_p, gu_s = util.make_weight(2 * I, H, seed=91)
    dn_p, dn_s = util.make_weight(H, I, seed=92)
    X, R = util.make_bf16((M, H), seed=93 + M), util.make_bf16((M, H), seed=94 + M)
    src, dst = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(src, "wb") as f:
        f.write(struct.pack("<iiiff", M, H, I, gs_gu, gs_dn))
        for a in (X, R, gu_p, gu_s, dn_p, dn_s):
            f.write(np.ascontiguousarray(a).tobytes())
    rc = subprocess.run([driver, str(src), str(dst)], capture_output=True, text=True)
    assert rc.returncode == 0, (rc.returncode, rc.stderr)
    got = np.fromfile(dst, np.uint16).reshape(M, H)
    want = ob.mlp(X, gu_p, gu_s, gs_gu, dn_p, dn_s, gs_dn, residual=R, mode=ob.GEMV if M <= 16 else ob.GEMM, threads=8)
    assert ob.rel_frobenius(got, want) <= 2e-3        # the SwiGLU between the projections amplifies last-bit differences
