"""CPU tests of the drop-in boundary: the shared library loads and exports every symbol the
public headers declare; without a GPU the entry points fail loudly instead of falling back."""
import ctypes
import glob
import os
import re

import pytest

import nvfp4

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header=None):
    """Function names declared in include/<header> (all headers when None)."""
    names = set()
    for path in glob.glob(os.path.join(ROOT, "include", header or "*.h")):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", text))
    return names


def libs():
    out = [nvfp4.load()]
    for name in ("libnvfp4_b200_tp.so", "libnvfp4_ckpt.so"):
        path = os.path.join(os.path.dirname(nvfp4.LIB_PATH), name)
        if os.path.exists(path):
            try:
                out.append(ctypes.CDLL(path))
            except OSError:
                pass
    return out


def test_library_exports_every_declared_symbol():
    loaded = libs()
    decl = declared_symbols()
    assert len(decl) >= 20
    assert len(loaded) == 3, "the tensor-parallel and the checkpoint library must be built"
    for name in sorted(decl):
        assert any(hasattr(l, name) for l in loaded), f"{name} declared in include/ but not exported"


def test_binding_covers_header():
    import nvfp4_ckpt
    import nvfp4_tp
    core = declared_symbols("nvfp4_b200.h")
    assert core == set(nvfp4.SIGNATURES), core ^ set(nvfp4.SIGNATURES)
    tp = declared_symbols("nvfp4_b200_tp.h")
    assert tp == set(nvfp4_tp.TP_SIGNATURES), tp ^ set(nvfp4_tp.TP_SIGNATURES)
    ck = declared_symbols("nvfp4_checkpoint.h")
    assert ck == set(nvfp4_ckpt.CKPT_SIGNATURES), ck ^ set(nvfp4_ckpt.CKPT_SIGNATURES)


def test_quantized_weight_layout():
    qw = nvfp4.QuantizedWeight
    assert ctypes.sizeof(qw) == 32
    assert [getattr(qw, f).offset for f in ("packed", "scale", "global_scale", "input_scale", "N", "K")] == \
        [0, 8, 16, 20, 24, 28]


def test_no_cpu_fallback_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is for GPU-less hosts")
    with pytest.raises(nvfp4.Nvfp4Error) as e:
        nvfp4.Handle(0, 1 << 20)
    assert e.value.status == -7
    lib = nvfp4.load()
    assert lib.nvfp4_status_string(-7).decode().startswith("no usable CUDA device")
    # the reference-shaped entry points record the failure instead of computing anything
    qw = nvfp4.QuantizedWeight(None, None, 1.0, 1.0, 16, 16)
    lib.nvfp4_invoke_fp4_gemv(None, ctypes.byref(qw), None, None)
    assert lib.nvfp4_last_status() != 0


def test_workspace_query_and_null_checks():
    lib = nvfp4.load()
    n = ctypes.c_size_t()
    assert lib.nvfp4_workspace_bytes(16, 34816, 5120, ctypes.byref(n)) == 0 and n.value >= 4 << 20
    assert lib.nvfp4_workspace_bytes(16, 0, 5120, ctypes.byref(n)) == -2
    assert lib.nvfp4_linear(None, None, 1, None, None, 1.0, 16, 16, None, None, None) == -1
    assert lib.nvfp4_destroy(None) == -1
    assert lib.nvfp4_scan_scales(None, None, 16, 16, None, None) == -1


def test_no_cluster_multicast_anywhere():
    """No source file may carry a TMA / bulk load with the cluster-wide broadcast qualifier."""
    pat = re.compile("multi" + "cast" + "::" + "cluster")
    for ext in ("cu", "cuh", "h", "hpp", "cpp", "py"):
        for path in glob.glob(os.path.join(ROOT, "**", f"*.{ext}"), recursive=True):
            rel = os.path.relpath(path, ROOT)
            if rel.split(os.sep)[0].startswith(("_", "gpu", "baseline")) or path.endswith("test_abi_cpu.py"):   # scratch folders are not shipped
                continue
            assert not pat.search(open(path, errors="ignore").read()), path


def test_reference_namespace_shim_compiles_and_links(tmp_path):
    """A translation unit written against the reference's own operator names compiles against the
    shim header and links the library; without a GPU the call records an error status."""
    import shutil
    import subprocess
    if not shutil.which("nvcc"):
        pytest.skip("nvcc not on PATH")
    src = tmp_path / "shim_check.cu"
    ref_engine = os.path.join(os.environ.get("REF_ROOT", os.path.join(os.path.dirname(ROOT), "reference")), "src", "engine")
    have_ref = os.path.exists(os.path.join(ref_engine, "layer.h"))
    src.write_text('''
#include <cstdint>
#ifdef NVFP4_TEST_REF_LAYER_H
#include "layer.h"                       // the reference's own definition (src/engine/layer.h:197-204)
#else
namespace qwen_thor { namespace core {   // stand-in with the same members, for hosts without the reference tree
struct QuantizedWeight { uint8_t* packed = nullptr; uint8_t* scale = nullptr; float global_scale = 1.0f;
                         float input_scale = 1.0f; int N = 0, K = 0; bool valid() const { return packed != nullptr; } };
}}
#endif
#include <cstddef>
#include "nvfp4_qwen_thor_shim.hpp"
static_assert(offsetof(qwen_thor::core::QuantizedWeight, packed) == offsetof(nvfp4_quantized_weight, packed), "layout");
static_assert(offsetof(qwen_thor::core::QuantizedWeight, scale) == offsetof(nvfp4_quantized_weight, scale), "layout");
static_assert(offsetof(qwen_thor::core::QuantizedWeight, global_scale) == offsetof(nvfp4_quantized_weight, global_scale), "layout");
static_assert(offsetof(qwen_thor::core::QuantizedWeight, input_scale) == offsetof(nvfp4_quantized_weight, input_scale), "layout");
static_assert(offsetof(qwen_thor::core::QuantizedWeight, N) == offsetof(nvfp4_quantized_weight, N), "layout");
static_assert(offsetof(qwen_thor::core::QuantizedWeight, K) == offsetof(nvfp4_quantized_weight, K), "layout");
static_assert(sizeof(qwen_thor::core::QuantizedWeight) == sizeof(nvfp4_quantized_weight), "layout");
int main() {
    qwen_thor::core::QuantizedWeight w;
    qwen_thor::ops::invoke_fp4_gemv(nullptr, w, nullptr);
    qwen_thor::ops::invoke_fp4_gemm_add(nullptr, w, nullptr, nullptr, 4);
    return nvfp4_last_status() == 0 ? 0 : 3;
}
''')
    lib_dir = os.path.dirname(nvfp4.LIB_PATH)
    exe = tmp_path / "shim_check"
    extra = ["-DNVFP4_TEST_REF_LAYER_H", "-I", ref_engine] if have_ref else []
    subprocess.run(["nvcc", "-std=c++17", "-Wno-deprecated-gpu-targets", "-I", os.path.join(ROOT, "qwen3-27b-thor-runner_b200", "include")]
                   + extra + ["-o", str(exe), str(src), "-L", lib_dir, "-lnvfp4_b200", "-Xlinker", "-rpath", "-Xlinker", lib_dir],
                   check=True, capture_output=True)
    rc = subprocess.run([str(exe)]).returncode
    assert rc == 3    # null pointers / no device: the call is refused and the status says so


def test_reference_struct_size_as_the_reference_compiler_sees_it():
    """sizeof(QuantizedWeight) as compiled from the reference's own layer.h (through the bridge that
    includes it) equals the C struct of the ABI."""
    import oracle_binding as ob
    if not ob.ref_available():
        pytest.skip("oracle/_ref not built")
    import ctypes
    ref = ctypes.CDLL(ob.REF_LIB)
    ref.ref_sizeof_quantized_weight.restype = ctypes.c_int
    assert ref.ref_sizeof_quantized_weight() == ctypes.sizeof(nvfp4.QuantizedWeight) == 32
