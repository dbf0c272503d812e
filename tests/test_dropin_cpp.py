"""The C++ drop-in (libsd_b200.so: sd::qgemm, sd::quantize_rowwise, sd::load_sdcpp, sd::matmul,
sd::blk::sdpa, Tensor)
exercised by a standalone C++ test binary written like the reference's own tests."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "self-evolve-diffusion-cpp_b200", "test_dropin")
GOLDEN = os.path.join(ROOT, "tests", "golden")


def _run(*args):
    assert os.path.exists(BIN), "build with __graft_entry__.build() first"
    return subprocess.run([BIN, *args], capture_output=True, text=True, timeout=600)


def test_dropin_host_part():
    r = _run("--cpu", GOLDEN)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout


@pytest.mark.gpu
def test_dropin_on_gpu():
    r = _run(GOLDEN)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout and "cosine" in r.stdout


def test_tensor_layout_matches_reference_header(tmp_path):
    """Where the reference tree is mounted: sd::Tensor here and there have the same layout,
    so objects compiled against the reference's header can link against this library."""
    from util import reference_tree
    ref = reference_tree()
    if not os.path.exists(os.path.join(ref, "src/core/tensor.h")):
        pytest.skip("reference tree not mounted")
    src = tmp_path / "layout.cpp"
    src.write_text(
        '#include <cstddef>\n'
        '#define sd sd_ref\n#include "%s/src/core/tensor.h"\n#undef sd\n'
        '#include "core/tensor.h"\n'
        'static_assert(sizeof(sd::Tensor) == sizeof(sd_ref::Tensor), "size");\n'
        'static_assert(offsetof(sd::Tensor, dtype) == offsetof(sd_ref::Tensor, dtype), "dtype");\n'
        'static_assert(offsetof(sd::Tensor, data) == offsetof(sd_ref::Tensor, data), "data");\n'
        'static_assert(offsetof(sd::Tensor, nbytes) == offsetof(sd_ref::Tensor, nbytes), "nbytes");\n'
        'static_assert(offsetof(sd::Tensor, owning) == offsetof(sd_ref::Tensor, owning), "owning");\n'
        'static_assert((int)sd::DType::I8 == (int)sd_ref::DType::I8 && (int)sd::DType::BF16 == (int)sd_ref::DType::BF16, "enum");\n'
        'int main() { return 0; }\n' % ref)
    inc = os.path.join(ROOT, "self-evolve-diffusion-cpp_b200", "csrc", "sd_dropin")
    r = subprocess.run(["g++", "-std=c++17", "-Wno-invalid-offsetof", "-fsyntax-only", "-I", inc, str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_dropin_exports_reference_symbols():
    """The mangled names a caller compiled against the reference's headers would look up."""
    so = os.path.join(ROOT, "self-evolve-diffusion-cpp_b200", "libsd_b200.so")
    out = subprocess.run(["nm", "-DC", "--defined-only", so], capture_output=True, text=True).stdout
    for sym in ("sd::qgemm(sd::Tensor const&, sd::Tensor const&, sd::Tensor const&, sd::Tensor&)",
                "sd::quantize_rowwise(sd::Tensor const&, sd::Tensor&, sd::Tensor&)",
                "sd::load_sdcpp(", "sd::parallel_for(", "sd::set_nthreads(int)", "sd::nthreads()",
                "sd::to_bf16(sd::Tensor const&, sd::Tensor&)", "sd::Tensor::reshape(",
                "sd::matmul(sd::Tensor const&, sd::Tensor const&, sd::Tensor&, float const*)",
                "sd::blk::sdpa(sd::Tensor const&, sd::Tensor const&, sd::Tensor const&, int, sd::Tensor&, bool)"):
        assert sym in out, sym
