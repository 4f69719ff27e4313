"""Builds a TRIMMED copy of the reference's CUDA extension `flash_sparse_attn_cuda` for sm_100 into baseline/_ref/
(git-ignored), so that the reference's own kernels can be timed on a B200 next to this library's.

What is compiled, straight from the reference checkout (nothing is copied into this repository):
  * csrc/flash_sparse_attn/flash_api.cpp (the pybind module: `fwd`, `bwd`, ...);
  * the forward and backward instantiations for bf16, head dim 128, causal, has_mask, has_bias
    (src/instantiations/flash_{fwd,bwd}_hdim128_bf16_causal_has_mask_has_bias_sm80.cu) -- the only ones the
    comparison calls;
  * a generated stub file that defines every OTHER `run_mha_fwd_` / `run_mha_fwd_splitkv_dispatch` / `run_mha_bwd_`
    specialisation flash_api.cpp refers to (setup.py builds 288 files of about two minutes each) as a function that
    raises.
CUTLASS: the reference expects its `csrc/cutlass` submodule, which is empty in the checkout; the CUTLASS headers
shipped inside the flashinfer wheel of this image are used instead.

    python baseline/build_ref_cuda.py [--reference <reference checkout>]

Needs nvcc and torch, no GPU. Output: baseline/_ref/flash_sparse_attn_cuda*.so next to the reference's Python
package (installed there with pip, FLASH_SPARSE_ATTENTION_SKIP_CUDA_BUILD=TRUE)."""
import argparse
import itertools
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUT = os.path.join(ROOT, "baseline", "_ref")
KEEP = ("bf16", 128, True, True, True)  # dtype, head dim, causal, has_mask, has_bias


def stub_source() -> str:
    lines = ['#include <c10/util/Exception.h>', '#include <cutlass/numeric_types.h>', '#include "namespace_config.h"',
             '#include "flash.h"', "namespace FLASH_NAMESPACE {"]
    ctype = {"bf16": "cutlass::bfloat16_t", "fp16": "cutlass::half_t"}
    for dt, hd, ca, hm, hb in itertools.product(("bf16", "fp16"), (32, 64, 96, 128, 192, 256), (False, True),
                                                 (False, True), (False, True)):
        args = f"{ctype[dt]}, {hd}, {str(ca).lower()}, {str(hm).lower()}, {str(hb).lower()}"
        msg = f'"this trimmed build only holds bf16 / head dim 128 / causal / mask / bias ({dt} {hd} {ca} {hm} {hb} asked)"'
        kinds = [("run_mha_fwd_splitkv_dispatch", "Flash_fwd_params")]
        if (dt, hd, ca, hm, hb) != KEEP:
            kinds += [("run_mha_fwd_", "Flash_fwd_params"), ("run_mha_bwd_", "Flash_bwd_params")]
        for fn, ptype in kinds:
            lines.append(f"template<> void {fn}<{args}>({ptype} &params, cudaStream_t stream) {{ TORCH_CHECK(false, {msg}); }}")
    lines.append("}  // namespace FLASH_NAMESPACE")
    return "\n".join(lines) + "\n"


def install_python_layer(reference: str, cutlass: str) -> None:
    """pip-installs the reference's Python package (no CUDA build) into baseline/_ref from a temporary copy of the
    checkout: its setup.py insists on csrc/cutlass/include being present, so the copy gets a link to the headers."""
    import subprocess
    import tempfile

    if os.path.isdir(os.path.join(OUT, "flash_sparse_attn")):
        return
    with tempfile.TemporaryDirectory() as tmp:
        copy = os.path.join(tmp, "ref")
        shutil.copytree(reference, copy, symlinks=True, ignore=shutil.ignore_patterns(".git"))
        os.makedirs(os.path.join(copy, "csrc", "cutlass"), exist_ok=True)
        link = os.path.join(copy, "csrc", "cutlass", "include")
        if not os.path.exists(link):
            os.symlink(cutlass, link)
        env = dict(os.environ, FLASH_SPARSE_ATTENTION_SKIP_CUDA_BUILD="TRUE")
        subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                        "--find-links", "/opt/wheelhouse", "--target", OUT, copy], check=True, env=env)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    args = ap.parse_args()
    import flashinfer
    from torch.utils import cpp_extension

    cutlass = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass", "include")
    os.makedirs(OUT, exist_ok=True)
    install_python_layer(args.reference, cutlass)
    src = os.path.join(args.reference, "csrc", "flash_sparse_attn")
    inst = os.path.join(src, "src", "instantiations")
    build = os.path.join(OUT, "build_cuda_ext")
    os.makedirs(build, exist_ok=True)
    stub = os.path.join(build, "stubs_generated.cu")
    with open(stub, "w") as f:
        f.write(stub_source())
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    cpp_extension.load(
        name="flash_sparse_attn_cuda",
        sources=[os.path.join(src, "flash_api.cpp"),
                 os.path.join(inst, "flash_fwd_hdim128_bf16_causal_has_mask_has_bias_sm80.cu"),
                 os.path.join(inst, "flash_bwd_hdim128_bf16_causal_has_mask_has_bias_sm80.cu"), stub],
        extra_include_paths=[src, os.path.join(src, "src"), cutlass],
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=["-O3", "-std=c++17", "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
                           "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
                           "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math"],
        build_directory=build, is_python_module=False, verbose=True)
    so = os.path.join(build, "flash_sparse_attn_cuda.so")
    shutil.copy(so, os.path.join(OUT, "flash_sparse_attn_cuda.so"))
    print("built", os.path.join(OUT, "flash_sparse_attn_cuda.so"))


if __name__ == "__main__":
    sys.exit(main())
