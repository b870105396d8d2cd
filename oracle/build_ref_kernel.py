"""Build the reference's own mma.sync FlashAttention-2 forward extension for sm_100, as an on-box
GPU baseline.  TEST / MEASUREMENT INFRASTRUCTURE ONLY: nothing in the product imports the result.

    python oracle/build_ref_kernel.py /path/to/Mini-Attention

Sources are compiled where they lie in the reference checkout
(kernels/flash_attn/cuda/sm_120/kernel/flash_attention.cu + include/, the newest kernel tree) with
the reference's own nvcc flags (kernels/flash_attn/cuda/sm_120/_bench_sm120.py:36-49) except for
the target architecture, which becomes compute_100 / sm_100.  Nothing is copied: only the built
extension is written, to oracle/_ref/ref_flash_sm100.so (git-ignored).  The build instantiates 133
kernels and takes several minutes.  bench.py --workload c2 times it beside the product kernel when
the file is present (key ``reference_kernel_on_this_gpu``).
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
NAME = "ref_flash_sm100"


def build(ref_root: Path) -> Path:
    from torch.utils.cpp_extension import load
    src = ref_root / "kernels/flash_attn/cuda/sm_120/kernel"
    build_dir = OUT_DIR / "build"
    build_dir.mkdir(parents=True, exist_ok=True)
    flags = ["-std=c++20", "--use_fast_math", "--expt-relaxed-constexpr",
             "-gencode", "arch=compute_100,code=sm_100", "-O3",
             "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
             "-U__CUDA_NO_HALF2_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__"]
    load(name=NAME, sources=[str(src / "flash_attention.cu")], extra_include_paths=[str(src / "include")],
         extra_cuda_cflags=flags, extra_cflags=["-O3"], build_directory=str(build_dir), verbose=False)
    out = OUT_DIR / f"{NAME}.so"
    shutil.copy2(build_dir / f"{NAME}.so", out)
    return out


def load_built():
    """Import oracle/_ref/ref_flash_sm100.so if it exists (returns None otherwise)."""
    import importlib.util
    so = OUT_DIR / f"{NAME}.so"
    if not so.exists():
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/build_ref_kernel.py /path/to/Mini-Attention")
    print(build(Path(sys.argv[1])))
