"""TEST INFRASTRUCTURE -- compiles the reference's own CUDA kernel as a comparison arm.

    python oracle/build_ref.py [/path/to/reference]      # -> oracle/_ref/nanolab_flash_attn.so

Without an argument the reference checkout is looked for beside this repository (a sibling
directory named ``reference``).

The reference's single CUDA source (``nanolab/csrc/flash_attn_cuda.cu``) is compiled where
it lies, with one direct nvcc command (no ninja, none of the reference's own build code),
into a Python extension module under ``oracle/_ref/`` (git-ignored; it travels to the GPU
box as a built file).  Nothing of the reference is copied into this repository.  The flags
are the ones ``torch.utils.cpp_extension`` passes for the reference's own JIT build
(``nanolab/flash_cuda.py:113-124``: ``-O3 -lineinfo``, no fast math).

Only the tests and the self-check table use the result, as a checker and a same-box
baseline; the product never loads it.  Takes about five minutes on eight cores.
"""
from __future__ import annotations

import pathlib
import subprocess
import sys
import sysconfig

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref" / "nanolab_flash_attn.so"


def build(ref_root: str | None = None, force: bool = False) -> pathlib.Path | None:
    root = pathlib.Path(ref_root) if ref_root else HERE.parent.parent / "reference"
    src = root / "nanolab" / "csrc" / "flash_attn_cuda.cu"
    if not src.exists():
        return OUT if OUT.exists() else None
    if OUT.exists() and not force and OUT.stat().st_mtime >= src.stat().st_mtime:
        return OUT
    import torch
    from torch.utils import cpp_extension as ce
    OUT.parent.mkdir(exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    lib = pathlib.Path(torch.__file__).parent / "lib"
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-shared",
           "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
           "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_BFLOAT16_CONVERSIONS__",
           "-D__CUDA_NO_HALF2_OPERATORS__", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-DTORCH_EXTENSION_NAME=nanolab_flash_attn", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, str(src), "-o", str(OUT), f"-L{lib}", f"-Xlinker=-rpath={lib}",
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"reference kernel did not compile:\n{r.stderr[-4000:]}")
    return OUT


def load():
    """The compiled module (``fwd``, ``bwd``, ``mma_probe``), or None when it was never built."""
    if not OUT.exists():
        return None
    import importlib.util
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location("nanolab_flash_attn", OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args[0] if args else None, force="--force" in sys.argv))
