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

``stage_nanolab()`` puts the reference's ``nanolab`` Python package (the caller of this
path: ``mixers.py``, ``model.py``, ``config.py``, ``optim.py``, ``bench_gpu.py`` and what they
import) beside it as ``oracle/_ref/nanolab/`` -- a git-ignored staging copy, like the built
module, so that the drop-in tests and the whole-model benchmark can run nanolab's own code,
unmodified, on a machine that has no reference checkout.  ``nanolab_on_path()`` makes it
importable.
"""
from __future__ import annotations

import pathlib
import subprocess
import sys
import sysconfig

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref" / "nanolab_flash_attn.so"
STAGED = HERE / "_ref" / "nanolab"
# the modules the attention caller imports, directly or not (nanolab/model.py:22-23,
# nanolab/bench_gpu.py:24-27); flash_cuda.py is staged too, as the module this package replaces
NANOLAB_MODULES = ("__init__", "config", "mixers", "model", "optim", "utils", "bench_gpu", "flash_cuda",
                   "schedules", "data", "diffusion", "bench_modes")


def _reference_root(ref_root: str | None) -> pathlib.Path:
    return pathlib.Path(ref_root) if ref_root else HERE.parent.parent / "reference"


def stage_nanolab(ref_root: str | None = None) -> pathlib.Path | None:
    """Copy the reference's nanolab modules into ``oracle/_ref/nanolab/`` (no-op without a checkout)."""
    import shutil
    src = _reference_root(ref_root) / "nanolab"
    if not (src / "mixers.py").exists():
        return STAGED if (STAGED / "mixers.py").exists() else None
    STAGED.mkdir(parents=True, exist_ok=True)
    for name in NANOLAB_MODULES:
        f = src / f"{name}.py"
        dst = STAGED / f.name
        if f.exists() and (not dst.exists() or dst.stat().st_mtime < f.stat().st_mtime):
            shutil.copyfile(f, dst)
    return STAGED


def nanolab_on_path() -> bool:
    """Put the staged package's parent on ``sys.path``; False when nothing is staged."""
    if not (STAGED / "mixers.py").exists():
        return False
    parent = str(STAGED.parent)
    if parent not in sys.path:
        sys.path.insert(0, parent)
    return True


def build(ref_root: str | None = None, force: bool = False) -> pathlib.Path | None:
    root = _reference_root(ref_root)
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
    print(stage_nanolab(args[0] if args else None))
