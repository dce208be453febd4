import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = pathlib.Path(__file__).parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 patterns -> exact float32 values."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def load_golden(path):
    d = np.load(path)
    B, T, H, Hkv, D, window, sinks = (int(x) for x in d["meta"][:7])
    block = int(d["meta"][7]) if len(d["meta"]) > 7 else 0           # block-causal fixtures carry their block length
    case = dict(name=pathlib.Path(path).stem, B=B, T=T, H=H, Hkv=Hkv, D=D,
                window=window, sinks=sinks, block=block, scale=float(d["scale"]))
    for key in ("q", "k", "v", "dout"):
        case[key] = bf16_bits_to_f32(d[key])
    for key in ("o", "lse", "dq", "dk", "dv"):
        case[key] = d[key]
    return case


def golden_paths():
    """The attention fixtures (the whole-model and prologue fixtures have their own loaders)."""
    return sorted([*GOLDEN.glob("causal_*.npz"), *GOLDEN.glob("swa_*.npz"), *GOLDEN.glob("blockcausal_*.npz")])


@pytest.fixture(params=golden_paths(), ids=lambda p: p.stem)
def golden(request):
    return load_golden(request.param)
