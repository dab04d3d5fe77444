"""Shared fixtures. Tests that need a GPU carry `@pytest.mark.gpu`; everything
else runs on the host (oracle vs golden vectors, host logic, C-ABI symbols)."""

import glob
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def _from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


class GoldenCase:
    """One reference-generated vector set (see tests/golden/make_golden.py)."""

    def __init__(self, path: str):
        z = np.load(path)
        self.name = os.path.basename(path)[:-4]
        self.q, self.k, self.v = (_from_bits(z[n]) for n in ("q", "k", "v"))
        bs, top_k, hkv, always, incl, low = (int(x) for x in z["meta"])
        self.block_size, self.top_k, self.hkv = bs, top_k, hkv
        self.always_current, self.includes_current = bool(always), bool(incl)
        self.low_dtype = torch.bfloat16 if low else torch.float32
        shape = tuple(int(x) for x in z["mask_shape"])
        n = int(np.prod(shape))
        self.mask = torch.from_numpy(np.unpackbits(z["mask"])[:n].astype(bool).reshape(shape))
        self.out = torch.from_numpy(z["out"])
        self.out_low = _from_bits(z["out_low"]) if "out_low" in z else None
        self.has_grads = "dq" in z
        if self.has_grads:
            self.do = _from_bits(z["do"])
            self.dq, self.dk, self.dv = (torch.from_numpy(z[n]) for n in ("dq", "dk", "dv"))
        cu = z["cu"]
        self.cu = torch.from_numpy(cu.astype(np.int32)) if cu.size else None
        self.max_seqlen = int((cu[1:] - cu[:-1]).max()) if cu.size else None

    @property
    def slots(self) -> int:
        seed = 1 if self.always_current else 0
        return self.top_k - (1 if (seed and self.includes_current) else 0) + seed

    def config(self):
        from moba_triton_b200 import MoBAConfig
        return MoBAConfig(block_size=self.block_size, top_k=self.top_k, dtype=self.low_dtype,
                          always_select_current=self.always_current,
                          top_k_includes_current=self.includes_current)


def golden_paths():
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def golden_ids():
    return [os.path.basename(p)[:-4] for p in golden_paths()]


@pytest.fixture(params=golden_paths(), ids=golden_ids())
def golden(request) -> GoldenCase:
    return GoldenCase(request.param)


@pytest.fixture(scope="session")
def device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


def make_qkv(shape, hkv=None, dtype=torch.float32, seed=0, with_do=False):
    """Seeded inputs from a CPU generator (q, k, v[, dO]); bfloat16-representable
    values so the same numbers replay in every precision."""
    g = torch.Generator().manual_seed(seed)
    b, s, hq, d = shape
    hkv = hq if hkv is None else hkv
    q = torch.randn(shape, generator=g).to(torch.bfloat16)
    k = torch.randn((b, s, hkv, d), generator=g).to(torch.bfloat16)
    v = torch.randn((b, s, hkv, d), generator=g).to(torch.bfloat16)
    out = [q.to(dtype), k.to(dtype), v.to(dtype)]
    if with_do:
        out.append((torch.randn(shape, generator=g) * 0.1).to(torch.bfloat16).to(dtype))
    return tuple(out)


@pytest.fixture(autouse=True)
def _device_error_word_stays_clear(request):
    """After every GPU test: no kernel may have reported a bounded wait giving up."""
    yield
    if request.node.get_closest_marker("gpu") is not None and torch.cuda.is_available():
        from moba_triton_b200 import _lib
        word = _lib.device_status()
        assert word == 0, f"a tensor-core kernel reported an error (status word {word:#x})"
