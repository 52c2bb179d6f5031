import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


class Golden:
    """Access to tests/golden/layers.npz: whole arrays, or (idx, val, sum, sumsq) samples of big ones."""

    def __init__(self):
        self.z = np.load(ROOT / "tests" / "golden" / "layers.npz")

    def has_full(self, case, key):
        return f"{case}/{key}" in self.z.files

    def full(self, case, key):
        return self.z[f"{case}/{key}"]

    def sample(self, case, key):
        p = f"{case}/{key}"
        return self.z[p + ".idx"], self.z[p + ".val"], float(self.z[p + ".sum"]), float(self.z[p + ".sumsq"])

    def pair(self, case, key, got):
        """(got restricted to the stored positions, stored reference values) as float64 torch tensors."""
        import torch
        if isinstance(got, torch.Tensor):
            got = got.detach().cpu().numpy()
        flat = np.asarray(got, dtype=np.float64).reshape(-1)
        if self.has_full(case, key):
            want = self.full(case, key).astype(np.float64).reshape(-1)
            assert want.size == flat.size, f"{case}/{key}: {flat.size} values vs {want.size}"
            return torch.from_numpy(flat), torch.from_numpy(want)
        idx, val, _, _ = self.sample(case, key)
        return torch.from_numpy(flat[idx]), torch.from_numpy(val.astype(np.float64))

    def check(self, case, key, got, rel=1e-5, abs_=1e-4):
        """Compare `got` (numpy or torch, any device) with the stored reference output.
        Returns (ok, max_abs_err, message)."""
        import torch
        if isinstance(got, torch.Tensor):
            got = got.detach().cpu().numpy()
        got = np.asarray(got, dtype=np.float64)
        if self.has_full(case, key):
            want = self.full(case, key).astype(np.float64)
            if want.shape != got.shape:
                return False, float("inf"), f"{case}/{key}: shape {got.shape} vs {want.shape}"
            err = np.abs(got - want)
            ok = bool(np.all(err <= abs_ + rel * np.abs(want))) and bool(np.all(np.isfinite(got)))
            worst = float(err.max()) if err.size else 0.0
            return ok, worst, f"{case}/{key}: max_abs_err={worst:.3e} over {want.size} values"
        idx, val, s1, s2 = self.sample(case, key)
        flat = got.reshape(-1)
        err = np.abs(flat[idx] - val.astype(np.float64))
        ok = bool(np.all(err <= abs_ + rel * np.abs(val))) and bool(np.all(np.isfinite(flat)))
        # checksums over the whole tensor: sum within n * tolerance-per-element, energy within rel
        n = flat.size
        sum_ok = abs(flat.sum() - s1) <= n * 0.0 + np.sqrt(n) * (abs_ + rel * np.sqrt(s2 / n)) * 4
        sq_ok = abs((flat ** 2).sum() - s2) <= 1e-4 * max(s2, 1e-30)
        worst = float(err.max())
        return ok and sum_ok and sq_ok, worst, (f"{case}/{key}: max_abs_err={worst:.3e} on {idx.size} samples, "
                                                 f"sum {flat.sum():.6e} vs {s1:.6e}, sumsq {(flat ** 2).sum():.6e} vs {s2:.6e}")


@pytest.fixture(scope="session")
def golden():
    return Golden()


@pytest.fixture(scope="session", autouse=True)
def _no_bounded_wait_ran_out():
    """Kernels that wait for the copy engine poll a bounded number of times and set a device flag when they
    give up.  After a GPU test session the flag must still be clear."""
    yield
    try:
        import torch
        if not torch.cuda.is_available():
            return
    except ImportError:
        return
    from addernetcuda_b200 import _lib
    assert _lib.device_status(reset=True) == 0, "a kernel's bounded wait for a bulk copy ran out during the tests"
