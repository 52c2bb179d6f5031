"""Shared rules for whole-network parity tests (logits, loss and gradients of one training step).

Plain rule everywhere: |got - want| <= 1e-4 + 1e-5 * |want| against the reference's float32 result.
A gradient tensor that misses it is judged by its distance to EXACT arithmetic instead: the fixtures
hold the same step evaluated in float64, so

    err(got, float64) <= 2 * err(reference_float32, float64) + 1e-4 + 1e-5 * |float64|

says "at least as close to the truth as the reference itself, up to a factor of two".  (A few weight
gradients of late layers are tiny sums of large terms that the norm rescale of adder.py:78 then blows
up; the reference's own float32 result is 1e-3 away from the float64 one there.)
"""
from __future__ import annotations

import numpy as np
import torch

from oracle import adder_oracle as O


def _np(t):
    if isinstance(t, torch.Tensor):
        t = t.detach().to("cpu", torch.float64).numpy()
    return np.asarray(t, dtype=np.float64)


def grad_ok(name, got, want32, want64):
    """Returns (ok, used_float64_anchor, message) for one gradient tensor (or sample of one)."""
    got, want32, want64 = _np(got).reshape(-1), _np(want32).reshape(-1), _np(want64).reshape(-1)
    err = np.abs(got - want32)
    worst = float(err.max()) if err.size else 0.0
    if bool(np.all(err <= 1e-4 + 1e-5 * np.abs(want32))) and bool(np.all(np.isfinite(got))):
        return True, False, f"{name}: max_abs_err={worst:.3e} ok"
    e_got = float(np.abs(got - want64).max())
    e_ref = float(np.abs(want32 - want64).max())
    bound = 2.0 * e_ref + 1e-4 + 1e-5 * float(np.abs(want64).max())
    ok = bool(np.all(np.isfinite(got))) and e_got <= bound
    return ok, True, (f"{name}: vs float32 reference {worst:.3e}; vs float64: ours {e_got:.3e}, "
                      f"reference's {e_ref:.3e}, bound {bound:.3e} {'ok' if ok else 'FAIL'}")


def check_step(z, logits, loss, named_grads, sampled: bool, max_anchored: int, log=print):
    """Compare one training step with a fixture `z` (np.load of tests/golden/<net>_b<batch>.npz).
    `sampled`: the fixture holds `grad/<k>.idx/.val` samples instead of whole tensors."""
    ok, worst, msg = O.compare("logits", logits, torch.from_numpy(z["logits"]))
    log("   ", msg)
    assert ok, msg
    want_loss = float(z["loss"])
    assert abs(float(loss) - want_loss) <= 1e-4 + 1e-5 * abs(want_loss), (float(loss), want_loss)
    failures, anchored, worst_name, worst_err, n = [], [], None, -1.0, 0
    for k, g in named_grads:
        n += 1
        if sampled:
            idx = z[f"grad/{k}.idx"]
            got = _np(g).reshape(-1)[idx]
            w32, w64 = z[f"grad/{k}.val"], z[f"grad64/{k}.val"]
            assert bool(torch.isfinite(g).all()), k
        else:
            got, w32, w64 = g, z["grad/" + k], z["grad64/" + k]
        ok, used64, msg = grad_ok(k, got, w32, w64)
        err = float(np.abs(_np(got).reshape(-1) - _np(w32).reshape(-1)).max())
        if err > worst_err:
            worst_name, worst_err = k, err
        if used64:
            anchored.append(msg)
        if not ok:
            failures.append(msg)
    log(f"    worst gradient tensor: {worst_name} max_abs_err={worst_err:.3e} "
        f"({n} tensors compared; {len(anchored)} judged against the float64 step)")
    for m in anchored:
        log("      ", m)
    assert not failures, "\n".join(failures)
    assert len(anchored) <= max_anchored, anchored
