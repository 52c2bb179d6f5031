"""Generates the golden fixtures under tests/golden/ from the UNMODIFIED reference sources.

    python tests/golden/make_golden.py [--reference /path/to/AdderNetCUDA]

Needs the reference checkout (it is not shipped with this repository); needs no GPU.  The
reference's adder.py does `import adder_cuda` unconditionally, so the CPU stand-in
oracle/adder_cuda_cpu.py (the reference's own ground-truth expressions with the extension's
buffer semantics) is registered under that name first; adder.py, resnet20.py etc. are then
imported unchanged.  While generating, every oracle restatement is checked against what the
reference returns, so a fixture is only written if oracle == reference on it.

Inputs are drawn from NumPy's PCG64 generator (platform independent) with the seed stored in
the fixture; large inputs are not stored, only their seed.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from oracle import adder_cuda_cpu, adder_oracle as O, adder_unfold  # noqa: E402
from tests.cases import LAYER_CASES, COL_CASES, draw_layer, draw_cols, resnet20_batch  # noqa: E402


def import_reference(path: str):
    sys.modules["adder_cuda"] = adder_cuda_cpu
    sys.path.insert(0, path)
    ref_adder = importlib.import_module("adder")
    assert Path(ref_adder.__file__).resolve().parent == Path(path).resolve(), ref_adder.__file__
    return ref_adder


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def exact(a: torch.Tensor, b: torch.Tensor, what: str):
    if not torch.equal(a, b):
        raise SystemExit(f"oracle != reference on {what}: max diff {(a - b).abs().max().item():.3e}")


def close(a, b, what, rel=1e-5, abs_=1e-4):
    ok, worst, rep = O.compare(what, a, b, rel, abs_)
    if not ok:
        raise SystemExit("oracle != reference: " + rep)
    return worst


def layer_fixture(ref_adder, case):
    """One adder2d layer through the reference's adder2d_function + autograd, fp32, CPU."""
    x, w, g = (t(a) for a in draw_layer(case))
    s, p = case["stride"], case["pad"]
    xr = x.clone().requires_grad_()
    wr = w.clone().requires_grad_()
    out = ref_adder.adder2d_function(xr, wr, s, p)
    out.backward(g)
    out = out.detach()
    # oracle port of the Python layer: bit-identical (same ops in the same order)
    xo = x.clone().requires_grad_()
    wo = w.clone().requires_grad_()
    out_o = adder_unfold.adder2d_function(xo, wo, s, p)
    out_o.backward(g)
    exact(out_o.detach(), out, f"{case['name']} out (port)")
    exact(xo.grad, xr.grad, f"{case['name']} grad_x (port)")
    exact(wo.grad, wr.grad, f"{case['name']} grad_w (port)")
    # functional restatements
    exact(O.adder2d_forward_unfold(x, w, s, p), out, f"{case['name']} out (unfold)")
    gx_u, gws_u, gw_u = O.adder2d_backward_unfold(g, x, w, s, p)
    exact(gx_u, xr.grad, f"{case['name']} grad_x (unfold)")
    exact(gws_u, wr.grad, f"{case['name']} grad_w (unfold)")
    # independent float64 direct form: agreement to fp32 rounding
    close(O.adder2d_forward_direct(x, w, s, p), out, f"{case['name']} out (direct64)")
    gx_d, gws_d, _ = O.adder2d_backward_direct(g, x, w, s, p)
    close(gx_d, xr.grad, f"{case['name']} grad_x (direct64)")
    close(gws_d, wr.grad, f"{case['name']} grad_w (direct64)")
    return {"out": out.numpy(), "grad_x": xr.grad.numpy(), "grad_w": wr.grad.numpy(), "grad_w_unscaled": gw_u.numpy()}


def col_fixture(ref_adder, case):
    """The reference's column-level Function adder.apply(W_col, X_col) and its backward."""
    W, X, g = (t(a) for a in draw_cols(case))
    Wr = W.clone().requires_grad_()
    Xr = X.clone().requires_grad_()
    y = ref_adder.adder.apply(Wr, Xr)
    y.backward(g)
    exact(O.forward_col(W, X), y.detach(), f"{case['name']} y")
    exact(O.rescale(O.grad_w_col(W, X, g)), Wr.grad, f"{case['name']} grad_W")
    exact(O.grad_x_col(W, X, g), Xr.grad, f"{case['name']} grad_X")
    return {"y": y.detach().numpy(), "grad_W": Wr.grad.numpy(), "grad_X": Xr.grad.numpy(),
            "grad_W_unscaled": O.grad_w_col(W, X, g).numpy()}


def subsample(a: np.ndarray, keep: int):
    """Deterministic sample of a large array: (flat indices, values) plus float64 sum and sum of squares."""
    flat = a.reshape(-1)
    if flat.size <= keep:
        idx = np.arange(flat.size)
    else:
        idx = (np.arange(keep, dtype=np.int64) * (flat.size // keep) + (np.arange(keep) % 7)).clip(0, flat.size - 1)
    return idx.astype(np.int64), flat[idx].copy(), np.float64(flat.astype(np.float64).sum()), \
        np.float64((flat.astype(np.float64) ** 2).sum())


def resnet20_fixture(ref_path: str, batch: int, seed: int):
    """One training step of the reference's resnet20.py (unchanged) on the CPU: logits, loss and all
    gradients after backward, plus the same through this repository's builder with the oracle layer
    (must agree exactly: same architecture, same weights, same op order)."""
    from addernetcuda_b200 import resnet as R
    ref_resnet20 = importlib.import_module("resnet20")
    assert Path(ref_resnet20.__file__).resolve().parent == Path(ref_path).resolve()
    torch.manual_seed(0)
    net_ref = ref_resnet20.resnet20()
    R.init_seeded(net_ref, seed)
    net_ora = R.resnet20(conv=adder_unfold.adder2d)
    R.init_seeded(net_ora, seed)
    assert list(net_ref.state_dict().keys()) == list(net_ora.state_dict().keys())
    for (k1, v1), (k2, v2) in zip(net_ref.state_dict().items(), net_ora.state_dict().items()):
        assert torch.equal(v1, v2), k1
    images, labels = resnet20_batch(batch, seed)
    images, labels = t(images), t(labels)
    res = {}
    for name, net in (("ref", net_ref), ("ora", net_ora)):
        net.train()
        logits = net(images)
        loss = torch.nn.functional.cross_entropy(logits, labels)
        loss.backward()
        res[name] = (logits.detach(), loss.detach(), {k: p.grad.clone() for k, p in net.named_parameters()})
    exact(res["ora"][0], res["ref"][0], "resnet20 logits (port)")
    exact(res["ora"][1], res["ref"][1], "resnet20 loss (port)")
    for k in res["ref"][2]:
        exact(res["ora"][2][k], res["ref"][2][k], f"resnet20 grad {k} (port)")
    logits, loss, grads = res["ref"]
    out = {"logits": logits.numpy(), "loss": np.float32(loss.item()), "keys": np.array(list(grads.keys()))}
    for k, v in grads.items():
        out["grad/" + k] = v.numpy()

    # How reproducible is the reference itself?  Two more runs of the same network:
    #  (a) in float64 (rounding removed), (b) in float32 with the images perturbed by 1e-6 relative
    #  noise (what a different but equally valid fp32 evaluation order upstream amounts to; ReLU gates
    #  of activations that sit within rounding of zero flip).  The per-tensor maximum of the two
    #  differences is stored as `noise/<name>`: no implementation can be expected to agree with the
    #  stored gradients more closely than the reference agrees with itself.
    def rerun(dtype, imgs):
        net = R.resnet20(conv=adder_unfold.adder2d)
        R.init_seeded(net, seed)
        net = net.to(dtype).train()
        lg = net(imgs.to(dtype))
        torch.nn.functional.cross_entropy(lg, labels).backward()
        return lg.detach(), {k: p.grad for k, p in net.named_parameters()}

    lg64, g64 = rerun(torch.float64, images)
    rng = np.random.default_rng(seed + 99)
    jitter = t((1.0 + 1e-6 * rng.standard_normal(tuple(images.shape))).astype(np.float32))
    lgp, gp = rerun(torch.float32, images * jitter)
    out["noise/logits"] = np.float64(max((lg64 - logits.double()).abs().max().item(),
                                         (lgp - logits).abs().max().item()))
    for k, v in grads.items():
        out["noise/" + k] = np.float64(max((g64[k] - v.double()).abs().max().item(), (gp[k] - v).abs().max().item()))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ADDERNET_REFERENCE_DIR", "/root/reference"))
    ap.add_argument("--skip-resnet", action="store_true")
    ap.add_argument("--resnet-batches", default="16,256")
    a = ap.parse_args()
    ref_adder = import_reference(a.reference)
    torch.set_num_threads(max(1, torch.get_num_threads()))
    manifest = {"reference": "LingYeAI/AdderNetCUDA", "torch": torch.__version__, "fixtures": []}

    small = {}

    def put(prefix, fx):
        """Arrays up to 8192 elements are stored whole; larger ones as a deterministic sample of
        4096 values plus float64 checksums."""
        for k, v in fx.items():
            if v.size <= 8192:
                small[f"{prefix}/{k}"] = v
            else:
                idx, val, s1, s2 = subsample(v, 4096)
                small[f"{prefix}/{k}.idx"] = idx
                small[f"{prefix}/{k}.val"] = val
                small[f"{prefix}/{k}.sum"] = s1
                small[f"{prefix}/{k}.sumsq"] = s2

    for case in LAYER_CASES:
        put(case["name"], layer_fixture(ref_adder, case))
        manifest["fixtures"].append(case["name"])
        print("layer", case["name"], "ok")
    for case in COL_CASES:
        put(case["name"], col_fixture(ref_adder, case))
        manifest["fixtures"].append(case["name"])
        print("cols ", case["name"], "ok")
    np.savez_compressed(HERE / "layers.npz", **small)

    if not a.skip_resnet:
        for b in [int(v) for v in a.resnet_batches.split(",")]:
            fx = resnet20_fixture(a.reference, b, seed=1234 + 200)
            np.savez_compressed(HERE / f"resnet20_b{b}.npz", **fx)
            manifest["fixtures"].append(f"resnet20_b{b}")
            print("resnet20 batch", b, "ok, loss", float(fx["loss"]))
    (HERE / "MANIFEST.json").write_text(json.dumps(manifest, indent=1) + "\n")


if __name__ == "__main__":
    main()
