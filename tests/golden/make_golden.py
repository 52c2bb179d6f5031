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


# fixture name, reference module, constructor, batch, input height = width, classes, seed
NETWORK_FIXTURES = [
    ("vgg11_bn_b4", "vgg", "vgg11_bn", 4, 32, 10, 1234 + 300),
    ("resnet50_b4", "resnet50", "resnet50", 4, 224, 1000, 1234 + 500),
]


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
    #  (a) in float64 (rounding removed), (b) three times in float32 with the images perturbed by 1e-6
    #  relative noise (what a different but equally valid fp32 evaluation order upstream amounts to; ReLU
    #  gates of activations that sit within rounding of zero flip).  The per-tensor maximum of all those
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
    out["logits64"] = lg64.to(torch.float32).numpy()
    # the float64 gradients themselves (rounded to float32 for storage): the anchor for judging an
    # implementation by ITS distance to exact arithmetic, next to the reference's own distance
    for k, v in g64.items():
        out["grad64/" + k] = v.to(torch.float32).numpy()
    noise = {k: (g64[k] - v.double()).abs().max().item() for k, v in grads.items()}
    noise_logits = (lg64 - logits.double()).abs().max().item()
    for j in range(3):       # three independent perturbations: the envelope of the reference's self-noise
        rng = np.random.default_rng(seed + 99 + j)
        jitter = t((1.0 + 1e-6 * rng.standard_normal(tuple(images.shape))).astype(np.float32))
        lgp, gp = rerun(torch.float32, images * jitter)
        noise_logits = max(noise_logits, (lgp - logits).abs().max().item())
        for k, v in grads.items():
            noise[k] = max(noise[k], (gp[k] - v).abs().max().item())
    out["noise/logits"] = np.float64(noise_logits)
    for k in grads:
        out["noise/" + k] = np.float64(noise[k])
    return out


def build_on(adder_module, module_name: str, ctor: str):
    """Import a reference model file with `adder` resolving to `adder_module` and build the network."""
    saved = sys.modules.get("adder")
    sys.modules["adder"] = adder_module
    sys.modules.pop(module_name, None)
    try:
        net = getattr(importlib.import_module(module_name), ctor)()
    finally:
        sys.modules.pop(module_name, None)
        if saved is not None:
            sys.modules["adder"] = saved
    return net


def network_batch(batch, in_hw, classes, seed):
    """Synthetic image batch ~ N(0,1) [B,3,H,W] with uniform labels (stand-in for CIFAR-10 / ImageNet)."""
    from addernetcuda_b200.synthetic import image_batch
    return image_batch(batch, in_hw, classes, seed)


def network_fixture(ref_adder, module_name: str, ctor: str, batch: int, in_hw: int, classes: int, seed: int,
                    keep: int = 256):
    """One training step (forward, cross-entropy, backward) of a reference model file, unchanged, on the
    CPU in float32 through the reference's adder.py; and the same network on the oracle port in float64.
    Stored: logits, loss, and per parameter a deterministic sample of the gradient (float32 run and
    float64 run at the same positions) with float64 checksums.  Dropout layers are put in eval mode
    (identity): a random mask cannot be reproduced across devices."""
    from addernetcuda_b200 import resnet as R
    images, labels = network_batch(batch, in_hw, classes, seed)
    images, labels = t(images), t(labels)

    def run(net, dtype, order_noise=None):
        R.init_seeded(net, seed)
        net = net.to(dtype).train()
        for m in net.modules():
            if isinstance(m, torch.nn.Dropout):
                m.eval()
        hooks = []
        if order_noise is not None:
            # A float32 sum of K terms carries a rounding error that depends on the order of the additions; for
            # the plain running sum a GPU thread forms it is a random walk of about sqrt(K) * 2^-24 relative
            # (torch's CPU sum is pairwise and far below that).  Every adder layer's output is perturbed by
            # that much, so that the envelope covers what any valid float32 evaluation order may produce.
            for m in net.modules():
                if type(m).__name__ == "adder2d":
                    sigma = math.sqrt(m.adder[0].numel()) * 2.0 ** -24
                    hooks.append(m.register_forward_hook(
                        lambda mod, inp, out, sigma=sigma: out * (1.0 + sigma * torch.from_numpy(
                            order_noise.standard_normal(tuple(out.shape)).astype(np.float32)))))
        logits = net(images.to(dtype))
        loss = torch.nn.functional.cross_entropy(logits, labels)
        loss.backward()
        for h in hooks:
            h.remove()
        return logits.detach(), loss.detach(), {k: p.grad for k, p in net.named_parameters()}

    lg, loss, grads = run(build_on(ref_adder, module_name, ctor), torch.float32)
    lg_o, loss_o, grads_o = run(build_on(adder_unfold, module_name, ctor), torch.float32)
    exact(lg_o, lg, f"{module_name} logits (port)")
    for k in grads:
        exact(grads_o[k], grads[k], f"{module_name} grad {k} (port)")
    lg64, loss64, grads64 = run(build_on(adder_unfold, module_name, ctor), torch.float64)
    # the reference's self-noise: how far its own float32 results move between float32 and float64, and under
    # three draws of (a) 1e-6 relative perturbations of the images (see resnet20_fixture) together with (b)
    # summation-order noise on every adder layer's output (see run)
    noise = {k: (grads64[k] - v.double()).abs().max().item() for k, v in grads.items()}
    noise_logits = (lg64 - lg.double()).abs().max().item()
    clean = images
    for j in range(3):
        rng = np.random.default_rng(seed + 99 + j)
        images = clean * t((1.0 + 1e-6 * rng.standard_normal(tuple(clean.shape))).astype(np.float32))
        lgp, _, gp = run(build_on(adder_unfold, module_name, ctor), torch.float32, order_noise=rng)
        noise_logits = max(noise_logits, (lgp - lg).abs().max().item())
        for k, v in grads.items():
            noise[k] = max(noise[k], (gp[k] - v).abs().max().item())
    images = clean
    out = {"logits": lg.numpy(), "loss": np.float32(loss.item()), "logits64": lg64.to(torch.float32).numpy(),
           "loss64": np.float64(loss64.item()), "noise/logits": np.float64(noise_logits),
           "keys": np.array(list(grads.keys())),
           "batch": np.int64(batch), "in_hw": np.int64(in_hw), "classes": np.int64(classes), "seed": np.int64(seed)}
    for k, v in grads.items():
        idx, val, s1, s2 = subsample(v.numpy(), keep)
        out[f"grad/{k}.idx"] = idx
        out[f"grad/{k}.val"] = val
        out[f"grad/{k}.sumsq"] = s2
        out[f"grad64/{k}.val"] = grads64[k].numpy().reshape(-1)[idx].astype(np.float32)
        out[f"noise/{k}"] = np.float64(noise[k])
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("ADDERNET_REFERENCE_DIR", ""),
                    help="checkout of the reference project (or set ADDERNET_REFERENCE_DIR)")
    ap.add_argument("--skip-layers", action="store_true")
    ap.add_argument("--skip-resnet", action="store_true")
    ap.add_argument("--skip-networks", action="store_true", help="skip the vgg11_bn and resnet50 fixtures")
    ap.add_argument("--resnet-batches", default="16,256")
    a = ap.parse_args()
    if not a.reference or not Path(a.reference, "adder.py").exists():
        raise SystemExit("give the reference checkout with --reference or ADDERNET_REFERENCE_DIR")
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
        manifest["fixtures"].append(case["name"])
        if a.skip_layers:
            continue
        put(case["name"], layer_fixture(ref_adder, case))
        print("layer", case["name"], "ok")
    for case in COL_CASES:
        manifest["fixtures"].append(case["name"])
        if a.skip_layers:
            continue
        put(case["name"], col_fixture(ref_adder, case))
        print("cols ", case["name"], "ok")
    if not a.skip_layers:
        np.savez_compressed(HERE / "layers.npz", **small)

    if not a.skip_resnet:
        for b in [int(v) for v in a.resnet_batches.split(",")]:
            fx = resnet20_fixture(a.reference, b, seed=1234 + 200)
            np.savez_compressed(HERE / f"resnet20_b{b}.npz", **fx)
            manifest["fixtures"].append(f"resnet20_b{b}")
            print("resnet20 batch", b, "ok, loss", float(fx["loss"]))
    # whole networks from the reference's other model files, unchanged: vgg.py (first layer K = 27) and
    # resnet50.py (the ImageNet bottleneck network), one small-batch training step each
    for name, module, ctor, batch, hw, classes, seed in NETWORK_FIXTURES:
        manifest["fixtures"].append(name)
        if a.skip_networks:
            continue
        fx = network_fixture(ref_adder, module, ctor, batch, hw, classes, seed)
        np.savez_compressed(HERE / f"{name}.npz", **fx)
        print(name, "ok, loss", float(fx["loss"]))
    (HERE / "MANIFEST.json").write_text(json.dumps(manifest, indent=1) + "\n")


if __name__ == "__main__":
    main()
