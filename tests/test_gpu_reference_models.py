"""The reference's own model files, byte for byte, training on the GPU through the drop-in.

`baseline/_ref/` holds resnet20.py, resnet50.py and vgg.py exactly as the reference ships them
(`python baseline/install_ref.py` copies them there).  After `install_dropin()` their `import adder`
resolves to this package, and one training step of each is compared with what the same file produced
on the CPU through the reference's adder.py (fixtures made by tests/golden/make_golden.py):

  * resnet20.py, batch 16: logits, loss and all 66 gradients;
  * vgg.py vgg11_bn, batch 4 (first layer 3 -> 64 channels: K = 27, a size at which the reference's CUDA
    kernels are wrong and only its closed form defines the result): logits, loss, gradient samples;
  * resnet50.py, batch 4: logits, loss, gradient samples; and every distinct adder layer shape of the
    network checked on the tensors it actually saw against the float64 oracle.
"""
import importlib
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import adder_oracle as O
from tests import netcheck
from tests.cases import resnet20_batch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _reference_model(module_name, ctor):
    """Build a network from the reference's unchanged model file on top of the drop-in `adder`."""
    if not (REF / f"{module_name}.py").exists():
        pytest.fail(f"{REF}/{module_name}.py is missing: run `python baseline/install_ref.py --reference <checkout>`")
    import addernetcuda_b200 as ab
    ab.install_dropin()
    ab.strict_fp32()
    sys.modules.pop(module_name, None)
    sys.path.insert(0, str(REF))
    try:
        mod = importlib.import_module(module_name)
        assert Path(mod.__file__).resolve().parent == REF.resolve()
        import adder
        assert adder.__name__ == "addernetcuda_b200.adder", "the model file did not pick up the drop-in"
        return getattr(mod, ctor)()
    finally:
        sys.path.remove(str(REF))
        sys.modules.pop(module_name, None)


def _network_batch(z):
    from addernetcuda_b200.synthetic import image_batch
    images, labels = image_batch(int(z["batch"]), int(z["in_hw"]), int(z["classes"]), int(z["seed"]))
    return torch.from_numpy(images).to(DEV), torch.from_numpy(labels).to(DEV)


def _train_step(net, images, labels):
    net.train()
    for m in net.modules():
        if isinstance(m, torch.nn.Dropout):
            m.eval()          # identity, as in the fixture: a random mask is not reproducible across devices
    logits = net(images)
    loss = torch.nn.functional.cross_entropy(logits, labels)
    loss.backward()
    torch.cuda.synchronize()
    return logits.detach(), float(loss.detach())


def test_reference_resnet20_file_trains_on_the_dropin():
    from addernetcuda_b200 import resnet as R
    z = np.load(ROOT / "tests" / "golden" / "resnet20_b16.npz")
    net = _reference_model("resnet20", "resnet20")
    R.init_seeded(net, 1434)
    net = net.to(DEV)
    assert type(net.layer1[0].conv1).__module__ == "addernetcuda_b200.adder"
    assert type(net.layer1[0].bn1) is torch.nn.BatchNorm2d       # the file's own modules, nothing substituted
    images, labels = resnet20_batch(16, 1434)
    logits, loss = _train_step(net, torch.from_numpy(images).to(DEV), torch.from_numpy(labels).to(DEV))
    netcheck.check_step(z, logits, loss, [(k, p.grad) for k, p in net.named_parameters()], sampled=False,
                        max_anchored=3)


def test_reference_vgg11_bn_file_trains_on_the_dropin():
    from addernetcuda_b200 import resnet as R
    z = np.load(ROOT / "tests" / "golden" / "vgg11_bn_b4.npz")
    net = _reference_model("vgg", "vgg11_bn")
    R.init_seeded(net, int(z["seed"]))
    net = net.to(DEV)
    first = net.features[0]
    assert type(first).__module__ == "addernetcuda_b200.adder" and tuple(first.adder.shape) == (64, 3, 3, 3)
    images, labels = _network_batch(z)
    logits, loss = _train_step(net, images, labels)
    netcheck.check_step(z, logits, loss, [(k, p.grad) for k, p in net.named_parameters()], sampled=True,
                        max_anchored=8)


def _resnet50_step(net, z, record):
    """One training step of a ResNet-50; with `record`, every adder layer's (grad_out, x, w, stride, pad)
    and the gradients it returned are kept."""
    from addernetcuda_b200 import adder_cuda as ac
    images, labels = _network_batch(z)
    rec = []
    orig = ac.backward

    def recording_backward(grad_out, x, w, stride=1, padding=0, eta=ac.ETA, fast_clamp=False, out_w=None, overlap=True):
        gx, gw = orig(grad_out, x, w, stride, padding, eta, fast_clamp, out_w, overlap)
        rec.append(dict(g=grad_out, x=x, w=w, s=stride, p=padding, gx=gx, gw=gw.clone()))
        return gx, gw

    if record:
        ac.backward = recording_backward
    try:
        logits, loss = _train_step(net, images, labels)
    finally:
        ac.backward = orig
    return logits, loss, rec


def test_reference_resnet50_file_trains_on_the_dropin():
    from addernetcuda_b200 import resnet as R, adder_cuda as ac
    z = np.load(ROOT / "tests" / "golden" / "resnet50_b4.npz")
    net = _reference_model("resnet50", "resnet50")
    R.init_seeded(net, int(z["seed"]))
    net = net.to(DEV)
    logits, loss, rec = _resnet50_step(net, z, record=True)
    # Batch 4 through 52 adder layers and as many batch norms (the last one over 4 samples) is a chaotic map:
    # most adder gradients move by 1e-3 under a 1e-6 perturbation of the images, in the reference itself.  The
    # network-level comparison therefore mostly runs on the self-noise rule of tests/netcheck.py and is a sanity
    # check; the parity gate of this test is the per-layer comparison below.
    netcheck.check_step(z, logits, loss, [(k, p.grad) for k, p in net.named_parameters()], sampled=True,
                        max_anchored=161)
    # 51 adder layers have an input gradient (the first one's input is the max-pooled stem output, which
    # needs one too): every layer went through the fused backward
    assert len(rec) == 52, len(rec)
    seen, picked = set(), []
    for r in rec:
        key = (tuple(r["w"].shape), tuple(r["x"].shape[2:]), r["s"])
        if key not in seen:
            seen.add(key)
            picked.append(r)
    assert len(picked) == 22, sorted(seen)          # distinct (weight shape, input size, stride) among the 52 layers
    for r in picked:
        g, x, w = r["g"].cpu(), r["x"].cpu(), r["w"].cpu()
        name = f"w{tuple(w.shape)} on {tuple(x.shape[2:])} s{r['s']}"
        want_gx, want_gws, _ = O.adder2d_backward_direct(g, x, w, r["s"], r["p"])
        want_out = O.adder2d_forward_direct(x[:1], w, r["s"], r["p"])
        for what, got, want in ((name + " grad_w", r["gw"], want_gws), (name + " grad_x", r["gx"], want_gx),
                                (name + " out[:1]", ac.forward(r["x"][:1].contiguous(), r["w"], r["s"], r["p"]), want_out)):
            ok, err, msg = O.compare(what, got, want)
            print("   ", msg)
            assert ok, msg


def test_builder_resnet50_step_matches_reference_fixture():
    """The package's own ResNet-50 builder (fused BatchNorm kernels) on the same step."""
    from addernetcuda_b200 import resnet as R
    import addernetcuda_b200 as ab
    ab.strict_fp32()
    z = np.load(ROOT / "tests" / "golden" / "resnet50_b4.npz")
    net = R.resnet50()
    R.init_seeded(net, int(z["seed"]))
    net = net.to(DEV)
    logits, loss, _ = _resnet50_step(net, z, record=False)
    netcheck.check_step(z, logits, loss, [(k, p.grad) for k, p in net.named_parameters()], sampled=True,
                        max_anchored=161)
