"""Whole-network parity: one ResNet-20 training step on the GPU against the outputs of the
reference's unchanged resnet20.py + adder.py stepped on the CPU (tests/golden/resnet20_b*.npz)."""
import numpy as np
import pytest
import torch

from oracle import adder_oracle as O
from tests.cases import resnet20_batch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SEED = 1434


def _build():
    import addernetcuda_b200 as ab
    from addernetcuda_b200 import resnet as R
    ab.strict_fp32()
    net = R.resnet20()
    R.init_seeded(net, SEED)
    return net.to(DEV)


@pytest.mark.parametrize("batch", [16, 256])
@pytest.mark.parametrize("fast_clamp", [False, True], ids=["exact", "fastclamp"])
def test_resnet20_step_matches_reference(batch, fast_clamp):
    from addernetcuda_b200 import adder as A
    z = np.load(f"tests/golden/resnet20_b{batch}.npz")
    net = _build()
    images, labels = resnet20_batch(batch, SEED)
    images, labels = torch.from_numpy(images).to(DEV), torch.from_numpy(labels).to(DEV)
    net.train()
    A.FAST_CLAMP = fast_clamp
    try:
        logits = net(images)
        loss = torch.nn.functional.cross_entropy(logits, labels)
        loss.backward()
    finally:
        A.FAST_CLAMP = False
    torch.cuda.synchronize()
    ok, worst, msg = O.compare("logits", logits, torch.from_numpy(z["logits"]))
    print("   ", msg)
    assert ok, msg
    assert abs(float(loss.detach()) - float(z["loss"])) <= 1e-4 + 1e-5 * abs(float(z["loss"]))
    worst_name, worst_err, failures = None, 0.0, []
    for k, p in net.named_parameters():
        ok, err, msg = O.compare(k, p.grad, torch.from_numpy(z["grad/" + k]))
        if err > worst_err:
            worst_name, worst_err = k, err
        if not ok:
            failures.append(msg)
    print(f"    worst gradient tensor: {worst_name} max_abs_err={worst_err:.3e} "
          f"({len(list(net.parameters()))} tensors compared)")
    assert not failures, "\n".join(failures)


def test_graph_captured_step_equals_eager_step():
    """The CUDA-graph path is the same computation: identical loss and weights after two steps."""
    from addernetcuda_b200.train import TrainStep
    images, labels = resnet20_batch(32, SEED)
    images, labels = torch.from_numpy(images), torch.from_numpy(labels)
    results = []
    for use_graph in (False, True):
        net = _build()
        net.train()
        ts = TrainStep(net, (32, 3, 32, 32), 10, use_graph=use_graph, device=DEV)
        ts.load_batch(images.to(DEV), labels.to(DEV))
        if use_graph:
            # capture without the warm-up updates so both runs start from the same weights
            state = {k: v.clone() for k, v in net.state_dict().items()}
            ts.warmup(1)
            ts.capture()
            net.load_state_dict(state)
            ts.opt.state.clear()
        losses = [float(ts.run()) for _ in range(2)]
        torch.cuda.synchronize()
        results.append((losses, {k: v.clone() for k, v in net.state_dict().items()}))
    (l0, s0), (l1, s1) = results
    assert abs(l0[0] - l1[0]) < 1e-6, (l0, l1)
    assert abs(l0[1] - l1[1]) < 1e-4, (l0, l1)
    for k in s0:
        if s0[k].dtype.is_floating_point:
            assert torch.allclose(s0[k], s1[k], rtol=1e-4, atol=1e-5), k


def test_reference_checkpoint_keys_load():
    """A state dict with the reference's key names (as saved from a DataParallel wrapper, test.py:37-39)
    loads into the builder's network."""
    from addernetcuda_b200 import resnet as R
    net = R.resnet20()
    sd = {"module." + k: v.clone() for k, v in net.state_dict().items()}
    stripped = {k[len("module."):]: v for k, v in sd.items()}
    missing, unexpected = R.resnet20().load_state_dict(stripped, strict=True)
    assert not missing and not unexpected
