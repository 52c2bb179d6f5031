"""Whole-network parity: one ResNet-20 training step on the GPU against the outputs of the
reference's unchanged resnet20.py + adder.py stepped on the CPU (tests/golden/resnet20_b*.npz)."""
import numpy as np
import pytest
import torch

from oracle import adder_oracle as O
from tests import netcheck
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
    # logits and loss at the plain tolerance; gradients at the plain tolerance, except that a tensor which
    # misses it must be at least as close to the float64 evaluation of the step as the reference's own
    # float32 result is, within a factor of two (tests/netcheck.py)
    netcheck.check_step(z, logits, float(loss.detach()), [(k, p.grad) for k, p in net.named_parameters()],
                        sampled=False, max_anchored=3)


def test_adder_layers_inside_the_network_match_oracle_on_their_own_inputs():
    """During a batch-256 ResNet-20 step every adder layer's (x, w, grad_out) is recorded; a set of
    layers covering every shape class, including the ill-conditioned last-stage ones, is then checked
    against the float64 oracle evaluated on exactly those tensors."""
    from addernetcuda_b200 import adder as A, adder_cuda as ac
    net = _build()
    images, labels = resnet20_batch(256, SEED)
    images, labels = torch.from_numpy(images).to(DEV), torch.from_numpy(labels).to(DEV)
    net.train()
    rec = []
    orig_bw = ac.backward_weight

    def rec_bw(grad_out, x, w, stride=1, padding=0, eta=ac.ETA, out=None, return_norm=False):
        r = orig_bw(grad_out, x, w, stride, padding, eta, out, return_norm)
        rec.append(dict(g=grad_out, x=x, w=w, s=stride, p=padding, gw=r.clone()))
        return r

    ac.backward_weight = rec_bw
    try:
        logits = net(images)
        torch.nn.functional.cross_entropy(logits, labels).backward()
    finally:
        ac.backward_weight = orig_bw
    torch.cuda.synchronize()
    assert len(rec) == 20
    # backward order: last layer first.  pick by weight shape: one of each class + both conv1 of stage 3
    seen, picked = {}, []
    for i, r in enumerate(rec):
        key = (tuple(r["w"].shape), r["s"])
        seen[key] = seen.get(key, 0) + 1
        if seen[key] == 1 or (key == ((64, 64, 3, 3), 1) and seen[key] in (2, 4)):
            picked.append(i)
    assert len(picked) >= 8
    for i in picked:
        r = rec[i]
        g, x, w = r["g"].cpu(), r["x"].cpu(), r["w"].cpu()
        want_gx, want_gws, _ = O.adder2d_backward_direct(g, x, w, r["s"], r["p"])
        want_out = O.adder2d_forward_direct(x[:8], w, r["s"], r["p"])
        name = f"layer#{i} w{tuple(w.shape)} s{r['s']}"
        for what, got, want in ((name + " grad_w", r["gw"], want_gws),
                                (name + " grad_x", ac.backward_input(r["g"], r["x"], r["w"], r["s"], r["p"]), want_gx),
                                (name + " grad_x(fast)", ac.backward_input(r["g"], r["x"], r["w"], r["s"], r["p"], True), want_gx),
                                (name + " out[:8]", ac.forward(r["x"][:8].contiguous(), r["w"], r["s"], r["p"]), want_out)):
            ok, err, msg = O.compare(what, got, want)
            print("   ", msg)
            assert ok, msg


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
            for st in ts.opt.state.values():          # the graph keeps using these buffers: reset in place
                st["momentum_buffer"].zero_()
        losses = [float(ts.run()) for _ in range(2)]
        torch.cuda.synchronize()
        results.append((losses, {k: v.clone() for k, v in net.state_dict().items()}))
    (l0, s0), (l1, s1) = results
    assert abs(l0[0] - l1[0]) < 1e-6, (l0, l1)
    assert abs(l0[1] - l1[1]) < 1e-4, (l0, l1)
    for k in s0:
        if s0[k].dtype.is_floating_point:
            assert torch.allclose(s0[k], s1[k], rtol=1e-4, atol=1e-5), k


def test_eval_mode_forward_matches_oracle_network():
    """Inference: eval-mode forward (running statistics) of the CUDA network equals the CPU oracle network
    loaded from the same state dict, as a checkpoint trained with the reference would be used (test.py:68-90)."""
    from addernetcuda_b200 import resnet as R
    from oracle import adder_unfold as U
    net = _build()
    # make the running statistics non-trivial: two training steps
    images, labels = resnet20_batch(16, SEED)
    xg = torch.from_numpy(images).to(DEV)
    net.train()
    with torch.no_grad():
        net(xg); net(xg * 0.5 + 0.1)
    ref = R.resnet20(conv=U.adder2d)
    ref.load_state_dict({k: v.cpu() for k, v in net.state_dict().items()})
    net.eval(); ref.eval()
    with torch.no_grad():
        got = net(xg)
        want = ref(torch.from_numpy(images))
    ok, err, msg = O.compare("eval logits", got, want, abs_=2e-4)
    print("   ", msg)
    assert ok, msg


def test_reference_checkpoint_keys_load():
    """A state dict with the reference's key names (as saved from a DataParallel wrapper, test.py:37-39)
    loads into the builder's network."""
    from addernetcuda_b200 import resnet as R
    net = R.resnet20()
    sd = {"module." + k: v.clone() for k, v in net.state_dict().items()}
    stripped = {k[len("module."):]: v for k, v in sd.items()}
    missing, unexpected = R.resnet20().load_state_dict(stripped, strict=True)
    assert not missing and not unexpected


def test_folded_batchnorm_inference_and_topk_harness():
    """The inference path: a checkpoint with the reference's `module.` key prefix loads, batch norm folds into
    a one-kernel per-channel affine epilogue (with the residual add and ReLU), the folded network's logits
    equal the unfolded evaluation-mode ones and the CPU oracle network's, and the top-1 / top-5 harness
    counts like a plain NumPy evaluation of the same logits."""
    from addernetcuda_b200 import inference as I, resnet as R
    from oracle import adder_unfold as U
    net = _build()
    images, labels = resnet20_batch(32, SEED)
    xg, yg = torch.from_numpy(images).to(DEV), torch.from_numpy(labels).to(DEV)
    net.train()
    with torch.no_grad():
        net(xg); net(xg * 0.7 - 0.2)                 # non-trivial running statistics
    checkpoint = {"module." + k: v.detach().cpu().clone() for k, v in net.state_dict().items()}
    fresh = R.resnet20().to(DEV)
    missing, unexpected = I.load_reference_checkpoint(fresh, checkpoint)
    assert not missing and not unexpected
    fresh.eval()
    with torch.no_grad():
        plain = fresh(xg)
    folded = I.fold_batchnorm(fresh)
    assert not any(isinstance(m, torch.nn.BatchNorm2d) for m in folded.modules())
    with torch.no_grad():
        got = folded(xg)
    ok, err, msg = O.compare("folded vs unfolded eval logits", got, plain, abs_=2e-4)
    print("   ", msg)
    assert ok, msg
    ref = R.resnet20(conv=U.adder2d)
    I.load_reference_checkpoint(ref, checkpoint)
    ref.eval()
    with torch.no_grad():
        want = ref(torch.from_numpy(images))
    ok, err, msg = O.compare("folded eval logits vs oracle network", got, want, abs_=2e-4)
    print("   ", msg)
    assert ok, msg
    # top-k harness against NumPy on the oracle's logits
    top1, top5 = I.validate([(xg[:16], yg[:16]), (xg[16:], yg[16:])], folded, topk=(1, 5))
    order = np.argsort(-want.numpy(), axis=1)
    want1 = 100.0 * np.mean(order[:, 0] == labels)
    want5 = 100.0 * np.mean([labels[i] in order[i, :5] for i in range(len(labels))])
    assert abs(top1 - want1) < 1e-3 and abs(top5 - want5) < 1e-3, (top1, want1, top5, want5)
