"""The one-kernel gradient exchange (adder_b200_peer_allreduce) on ONE GPU.

Several ranks are emulated inside a single cooperative launch (their CTAs wait on each other, so they must
not be separate launches on one GPU): every rank pushes its bucket into every rank's receive area, waits
for the others and adds the copies in rank order.  Checked: the average is exact in that order and
bit-identical on all ranks, over several calls (the slots alternate between two parities), also when
replayed from a CUDA graph; and a wait that cannot be satisfied (world of 2, only rank 0 launched) ends by
itself with ADDER_ERR_TIMEOUT in the status word and leaves the context usable."""
import ctypes

import pytest
import torch

from addernetcuda_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make(world, ranks_here, n, max_polls, first_rank=0, chunks=0):
    lib = _lib.load()
    nbytes = lib.adder_b200_peer_area_bytes(n, world)
    assert nbytes > 0
    areas = [torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    data = [torch.zeros(n, dtype=torch.float32, device=DEV) for _ in range(ranks_here)]
    comm = ctypes.c_void_p()
    d = (ctypes.c_void_p * ranks_here)(*[t.data_ptr() for t in data])
    a = (ctypes.c_void_p * world)(*[t.data_ptr() for t in areas])
    _lib.check(lib.adder_b200_peer_comm_create(ctypes.byref(comm), world, first_rank, ranks_here, d, a, n, chunks, max_polls),
               "adder_b200_peer_comm_create")
    return lib, comm, data, areas


def _status(lib, comm, reset=False):
    st, ep = ctypes.c_int(0), ctypes.c_uint(0)
    _lib.check(lib.adder_b200_peer_comm_status(comm, ctypes.byref(st), ctypes.byref(ep), int(reset)), "status")
    return st.value, ep.value


@pytest.mark.parametrize("world,n", [(2, 4096), (4, 270_000), (8, 40_004), (3, 4)])
def test_emulated_ranks_average_in_rank_order_bit_identically(world, n):
    lib, comm, data, areas = _make(world, world, n, max_polls=1 << 20)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.manual_seed(world * 1000 + n % 97)
    for call in range(3):
        src = [torch.randn(n, device=DEV) for _ in range(world)]
        for d, s in zip(data, src):
            d.copy_(s)
        _lib.check(lib.adder_b200_peer_allreduce(comm, stream), "adder_b200_peer_allreduce")
        torch.cuda.synchronize()
        want = src[0].clone()
        for s in src[1:]:
            want += s
        want *= 1.0 / world
        st, ep = _status(lib, comm)
        assert st == 0 and ep == call + 1, (st, ep)
        for r, d in enumerate(data):
            assert torch.equal(d, want), (call, r, (d - want).abs().max().item())
    _lib.check(lib.adder_b200_peer_comm_destroy(comm), "destroy")


def test_graph_replay_advances_the_epoch_on_the_device():
    world, n = 4, 65536
    lib, comm, data, areas = _make(world, world, n, max_polls=1 << 20)
    src = [torch.randn(n, device=DEV) for _ in range(world)]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for d, s in zip(data, src):       # warm-up call outside the graph
            d.copy_(s)
        _lib.check(lib.adder_b200_peer_allreduce(comm, ctypes.c_void_p(side.cuda_stream)), "warm-up")
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for d, s in zip(data, src):
                d.copy_(s)
            _lib.check(lib.adder_b200_peer_allreduce(comm, ctypes.c_void_p(side.cuda_stream)), "captured")
    want = (src[0] + src[1] + src[2] + src[3]) * 0.25
    for replay in range(4):
        for d in data:
            d.zero_()
        graph.replay()
        torch.cuda.synchronize()
        st, ep = _status(lib, comm)
        assert st == 0 and ep == 2 + replay, (st, ep)
        for d in data:
            assert torch.equal(d, want)
    _lib.check(lib.adder_b200_peer_comm_destroy(comm), "destroy")


def test_a_wait_that_cannot_be_satisfied_times_out_and_reports():
    # world of 2, but only rank 0 is ever launched: its wait for rank 1's flags must run out by itself
    lib, comm, data, areas = _make(2, 1, 8192, max_polls=200)
    data[0].fill_(3.0)
    _lib.check(lib.adder_b200_peer_allreduce(comm, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "launch")
    torch.cuda.synchronize()                       # returns: the kernel gave up instead of spinning forever
    st, ep = _status(lib, comm, reset=True)
    assert st == _lib.ERR_TIMEOUT, st
    assert ep == 1                                 # the call still counts, so the ranks' epochs stay in step
    assert torch.all(data[0] == 3.0)               # nothing was reduced
    assert _status(lib, comm)[0] == 0              # cleared by the reset
    # the context is intact
    assert float((torch.ones(8, device=DEV) * 2).sum()) == 16.0
    _lib.check(lib.adder_b200_peer_comm_destroy(comm), "destroy")


def test_arguments_are_checked():
    lib = _lib.load()
    comm = ctypes.c_void_p()
    t = torch.zeros(64, device=DEV)
    area = torch.zeros(lib.adder_b200_peer_area_bytes(64, 2), dtype=torch.uint8, device=DEV)
    d = (ctypes.c_void_p * 1)(t.data_ptr())
    a = (ctypes.c_void_p * 2)(area.data_ptr(), area.data_ptr())
    assert lib.adder_b200_peer_comm_create(ctypes.byref(comm), 2, 0, 1, d, a, 63, 0, 100) == _lib.ERR_BAD_SHAPE    # n % 4
    assert lib.adder_b200_peer_comm_create(ctypes.byref(comm), 99, 0, 1, d, a, 64, 0, 100) == _lib.ERR_BAD_SHAPE   # world
    assert lib.adder_b200_peer_comm_create(ctypes.byref(comm), 2, 1, 2, d, a, 64, 0, 100) == _lib.ERR_BAD_SHAPE    # ranks
    assert lib.adder_b200_peer_area_bytes(0, 2) == 0
    assert lib.adder_b200_peer_allreduce(None, None) == _lib.ERR_NULL_POINTER
