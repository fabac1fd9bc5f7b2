"""The peer-memory exchange kernels on ONE GPU: ``world`` logical ranks in one process, every "peer pointer" a local buffer, the
phases launched one after the other on one stream (no kernel ever waits for another). The harness (``loopback_case.py``) is the
one that ``test_sparse_core.py`` runs against the kernels' host twins; the kernels themselves also run in the 2-GPU tests. The
file name sorts last on purpose: it is the newest GPU test of the suite."""
import pytest
import torch

from loopback_case import run_loopback, run_loopback_overflow


@pytest.mark.gpu
@pytest.mark.parametrize("world,dim", [(2, 16), (4, 128), (8, 64)])
def test_exchange_kernels_loopback_on_one_gpu(world, dim):
    run_loopback(torch.device("cuda:0"), world, dim)


@pytest.mark.gpu
@pytest.mark.parametrize("world,dim", [(3, 8), (4, 32)])
def test_exchange_kernels_clamp_an_overflowing_receive_window(world, dim):
    """Ids skewed to one owner with a receive window that is too small: the same case passes on the kernels' host twins (where
    an out-of-range index would be caught by the guard rows), so the device kernels only ever see in-range indices here too."""
    run_loopback_overflow(torch.device("cuda:0"), world, dim)


@pytest.mark.gpu
def test_wait_on_a_flag_that_nothing_sets_gives_up_with_a_status_bit():
    """A bounded device-side wait that runs out: the flag pad stays at zero, the limit is 0.2 s; the kernel returns, the status
    word carries the time-out bit, and the context goes on working."""
    import time
    import recis_b200
    C = recis_b200.native()
    dev = torch.device("cuda:0")
    world = 4
    flags = torch.zeros(C.N_CHANNELS * world, dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int64, device=dev)
    torch.cuda.synchronize()
    t0 = time.monotonic()
    C.comm_wait(flags, 0, world, 1, 200_000, status)             # channel 0, epoch 1, limit in microseconds
    torch.cuda.synchronize()
    took = time.monotonic() - t0
    assert int(status.item()) & 4
    assert 0.15 < took < 5.0
    # a flag that is already there is not a time-out, and the device still computes
    flags.fill_(1)
    status.zero_()
    C.comm_wait(flags, 0, world, 1, 200_000, status)
    assert int(status.item()) == 0
    assert float((torch.ones(1000, device=dev) * 2).sum()) == 2000.0
