"""The peer-memory exchange kernels on ONE GPU: ``world`` logical ranks in one process, every "peer pointer" a local buffer, the
phases launched one after the other on one stream (no kernel ever waits for another). The harness (``loopback_case.py``) is the
one that ``test_sparse_core.py`` runs against the kernels' host twins; the kernels themselves also run in the 2-GPU tests. The
file name sorts last on purpose: it is the newest GPU test of the suite."""
import pytest
import torch

from loopback_case import run_loopback


@pytest.mark.gpu
@pytest.mark.parametrize("world,dim", [(2, 16), (4, 128), (8, 64)])
def test_exchange_kernels_loopback_on_one_gpu(world, dim):
    run_loopback(torch.device("cuda:0"), world, dim)
