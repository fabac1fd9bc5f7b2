"""The allocation-free dedup entry point, called through its exported C symbol.

Who needs it: hosts that cannot allocate device memory when they run the op (inside a CUDA-graph capture, on a serving path
with a no-allocation rule) or that have no tensor framework at all and link the shared object from C. The test therefore
bypasses the Python bindings: it loads the library with ctypes, passes raw device pointers, and compares the result with the
regular (scratch-from-the-caller) entry point on two consecutive calls, the second one reusing the dirty built-in scratch.
"""
import ctypes

import pytest
import torch

import recis_b200
from recis_b200 import _ext

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_IDS = 1 << 18


def _lib():
    recis_b200.native()                          # builds / loads the extension; ctypes then opens the same shared object
    lib = ctypes.CDLL(_ext._so_path())
    fn = lib.rb_dedup_partition_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _call(fn, ids, world):
    n = ids.numel()
    counts = torch.empty(world, dtype=torch.int32, device=DEV)
    offsets = torch.empty(world + 1, dtype=torch.int32, device=DEV)
    uniq = torch.empty(max(n, 1), dtype=torch.int64, device=DEV)
    rev = torch.empty(max(n, 1), dtype=torch.int32, device=DEV)
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(ids.data_ptr(), n, world, counts.data_ptr(), offsets.data_ptr(), uniq.data_ptr(), rev.data_ptr(), stream, err, 256)
    torch.cuda.synchronize()
    return rc, err.value.decode(), counts, offsets, uniq, rev


def _check_against_regular(fn, ids, world):
    C = recis_b200.native()
    rc, msg, counts, offsets, uniq, rev = _call(fn, ids, world)
    assert rc == 0, msg
    r_uniq, r_rev, r_counts, r_offsets = C.dedup_partition(ids, world)
    assert torch.equal(counts, r_counts) and torch.equal(offsets, r_offsets)
    n_u = int(offsets[-1])
    # same buckets (order inside a bucket is unspecified for both entry points) and a consistent reverse index
    for r in range(world):
        a = uniq[int(offsets[r]):int(offsets[r + 1])].sort().values
        b = r_uniq[int(r_offsets[r]):int(r_offsets[r + 1])].sort().values
        assert torch.equal(a, b)
    assert torch.equal(uniq[:n_u][rev[:ids.numel()].long()], ids)


def test_noalloc_matches_regular_entry_point_twice():
    fn = _lib()
    torch.manual_seed(0)
    torch.cuda.set_device(0)
    ids1 = (torch.randint(0, 50_000, (200_000,), device=DEV) * 2654435761) - 3
    ids2 = torch.randint(0, 1 << 40, (MAX_IDS,), device=DEV)
    ids2[::7] = ids2[0]
    _check_against_regular(fn, ids1, 8)      # first call on this device: performs the symbol look-up
    _check_against_regular(fn, ids2, 3)      # second call: the built-in scratch still holds the first call's keys
    _check_against_regular(fn, ids1[:5], 1)


def test_noalloc_sentinel_id_and_empty_call():
    """The id -1 is the hash set's "empty" marker and lives in a spare cell whose position depends on the call's size: a large
    call followed by a small one (both containing -1) exercises both positions; an empty call only clears the outputs."""
    fn = _lib()
    torch.manual_seed(1)
    big = torch.randint(0, 1 << 30, (150_000,), device=DEV)
    big[::11] = -1
    small = torch.tensor([7, -1, 7, -1, 9, -2, -1], dtype=torch.int64, device=DEV)
    _check_against_regular(fn, big, 4)
    _check_against_regular(fn, small, 4)
    rc, msg, counts, offsets, _u, _r = _call(fn, small[:0], 4)
    assert rc == 0, msg
    assert int(counts.abs().sum()) == 0 and int(offsets.abs().sum()) == 0
    _check_against_regular(fn, small, 2)       # the scratch is usable after the empty call


def test_noalloc_rejects_oversize_and_bad_arguments():
    fn = _lib()
    ids = torch.zeros(MAX_IDS + 1, dtype=torch.int64, device=DEV)
    rc, msg, *_ = _call(fn, ids, 2)
    assert rc == 2 and "limit" in msg
    rc, msg, *_ = _call(fn, ids[:10], 5000)
    assert rc == 1


def test_noalloc_allocates_nothing():
    fn = _lib()
    ids = torch.randint(0, 1000, (10_000,), device=DEV)
    _call(fn, ids, 2)                         # warm: symbol look-up done
    outs = [torch.empty(2, dtype=torch.int32, device=DEV), torch.empty(3, dtype=torch.int32, device=DEV),
            torch.empty(10_000, dtype=torch.int64, device=DEV), torch.empty(10_000, dtype=torch.int32, device=DEV)]
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    err = ctypes.create_string_buffer(64)
    rc = fn(ids.data_ptr(), 10_000, 2, outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(), outs[3].data_ptr(),
            torch.cuda.current_stream().cuda_stream, err, 64)
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.cuda.memory_reserved() == reserved_before
    assert free_before - torch.cuda.mem_get_info()[0] < (1 << 20)      # the device's free memory did not shrink either
