"""GPU: the workspace-free event vecmat (``bsx_event_vecmat_static``).

Some users of the library cannot pass a workspace because they cannot allocate
device memory at the point of the call — a custom-call handler inside a
framework that owns the GPU's memory pool, or a loop that must not suffer the
device-wide stall of an allocation.  For them the queue of active rows lives in
a 4 MiB array inside the library.  This file checks, through the C ABI, that the
entry point returns what ``bsx_event_vecmat`` returns — and what the CPU oracle
computes — on two consecutive calls (the second must not see leftovers of the
first), for every spike format, that it holds no extra device memory after a call,
and that inputs beyond the built-in queue are refused.

The file name sorts last so that a failure here cannot hide the other tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import event_oracle as eo

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-6      # float32 sums of atomically added weights; same bar as the other GPU tests


def _conn(cuda, n_pre, n_post, K, hetero, seed):
    from brainstate_b200 import FixedPostNumConn
    rs = np.random.RandomState(seed)
    idx = torch.from_numpy(rs.randint(0, n_post, (n_pre, K)).astype(np.int32)).to(cuda)
    w = torch.from_numpy(rs.uniform(0.05, 0.15, (n_pre, K)).astype(np.float32)).to(cuda) if hetero else 0.1
    return FixedPostNumConn((w, idx), shape=(n_pre, n_post))


def _with_workspace(bsx, conn, spk, fmt, batch, n_post):
    from brainstate_b200 import _lib
    st = conn._struct()
    out = torch.full((batch, n_post), 7.0, dtype=torch.float32, device=spk.device)
    nbytes = bsx.bsx_event_vecmat_workspace_bytes(batch, conn.shape[0])
    ws = torch.empty(nbytes, dtype=torch.uint8, device=spk.device)
    _lib.check(bsx.bsx_event_vecmat(C.byref(st), spk.data_ptr(), fmt, batch, out.data_ptr(), 0,
                                    ws.data_ptr(), nbytes, _lib.current_stream()))
    return out


def _static(bsx, conn, spk, fmt, batch, n_post, accumulate=0, out=None):
    from brainstate_b200 import _lib
    st = conn._struct()
    if out is None:
        out = torch.full((batch, n_post), -3.0, dtype=torch.float32, device=spk.device)
    _lib.check(bsx.bsx_event_vecmat_static(C.byref(st), spk.data_ptr(), fmt, batch, out.data_ptr(), accumulate,
                                           _lib.current_stream()))
    return out


@pytest.mark.parametrize('hetero', [False, True])
def test_static_queue_matches_workspace_entry_point_on_two_calls(hetero, bsx, cuda):
    from brainstate_b200 import _lib
    n_pre, n_post, K, batch = 3001, 5003, 37, 3
    conn = _conn(cuda, n_pre, n_post, K, hetero, seed=31)
    rs = np.random.RandomState(32)
    # the first call fills the queue with many rows, the second with few: stale
    # entries of the first must not be replayed
    for rate in (0.4, 0.02):
        spk = torch.from_numpy(rs.random_sample((batch, n_pre)) < rate).to(cuda)
        ref = _with_workspace(bsx, conn, spk, _lib.SPK_BOOL8, batch, n_post)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        got = _static(bsx, conn, spk, _lib.SPK_BOOL8, batch, n_post)
        torch.cuda.synchronize()
        if rate != 0.4:           # past the first call (module load, symbol lookup): nothing new is held
            assert torch.cuda.mem_get_info()[0] >= free_before
        if hetero:
            np.testing.assert_allclose(got.cpu().numpy(), ref.cpu().numpy(), rtol=RTOL, atol=ATOL)
        else:
            assert torch.equal(got, ref)
        # and against the CPU restatement of the product itself, not only the sibling entry point
        w_host = conn.data.cpu().numpy() if hetero else np.float32(0.1)
        expect = eo.event_vecmat(spk.cpu().numpy(), conn.indices.cpu().numpy(), w_host, n_post)
        np.testing.assert_allclose(got.cpu().numpy(), expect, rtol=RTOL, atol=ATOL)
        # accumulate = 1 adds on top of the previous result
        twice = _static(bsx, conn, spk, _lib.SPK_BOOL8, batch, n_post, accumulate=1, out=got.clone())
        np.testing.assert_allclose(twice.cpu().numpy(), 2 * ref.cpu().numpy(), rtol=RTOL, atol=ATOL)
    # float spikes and packed words go through the same queue; a compacted list needs none
    spk = rs.random_sample((batch, n_pre)) < 0.1
    w_host = conn.data.cpu().numpy() if hetero else np.float32(0.1)
    expect = eo.event_vecmat(spk, conn.indices.cpu().numpy(), w_host, n_post)
    sf = torch.from_numpy((spk * rs.uniform(0.5, 2.0, spk.shape)).astype(np.float32)).to(cuda)
    ref = _with_workspace(bsx, conn, sf, _lib.SPK_F32, batch, n_post)
    got = _static(bsx, conn, sf, _lib.SPK_F32, batch, n_post)
    np.testing.assert_allclose(got.cpu().numpy(), ref.cpu().numpy(), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(got.cpu().numpy(), expect, rtol=RTOL, atol=ATOL)
    words = torch.from_numpy(np.stack([eo.pack_bits(r) for r in spk]).view(np.int32)).to(cuda)
    got = _static(bsx, conn, words, _lib.SPK_BITS32, batch, n_post)
    np.testing.assert_allclose(got.cpu().numpy(), expect, rtol=RTOL, atol=ATOL)
    active = np.nonzero(spk[0])[0].astype(np.int32)
    lst = torch.from_numpy(np.concatenate([[active.size], active]).astype(np.int32)).to(cuda)
    got = _static(bsx, conn, lst, _lib.SPK_LIST, 1, n_post)
    np.testing.assert_allclose(got.cpu().numpy(), expect[:1], rtol=RTOL, atol=ATOL)


def test_static_queue_with_a_batch_that_fills_the_gpu(bsx, cuda):
    """A batch large enough for the library to pick the shared-memory scatter (which needs no
    queue at all) still fits the entry point's size limit and gives the oracle's result."""
    from brainstate_b200 import _lib
    n_pre, n_post, K, batch = 4000, 6000, 29, 160          # 640 000 queue entries at most
    conn = _conn(cuda, n_pre, n_post, K, True, seed=35)
    st = conn._struct()
    assert bsx.bsx_event_vecmat_variant(C.byref(st), _lib.SPK_BOOL8, batch) == _lib.VECMAT_SHARED_SLICES
    spk = np.random.RandomState(36).random_sample((batch, n_pre)) < 0.03
    expect = eo.event_vecmat(spk, conn.indices.cpu().numpy(), conn.data.cpu().numpy(), n_post)
    ts = torch.from_numpy(spk).to(cuda)
    for _ in range(2):
        got = _static(bsx, conn, ts, _lib.SPK_BOOL8, batch, n_post)
        np.testing.assert_allclose(got.cpu().numpy(), expect, rtol=RTOL, atol=ATOL)


def test_static_queue_refuses_inputs_beyond_its_size(bsx, cuda):
    from brainstate_b200 import _lib
    n_pre, n_post, K = 70000, 64, 2
    conn = _conn(cuda, n_pre, n_post, K, False, seed=33)
    batch = 15                                   # 15 * 70000 = 1 050 000 > 1 048 000 queue entries
    spk = torch.zeros((batch, n_pre), dtype=torch.bool, device=cuda)
    out = torch.full((batch, n_post), 5.0, dtype=torch.float32, device=cuda)
    st = conn._struct()
    rc = bsx.bsx_event_vecmat_static(C.byref(st), spk.data_ptr(), _lib.SPK_BOOL8, batch, out.data_ptr(), 0,
                                     _lib.current_stream())
    assert rc == _lib.BSX_ERR_WORKSPACE
    assert b'exceeds the built-in queue' in bsx.bsx_last_error_string()
    torch.cuda.synchronize()
    assert bool((out == 5.0).all())              # nothing was launched
    # just inside the limit it runs
    batch = 14
    got = _static(bsx, conn, spk[:batch], _lib.SPK_BOOL8, batch, n_post)
    assert bool((got == 0).all())
