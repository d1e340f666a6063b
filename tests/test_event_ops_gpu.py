"""GPU parity: every product of the C-ABI library against the CPU oracle on the
same seeded inputs, at the reference's test shapes, at ragged/edge shapes and at
the full size of the standalone microbenchmark (65 536 x 65 536, p = 0.01).

Tolerances: integer/index work is compared bit for bit; float32 sums within
rtol 1e-5 / atol 1e-6 (``brainstate/_testing.py:56-57``), with the absolute term
scaled by the sum of magnitudes where a row mixes signs.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import event_oracle as eo

pytestmark = pytest.mark.gpu

GOLD = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'event_golden.npz'))
RTOL, ATOL = 1e-5, 1e-6


def close(actual, desired, scale=1.0):
    a = actual.detach().cpu().numpy() if isinstance(actual, torch.Tensor) else np.asarray(actual)
    np.testing.assert_allclose(a, desired, rtol=RTOL, atol=ATOL * scale)


def make(n_pre, n_post, K, seed, hetero, cuda, csr_ratio=None):
    from brainstate_b200 import FixedPostNumConn, CSR
    rs = np.random.RandomState(seed + 77)
    if csr_ratio is None:
        idx = eo.fixed_num_indices(seed, n_pre, n_post, K)
        indptr = None
    else:
        idx, indptr, _ = eo.afferent_csr(seed, n_pre, n_post, K, csr_ratio)
    w = rs.uniform(0.05, 0.15, size=idx.shape).astype(np.float32) if hetero else np.float32(0.1)
    ti = torch.from_numpy(idx).to(cuda)
    tw = torch.as_tensor(w, device=cuda)
    if indptr is None:
        conn = FixedPostNumConn((tw, ti), shape=(n_pre, n_post))
    else:
        conn = CSR((tw, ti, torch.from_numpy(indptr).to(cuda)), shape=(n_pre, n_post))
    return conn, idx, indptr, w


SHAPES = [(20, 30, 3), (20, 40, 4), (33, 1000, 17), (64, 128, 128), (257, 513, 131), (1000, 96, 7)]


@pytest.mark.parametrize('shape', SHAPES)
@pytest.mark.parametrize('hetero', [False, True])
@pytest.mark.parametrize('layout', ['fixed', 'csr'])
def test_event_vecmat_matches_oracle(shape, hetero, layout, cuda):
    from brainstate_b200 import EventArray
    n_pre, n_post, K = shape
    conn, idx, indptr, w = make(n_pre, n_post, K, 5, hetero, cuda, 0.6 if layout == 'csr' else None)
    conn.validate()
    rs = np.random.RandomState(9)
    for rate in (0.0, 0.05, 0.3, 1.0):
        spk = rs.random_sample(n_pre) < rate
        ref = eo.event_vecmat(spk, idx, w, n_post, indptr)
        for t in (torch.from_numpy(spk).to(cuda),                                   # bool
                  torch.from_numpy(spk.astype(np.uint8)).to(cuda),                  # uint8
                  torch.from_numpy((spk * rs.uniform(0.5, 2, n_pre)).astype(np.float32)).to(cuda)):  # float events
            y = EventArray(t) @ conn
            assert y.shape == (n_post,) and y.dtype == torch.float32
            if hetero:
                close(y, ref)
            else:  # identical addends: any summation order gives the same bits
                assert np.array_equal(y.cpu().numpy(), ref)
        yg = conn._vecmat(torch.from_numpy(spk).to(cuda), event=True, method='gather')
        close(yg, ref)


@pytest.mark.parametrize('lead', [(3,), (2, 3), (5, 1)])
def test_leading_batch_dimensions(lead, cuda):
    from brainstate_b200 import EventArray
    n_pre, n_post, K = 70, 90, 9
    conn, idx, _, w = make(n_pre, n_post, K, 3, True, cuda)
    rs = np.random.RandomState(1)
    spk = rs.random_sample(lead + (n_pre,)) < 0.2
    y = EventArray(torch.from_numpy(spk).to(cuda)) @ conn
    assert tuple(y.shape) == lead + (n_post,)
    close(y, eo.event_vecmat(spk, idx, w, n_post))
    x = rs.standard_normal(lead + (n_pre,)).astype(np.float32)
    close(torch.from_numpy(x).to(cuda) @ conn, eo.float_vecmat(x, idx, w, n_post), scale=10)
    v = rs.standard_normal(lead + (n_post,)).astype(np.float32)
    close(conn @ torch.from_numpy(v).to(cuda), eo.float_matvec(v, idx, w, n_pre), scale=10)
    s = rs.random_sample(lead + (n_post,)) < 0.3
    close(conn @ EventArray(torch.from_numpy(s).to(cuda)), eo.event_matvec(s, idx, w, n_pre))


@pytest.mark.parametrize('hetero', [False, True])
def test_unaligned_views_and_ragged_sizes(hetero, cuda):
    """Sliced tensors start off the 16-byte grid; sizes are not multiples of 4 or 32."""
    from brainstate_b200 import EventArray
    n_pre, n_post, K = 101, 203, 13
    conn, idx, _, w = make(n_pre, n_post, K, 8, hetero, cuda)
    rs = np.random.RandomState(4)
    for off in (1, 2, 3, 5):
        spk = rs.random_sample(n_pre + off) < 0.4
        t = torch.from_numpy(spk).to(cuda)[off:]
        close(EventArray(t) @ conn, eo.event_vecmat(spk[off:], idx, w, n_post))
        tf = torch.from_numpy(spk.astype(np.float32)).to(cuda)[off:]
        close(EventArray(tf) @ conn, eo.event_vecmat(spk[off:], idx, w, n_post))
        s = rs.random_sample(n_post + off) < 0.4
        close(conn @ EventArray(torch.from_numpy(s).to(cuda)[off:]), eo.event_matvec(s[off:], idx, w, n_pre))


def test_spike_formats_bits_and_list(bsx, cuda):
    from brainstate_b200 import _lib
    from brainstate_b200.event import pack_spikes, event_matvec
    n_pre, n_post, K = 300, 170, 11
    conn, idx, _, w = make(n_pre, n_post, K, 2, True, cuda)
    rs = np.random.RandomState(6)
    spk = rs.random_sample((3, n_pre)) < 0.25
    bits = pack_spikes(torch.from_numpy(spk).to(cuda))
    assert np.array_equal(bits.cpu().numpy().view(np.uint32),
                          np.stack([eo.pack_bits(s) for s in spk]))
    ref = eo.event_vecmat(spk, idx, w, n_post)
    st = conn._struct()
    ws_bytes = bsx.bsx_event_vecmat_workspace_bytes(3, n_pre)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=cuda)
    out = torch.empty((3, n_post), dtype=torch.float32, device=cuda)
    stream = _lib.current_stream()
    _lib.check(bsx.bsx_event_vecmat(C.byref(st), bits.data_ptr(), _lib.SPK_BITS32, 3, out.data_ptr(), 0,
                                    ws.data_ptr(), ws_bytes, stream))
    close(out, ref)
    # accumulate=1 adds onto what is there
    _lib.check(bsx.bsx_event_vecmat(C.byref(st), bits.data_ptr(), _lib.SPK_BITS32, 3, out.data_ptr(), 1,
                                    ws.data_ptr(), ws_bytes, stream))
    close(out, 2 * ref)
    # an index list: count first, then the active rows
    act = np.nonzero(spk[0])[0].astype(np.int32)
    lst = torch.from_numpy(np.concatenate([[act.size], act]).astype(np.int32)).to(cuda)
    o1 = torch.empty(n_post, dtype=torch.float32, device=cuda)
    _lib.check(bsx.bsx_event_vecmat(C.byref(st), lst.data_ptr(), _lib.SPK_LIST, 1, o1.data_ptr(), 0, None, 0, stream))
    close(o1, ref[0])
    # matvec from packed words
    s = rs.random_sample((2, n_post)) < 0.3
    close(event_matvec(conn, pack_spikes(torch.from_numpy(s).to(cuda)), bits=True), eo.event_matvec(s, idx, w, n_pre))
    # a too-small workspace is refused, not overrun
    rc = bsx.bsx_event_vecmat(C.byref(st), bits.data_ptr(), _lib.SPK_BITS32, 3, out.data_ptr(), 0, ws.data_ptr(), 64, stream)
    assert rc == _lib.BSX_ERR_WORKSPACE


@pytest.mark.parametrize('c', [0, 1, 2, 3])
def test_golden_fixtures(c, cuda):
    """Committed fixtures (connectivity from the reference's NumPy calls, products
    from an independent restatement of the reference's in-test oracle)."""
    from brainstate_b200 import EventArray, FixedPostNumConn
    from brainstate_b200.nn import EventFixedProb, FixedNumConn
    seed, n_pre, n_post, K = (int(v) for v in GOLD[f'c{c}_meta'])
    layer = EventFixedProb(n_pre, n_post, K, 1.5, seed=seed)
    assert np.array_equal(layer.conn.indices.cpu().numpy(), GOLD[f'c{c}_indices'])     # bit-exact connectivity
    spk = torch.from_numpy(GOLD[f'c{c}_spk']).to(cuda)
    assert np.array_equal(layer(spk).cpu().numpy(), GOLD[f'c{c}_y_event_homo'])
    w = torch.from_numpy(GOLD[f'c{c}_w_het']).to(cuda)
    het = EventFixedProb(n_pre, n_post, K, w, seed=seed)
    close(het(spk), GOLD[f'c{c}_y_event_het'])
    xf = torch.from_numpy(GOLD[f'c{c}_xf']).to(cuda)
    close(het(xf), GOLD[f'c{c}_y_event_het'])
    flt = FixedNumConn(n_pre, n_post, K, w, seed=seed)
    close(flt(xf), GOLD[f'c{c}_y_float_het'])
    sub = FixedNumConn(n_pre, n_post, K, 1.0, seed=seed, afferent_ratio=0.5)
    assert np.array_equal(sub.pre_selected, GOLD[f'c{c}_pre_selected'])
    assert np.array_equal(sub.conn.indices.cpu().numpy(), GOLD[f'c{c}_indices'][GOLD[f'c{c}_pre_selected']].reshape(-1))
    # reverse mode through autograd
    ct = torch.from_numpy(GOLD[f'c{c}_ct']).to(cuda)
    x = xf.clone().requires_grad_(True)
    wp = w.clone().requires_grad_(True)
    flt.weight.value = wp
    (flt(x) * ct).sum().backward()
    close(x.grad, GOLD[f'c{c}_dx_het'], scale=20)
    close(wp.grad, GOLD[f'c{c}_dw_het_float'])
    x2 = xf.clone().requires_grad_(True)
    wp2 = w.clone().requires_grad_(True)
    het.weight.value = wp2
    (het(x2) * ct).sum().backward()
    close(x2.grad, GOLD[f'c{c}_dx_het'], scale=20)
    close(wp2.grad, GOLD[f'c{c}_dw_het_event'])
    wh = torch.tensor(1.5, device=cuda, requires_grad=True)
    layer.weight.value = wh
    (layer(spk) * ct).sum().backward()
    close(wh.grad, GOLD[f'c{c}_dw_homo_event'], scale=20)


@pytest.mark.parametrize('homo_w', [True, False])
def test_vjp_like_the_reference_test(homo_w, cuda):
    """``brainstate/nn/_event_fixedprob_test.py:56-88``: n_in=20, n_out=30, p=0.1, seed=123."""
    from brainstate_b200.nn import EventFixedProb
    n_in, n_out = 20, 30
    rs = np.random.RandomState(0)
    xn = (rs.random_sample(n_in) < 0.3).astype(np.float32)
    init = (lambda shape: rs.uniform(-0.5, 0.5, shape).astype(np.float32))
    fn = EventFixedProb(n_in, n_out, 0.1, 1.5 if homo_w else init, seed=123)
    assert fn.conn_num == 3
    x = torch.from_numpy(xn).to(cuda).requires_grad_(True)
    w = fn.weight.value.clone().requires_grad_(True)
    fn.weight.value = w
    fn(x).sum().backward()
    idx = fn.conn.indices.cpu().numpy()
    wn = w.detach().cpu().numpy()
    dx, dw = eo.vecmat_vjp(xn, np.ones(n_out, np.float32), idx, wn, event=True)
    close(x.grad, dx)
    close(w.grad, dw)
    # a bool spike vector is not differentiable; the weight still is
    w2 = fn.weight.value.detach().clone().requires_grad_(True)
    fn.weight.value = w2
    fn(torch.from_numpy(xn != 0).to(cuda)).sum().backward()
    close(w2.grad, dw)


@pytest.mark.parametrize('homo_w', [True, False])
def test_jvp_like_the_reference_test(homo_w, cuda):
    """``brainstate/nn/_event_fixedprob_test.py:90-126`` with forward-mode AD."""
    import torch.autograd.forward_ad as fwAD
    from brainstate_b200.nn import EventFixedProb
    n_in, n_out = 20, 30
    rs = np.random.RandomState(1)
    xn = (rs.random_sample(n_in) < 0.3).astype(np.float32)
    init = (lambda shape: rs.uniform(-0.5, 0.5, shape).astype(np.float32))
    fn = EventFixedProb(n_in, n_out, 0.1, 1.5 if homo_w else init, seed=123)
    w = fn.weight.value
    x = torch.from_numpy(xn).to(cuda)
    with fwAD.dual_level():
        fn.weight.restore_value(fwAD.make_dual(w, torch.ones_like(w)))
        out = fn(fwAD.make_dual(x, torch.ones_like(x)))
        primal, tangent = fwAD.unpack_dual(out)
    fn.weight.restore_value(w)
    idx = fn.conn.indices.cpu().numpy()
    wn = w.cpu().numpy()
    close(primal, eo.event_vecmat(xn, idx, wn, n_out))
    ref = eo.vecmat_jvp(xn, np.ones(n_in, np.float32), np.ones_like(wn), idx, wn, n_out, event=True)
    np.testing.assert_allclose(tangent.cpu().numpy(), ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize('hetero', [False, True])
@pytest.mark.parametrize('batch', [1, 3, 4, 37, 70])
def test_raw_vjp_entry_point(hetero, batch, bsx, cuda, c_oracle):
    from brainstate_b200.event import _raw_vjp
    n_pre, n_post, K = 150, 220, 21
    for layout in (None, 0.5):
        conn, idx, indptr, w = make(n_pre, n_post, K, 12, hetero, cuda, layout)
        rs = np.random.RandomState(13)
        x = (rs.standard_normal((batch, n_pre)) * (rs.random_sample((batch, n_pre)) < 0.4)).astype(np.float32)
        ct = rs.standard_normal((batch, n_post)).astype(np.float32)
        for event in (False, True):
            dx_ref, dw_ref = eo.vecmat_vjp(x, ct, idx, w, indptr, event=event)
            for need_dx in (True, False):
                dx, dw = _raw_vjp(conn, torch.from_numpy(x).to(cuda), conn.data, torch.from_numpy(ct).to(cuda),
                                  event, need_dx, True)
                if need_dx:
                    close(dx, dx_ref, scale=30)
                close(dw.reshape(np.shape(dw_ref)), dw_ref, scale=30 * (1 if hetero else 50))


def test_batched_training_step_at_microbenchmark_size(microbench, c_oracle, cuda):
    """The batched event matmul with gradient: 64 x 65 536 spikes at 2 %, dense N(0,1)
    cotangent; forward, input cotangent and weight cotangent against the C oracle."""
    from brainstate_b200 import FixedPostNumConn
    from brainstate_b200.event import _raw_vjp
    n, K, idx, w, ti, tw = microbench
    B = 64
    spk = np.random.RandomState(220).random_sample((B, n)) < 0.02
    ct = np.random.RandomState(221).standard_normal((B, n)).astype(np.float32)
    het = FixedPostNumConn((tw, ti), shape=(n, n))
    ts, tct = torch.from_numpy(spk).to(cuda), torch.from_numpy(ct).to(cuda)
    y = het._vecmat(ts, event=True)
    close(y, c_oracle.event_vecmat_u8(spk, idx, w, n))
    yg = het._vecmat(ts, event=True, method='gather')
    close(yg, c_oracle.event_vecmat_u8(spk, idx, w, n))
    dx, dw = _raw_vjp(het, ts, tw, tct, True, True, True)
    close(dx, c_oracle.float_matvec(ct, idx, w, n), scale=30)
    close(dw, c_oracle.vecmat_dw(spk.astype(np.float32), ct, idx, n, n, event=True), scale=30)
    dx2, dw2 = _raw_vjp(het, ts, tw, tct, True, True, True)
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2)         # no atomics: reproducible


@pytest.mark.parametrize('n_post', [1000, 32768, 40001, 70003, 131072])
@pytest.mark.parametrize('hetero', [False, True])
def test_batched_scatter_with_output_in_shared_memory(n_post, hetero, bsx, cuda):
    """The opt-in scatter that keeps output slices in shared memory (batches of 16 or
    more over at most 131 072 columns; blocks_per_sm = -1 in the tuned entry point) must
    agree with the oracle for every spike format, for CSR rows and when accumulating."""
    from brainstate_b200 import _lib, EventArray
    from brainstate_b200.event import pack_spikes
    n_pre, K, B = 777, 29, 19
    rs = np.random.RandomState(n_post % 97)
    for layout in (None, 0.7):
        conn, idx, indptr, w = make(n_pre, n_post, K, 41, hetero, cuda, layout)
        spk = rs.random_sample((B, n_pre)) < 0.15
        ref = eo.event_vecmat(spk, idx, w, n_post, indptr)
        ts = torch.from_numpy(spk).to(cuda)
        st = conn._struct()
        ws_bytes = bsx.bsx_event_vecmat_workspace_bytes(B, n_pre)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=cuda)
        stream = _lib.current_stream()

        def smem_scatter(t, fmt, out, accumulate=0):
            _lib.check(bsx.bsx_event_vecmat_tuned(C.byref(st), t.data_ptr(), fmt, B, out.data_ptr(), accumulate,
                                                  ws.data_ptr(), ws_bytes, 0, -1, stream))
            return out

        y = smem_scatter(ts, _lib.SPK_BOOL8, torch.full((B, n_post), 9.0, device=cuda))
        if hetero:
            close(y, ref)
        else:   # homogeneous weights: integer hit counts times the weight, rounded once — exactly
            counts = eo.event_vecmat(spk, idx, np.float32(1.0), n_post, indptr)
            assert np.array_equal(y.cpu().numpy(), (counts * np.float32(w)).astype(np.float32))
            close(y, ref)
        xf = torch.from_numpy((spk * rs.uniform(0.5, 2, spk.shape)).astype(np.float32)).to(cuda)
        close(smem_scatter(xf, _lib.SPK_F32, torch.empty_like(y)), ref)            # float spikes are events
        bits = pack_spikes(ts)
        close(smem_scatter(bits, _lib.SPK_BITS32, y.clone(), accumulate=1), 2 * ref)
        close(EventArray(ts) @ conn, ref)                                          # the default kernel, same input


def test_host_buffer_pipeline_equals_device_path(cuda):
    """Pinned host spikes in, pinned host results out, chunks overlapped on three streams."""
    from brainstate_b200 import EventArray
    from brainstate_b200.host import HostEventProducts
    n, K = 1000, 37
    conn, idx, _, w = make(n, n, K, 31, True, cuda)
    rs = np.random.RandomState(32)
    for T in (5, 16, 50):
        spk = rs.random_sample((T, n)) < 0.05
        hs = torch.from_numpy(spk).pin_memory()
        h1 = torch.empty((T, n), dtype=torch.float32).pin_memory()
        h2 = torch.empty((T, n), dtype=torch.float32).pin_memory()
        pipe = HostEventProducts(conn, chunk=16)
        pipe(hs, h1, h2)
        pipe(hs, h1, h2)                                   # reusable
        torch.cuda.synchronize()
        close(h1, eo.event_vecmat(spk, idx, w, n))
        close(h2, eo.event_matvec(spk, idx, w, n))
        d2 = conn @ EventArray(torch.from_numpy(spk).to(cuda))
        assert torch.equal(h2.to(cuda), d2)
    with pytest.raises(ValueError):
        HostEventProducts(conn)(torch.from_numpy(spk), h1, h2)         # not pinned


def test_transposed_copy_is_canonical(cuda):
    n_pre, n_post, K = 123, 77, 19
    for layout in (None, 0.5):
        conn, idx, indptr, w = make(n_pre, n_post, K, 21, True, cuda, layout)
        t = conn.transposed()
        flat = idx.reshape(-1)
        order = np.argsort(flat, kind='stable')                # ascending column, then position
        assert np.array_equal(t.perm.cpu().numpy(), order.astype(np.int32))
        counts = np.bincount(flat, minlength=n_post)
        assert np.array_equal(t.indptr.cpu().numpy(), np.concatenate([[0], np.cumsum(counts)]))
        starts = np.arange(n_pre + 1) * K if indptr is None else indptr
        rows = np.searchsorted(starts, order, side='right') - 1
        assert np.array_equal(t.indices.cpu().numpy(), rows.astype(np.int32))


def test_validate_catches_bad_indices(cuda):
    from brainstate_b200 import FixedPostNumConn, CSR
    idx = torch.randint(0, 50, (40, 6), dtype=torch.int32, device=cuda)
    conn = FixedPostNumConn((1.0, idx), shape=(40, 50))
    conn.validate()
    bad = idx.clone()
    bad[17, 3] = 50
    with pytest.raises(ValueError):
        FixedPostNumConn((1.0, bad), shape=(40, 50)).validate()
    bad[17, 3] = -1
    with pytest.raises(ValueError):
        FixedPostNumConn((1.0, bad), shape=(40, 50)).validate()
    indptr = torch.arange(0, 41, dtype=torch.int32, device=cuda) * 6
    CSR((1.0, idx.reshape(-1), indptr), shape=(40, 50)).validate()
    indptr[5] = 100
    with pytest.raises(ValueError):
        CSR((1.0, idx.reshape(-1), indptr), shape=(40, 50)).validate()


def test_zero_connection_and_empty_inputs(cuda):
    from brainstate_b200.nn import FixedNumConn, EventFixedProb
    m = FixedNumConn(20, 40, 0.0, 1.0, seed=1)
    assert m.conn_num == 0
    out = m(torch.rand(20, device=cuda))
    assert out.shape == (40,) and bool((out == 0).all())
    out = EventFixedProb(20, 40, 0.0, 1.0, seed=1)(torch.rand(3, 20, device=cuda) < 0.5)
    assert out.shape == (3, 40) and bool((out == 0).all())
    ev = EventFixedProb(20, 40, 0.1, 1.0, seed=123)
    assert bool((ev(torch.zeros(20, dtype=torch.bool, device=cuda)) == 0).all())
    assert ev(torch.zeros((0, 20), dtype=torch.bool, device=cuda)).shape == (0, 40)
    sub = FixedNumConn(20, 40, 0.2, 1.0, afferent_ratio=0.5, seed=1)
    assert sub.pre_selected.shape == (20,) and sub(torch.rand(20, device=cuda)).shape == (40,)
    m1 = FixedNumConn(20, 40, 0.2, 1.0, afferent_ratio=0.5, seed=7)
    m2 = FixedNumConn(20, 40, 0.2, 1.0, afferent_ratio=0.5, seed=7)
    assert np.array_equal(m1.pre_selected, m2.pre_selected)
    nr = FixedNumConn(20, 40, 0.2, 1.0, seed=3, allow_multi_conn=False, conn_init='for_loop')
    assert nr(torch.rand(20, device=cuda)).shape == (40,)


def test_event_update_matches_scatter_reference(cuda):
    """``brainstate/nn/_event_fixedprob_test.py:247-260``."""
    from brainstate_b200.nn import EventFixedProb
    n_in, n_out = 20, 30
    fn = EventFixedProb(n_in, n_out, 0.2, 1.5, seed=11)
    spk = (np.random.RandomState(2).random_sample(n_in) < 0.3).astype(np.float32)
    out = fn(torch.from_numpy(spk).to(cuda)).cpu().numpy()
    indices = fn.conn.indices.cpu().numpy()
    ref = np.zeros((n_out,))
    for i in range(n_in):
        np.add.at(ref, indices[i], 1.5 * float(spk[i]))
    assert np.allclose(out, ref, rtol=1e-4, atol=1e-4)


def test_event_linear(cuda):
    from brainstate_b200.nn import EventLinear
    spk = torch.from_numpy(GOLD['dense_spk']).to(cuda)
    for fae, expect in ((True, GOLD['dense_event_true']), (False, GOLD['dense_event_false'])):
        y = EventLinear(10, 6, 1.5, float_as_event=fae)(spk)
        assert y.shape == (6,) and bool((y == float(expect)).all())
    rs = np.random.RandomState(3)
    for (n_in, n_out, lead) in ((10, 6, ()), (300, 1030, (3,)), (2500, 257, (2, 2))):
        W = rs.standard_normal((n_in, n_out)).astype(np.float32)
        s = (rs.random_sample(lead + (n_in,)) < 0.3)
        sf = (s * rs.uniform(0.5, 2, s.shape)).astype(np.float32)
        layer = EventLinear(n_in, n_out, W, float_as_event=True)
        for t in (torch.from_numpy(s).to(cuda), torch.from_numpy(sf).to(cuda)):
            y = layer(t)
            assert tuple(y.shape) == lead + (n_out,)
            close(y, eo.event_linear(s, W, n_out, True), scale=100)
        y2 = EventLinear(n_in, n_out, W, float_as_event=False)(torch.from_numpy(sf).to(cuda))
        np.testing.assert_allclose(y2.cpu().numpy(), sf @ W, rtol=1e-4, atol=1e-3)
    # gradients of the event product: d spk = ct @ W^T, dW = [spk != 0]^T ct
    W = torch.from_numpy(rs.standard_normal((10, 6)).astype(np.float32)).to(cuda).requires_grad_(True)
    x = spk.clone().requires_grad_(True)
    layer = EventLinear(10, 6, W)
    layer(x).sum().backward()
    close(x.grad, W.detach().sum(dim=1).cpu().numpy(), scale=10)
    close(W.grad, ((spk != 0).float()[:, None] * torch.ones(6, device=cuda)).cpu().numpy())


def test_event_linear_kernels_at_a_realistic_size(bsx, cuda):
    """The dense event layer at 8192 x 4096 with a batch of 24: forward, the weight cotangent
    ``[spk != 0]^T @ ct`` (own kernel, ascending batch order, rows that never fired are zeros)
    and the scalar-weight form with its gradients, against NumPy in float64."""
    from brainstate_b200.nn import EventLinear
    rs = np.random.RandomState(11)
    n_in, n_out, B = 8192, 4096, 24
    W = rs.standard_normal((n_in, n_out)).astype(np.float32)
    s = rs.random_sample((B, n_in)) < 0.02
    s[:, 5] = False                                             # a neuron that never fires
    sf = (s * rs.uniform(0.5, 2, s.shape)).astype(np.float32)
    ct = rs.standard_normal((B, n_out)).astype(np.float32)
    Wt = torch.from_numpy(W).to(cuda).requires_grad_(True)
    x = torch.from_numpy(sf).to(cuda).requires_grad_(True)
    layer = EventLinear(n_in, n_out, Wt)
    y = layer(x)
    ref = s.astype(np.float64) @ W.astype(np.float64)
    np.testing.assert_allclose(y.detach().cpu().numpy(), ref, rtol=1e-5, atol=2e-4)
    (y * torch.from_numpy(ct).to(cuda)).sum().backward()
    dW = s.astype(np.float64).T @ ct.astype(np.float64)
    np.testing.assert_allclose(Wt.grad.cpu().numpy(), dW, rtol=1e-5, atol=1e-5)
    assert bool((Wt.grad[5] == 0).all())
    np.testing.assert_allclose(x.grad.cpu().numpy(), ct.astype(np.float64) @ W.astype(np.float64).T, rtol=1e-4, atol=2e-3)
    # boolean spikes take the same kernels
    yb = layer(torch.from_numpy(s).to(cuda))
    assert torch.equal(yb, y.detach())
    # scalar weight: count or value sum, broadcast; gradients through the value sum
    for fae in (True, False):
        w0 = torch.tensor(1.5, device=cuda, requires_grad=True)
        xs = torch.from_numpy(sf).to(cuda).requires_grad_(True)
        ys = EventLinear(n_in, n_out, w0, float_as_event=fae)(xs)
        r = s.sum(axis=1).astype(np.float64) if fae else sf.astype(np.float64).sum(axis=1)
        np.testing.assert_allclose(ys.detach().cpu().numpy(), np.repeat((r * 1.5)[:, None], n_out, 1), rtol=1e-5)
        (ys * torch.from_numpy(ct).to(cuda)).sum().backward()
        row = ct.astype(np.float64).sum(axis=1)
        np.testing.assert_allclose(float(w0.grad), float((row * r).sum()), rtol=1e-4)
        np.testing.assert_allclose(xs.grad.cpu().numpy(), np.repeat((1.5 * row)[:, None], n_in, 1), rtol=1e-4, atol=1e-5)


@pytest.fixture(scope='module')
def microbench(cuda, c_oracle):
    """The standalone microbenchmark matrix at full size: 65 536^2, p = 0.01."""
    n, K = 65536, 655
    idx = c_oracle.fixed_num_indices(200, n, n, K)
    w = np.random.RandomState(201).normal(0.1, 0.01, (n, K)).astype(np.float32)
    return n, K, idx, w, torch.from_numpy(idx).to(cuda), torch.from_numpy(w).to(cuda)


@pytest.mark.parametrize('rate_id', [0, 1, 2])
def test_microbenchmark_size_against_c_oracle(rate_id, microbench, c_oracle, cuda):
    from brainstate_b200 import EventArray, FixedPostNumConn
    from brainstate_b200.nn import fixed_num_indices
    n, K, idx, w, ti, tw = microbench
    rate = (0.001, 0.01, 0.1)[rate_id]
    if rate_id == 0:
        assert np.array_equal(fixed_num_indices(200, n, n, K), idx)
    spk = np.random.RandomState(210 + rate_id).random_sample((2, n)) < rate
    ts = torch.from_numpy(spk).to(cuda)
    het = FixedPostNumConn((tw, ti), shape=(n, n))
    hom = FixedPostNumConn((0.1, ti), shape=(n, n))
    ref_het = c_oracle.event_vecmat_u8(spk, idx, w, n)
    ref_hom = c_oracle.event_vecmat_u8(spk, idx, np.float32(0.1), n)
    close(EventArray(ts) @ het, ref_het)
    assert np.array_equal((EventArray(ts) @ hom).cpu().numpy(), ref_hom)
    close(het @ EventArray(ts), c_oracle.event_matvec_u8(spk, idx, w, n))
    close(hom @ EventArray(ts), c_oracle.event_matvec_u8(spk, idx, np.float32(0.1), n))
    # size-independent properties: linearity in the spikes and agreement of the two
    # forward variants (scatter vs deterministic gather over the transposed copy)
    a, b = ts[0] & ~ts[1], ts[1] & ~ts[0]
    both = a | b
    close((EventArray(a) @ hom) + (EventArray(b) @ hom), (EventArray(both) @ hom).cpu().numpy(), scale=10)
    if rate_id == 1:
        yg = het._vecmat(ts, event=True, method='gather')
        close(yg, ref_het)
        yg2 = het._vecmat(ts, event=True, method='gather')
        assert torch.equal(yg, yg2)                    # deterministic
        ct = np.random.RandomState(221).standard_normal((1, n)).astype(np.float32)
        dx = het @ torch.from_numpy(ct).to(cuda)
        close(dx, c_oracle.float_matvec(ct, idx, w, n), scale=30)


@pytest.mark.parametrize('shape', [(20, 30, 3), (33, 1000, 17), (257, 513, 131), (1000, 96, 7)])
@pytest.mark.parametrize('hetero', [False, True])
@pytest.mark.parametrize('layout', ['fixed', 'csr'])
def test_event_driven_matvec_over_the_transposed_copy(shape, hetero, layout, cuda):
    """``W @ spikes`` with ``method='scatter'``: the active columns scatter along the transposed
    copy.  Same sums as the gather within tolerance; reproducible for homogeneous weights."""
    from brainstate_b200 import EventArray
    from brainstate_b200.event import event_matvec, pack_spikes
    n_pre, n_post, K = shape
    conn, idx, indptr, w = make(n_pre, n_post, K, 41, hetero, cuda, 0.6 if layout == 'csr' else None)
    rs = np.random.RandomState(42)
    for rate in (0.0, 0.02, 0.3, 1.0):
        for lead in ((), (5,), (2, 9)):
            spk = rs.random_sample(lead + (n_post,)) < rate
            ts = torch.from_numpy(spk).to(cuda)
            ref = eo.event_matvec(spk.reshape(-1, n_post), idx, w, n_pre, indptr=indptr).reshape(lead + (n_pre,))
            y = event_matvec(conn, ts, method='scatter')
            assert y.shape == ref.shape
            if hetero:
                close(y, ref)
            else:
                assert torch.equal(y, event_matvec(conn, ts, method='scatter'))   # identical addends: any order, one sum
                close(y, ref)
            close(event_matvec(conn, pack_spikes(ts), bits=True, method='scatter'), ref)
    conn.matvec_method = 'scatter'                                     # what ``conn @ EventArray`` uses
    close(conn @ EventArray(ts), ref)
    with pytest.raises(ValueError):
        event_matvec(conn, ts, method='sorted')


def test_transposed_weights_follow_the_weight_tensor(cuda):
    """The permuted weight copy behind the event-driven matvec is kept between calls and
    refreshed after an in-place update or ``with_data``."""
    from brainstate_b200.event import event_matvec
    n_pre, n_post, K = 300, 200, 11
    conn, idx, _, w = make(n_pre, n_post, K, 43, True, cuda)
    spk = np.random.RandomState(44).random_sample(n_post) < 0.2
    ts = torch.from_numpy(spk).to(cuda)
    close(event_matvec(conn, ts, method='scatter'), eo.event_matvec(spk, idx, w, n_pre))
    kept = conn._derived['w_t'][1]
    event_matvec(conn, ts, method='scatter')
    assert conn._derived['w_t'][1] is kept                                   # no second permutation
    conn.data.mul_(2.0)                                                 # optimiser-style in-place step
    close(event_matvec(conn, ts, method='scatter'), eo.event_matvec(spk, idx, 2 * w, n_pre))
    w3 = (3 * w).astype(np.float32)
    c3 = conn.with_data(torch.from_numpy(w3).to(cuda))
    close(event_matvec(c3, ts, method='scatter'), eo.event_matvec(spk, idx, w3, n_pre))
    close(event_matvec(conn, ts, method='scatter'), eo.event_matvec(spk, idx, 2 * w, n_pre))


def test_host_buffer_pipeline_event_driven_reverse(cuda):
    from brainstate_b200.host import HostEventProducts
    n, K = 1000, 37
    conn, idx, _, w = make(n, n, K, 31, True, cuda)
    spk = np.random.RandomState(45).random_sample((40, n)) < 0.02
    hs = torch.from_numpy(spk).pin_memory()
    h1 = torch.empty((40, n), dtype=torch.float32).pin_memory()
    h2 = torch.empty((40, n), dtype=torch.float32).pin_memory()
    pipe = HostEventProducts(conn, chunk=16, reverse_method='scatter')
    pipe(hs, h1, h2)
    pipe(hs, h1, h2)
    torch.cuda.synchronize()
    close(h1, eo.event_vecmat(spk, idx, w, n))
    close(h2, eo.event_matvec(spk, idx, w, n))
    with pytest.raises(ValueError):
        HostEventProducts(conn, reverse_method='sorted')


@pytest.mark.parametrize('rate', [0.0, 0.02, 0.5, 1.0])
def test_shared_memory_scatter_lists_many_presynaptic_rows(rate, bsx, cuda):
    """More presynaptic neurons than one round of the in-block row list holds (2048): sparse
    vectors take one round over the whole vector, dense ones fall back to 2048-neuron spans.
    Odd sizes put the byte, float and word scans on unaligned starts."""
    from brainstate_b200 import _lib
    from brainstate_b200.event import pack_spikes
    n_pre, n_post, K, B = 20011, 40001, 5, 17
    conn, idx, indptr, w = make(n_pre, n_post, K, 47, True, cuda)
    spk = np.random.RandomState(48).random_sample((B, n_pre)) < rate
    ref = eo.event_vecmat(spk, idx, w, n_post)
    ts = torch.from_numpy(spk).to(cuda)
    st = conn._struct()
    stream = _lib.current_stream()
    for t, fmt in ((ts, _lib.SPK_BOOL8), (ts.to(torch.float32) * 3.0, _lib.SPK_F32), (pack_spikes(ts), _lib.SPK_BITS32)):
        out = torch.full((B, n_post), 7.0, device=cuda)
        _lib.check(bsx.bsx_event_vecmat_tuned(C.byref(st), t.data_ptr(), fmt, B, out.data_ptr(), 0, None, 0, 0, -1, stream))
        close(out, ref, scale=4)


@pytest.mark.parametrize('n_post', [1000, 32768, 40001, 70003, 131072])
@pytest.mark.parametrize('layout', ['fixed', 'csr'])
def test_rows_grouped_by_output_slice(n_post, layout, bsx, cuda):
    """``bsx_sliced_build``: every row's entries grouped by ``column // 32768``; inside a group
    sorted by shared-memory bank (``column % 32``, stable) and dealt round-robin over the group's
    32-entry stretches.  Offsets, regrouped targets and the permutation bit for bit against NumPy."""
    from brainstate_b200 import _lib
    n_pre, K = 333, 157
    conn, idx, indptr, w = make(n_pre, n_post, K, 51, True, cuda, 0.7 if layout == 'csr' else None)
    S = int(bsx.bsx_sliced_slices(n_post))
    assert S == (n_post + 32767) // 32768
    flat = idx.reshape(-1)
    ip = indptr if indptr is not None else np.arange(n_pre + 1, dtype=np.int64) * K
    ref_ptr = np.empty(n_pre * S + 1, dtype=np.int64)
    ref_idx, ref_perm = np.full_like(flat, -7), np.full(flat.size, -7, dtype=np.int32)
    for i in range(n_pre):
        s, e = int(ip[i]), int(ip[i + 1])
        sl = flat[s:e] // 32768
        start = s
        for k in range(S):
            ref_ptr[i * S + k] = start
            members = np.nonzero(sl == k)[0]                       # original order
            n = members.size
            by_bank = members[np.argsort(flat[s:e][members] % 32, kind='stable')]
            J = (n + 31) // 32
            m = n - 32 * (J - 1)
            for ks, src in enumerate(by_bank):
                if ks < m * J:
                    stretch, slot = ks % J, ks // J
                else:
                    k2 = ks - m * J
                    stretch, slot = k2 % (J - 1), m + k2 // (J - 1)
                ref_idx[start + 32 * stretch + slot] = flat[s + src]
                ref_perm[start + 32 * stretch + slot] = s + src
            start += n
    ref_ptr[-1] = flat.size
    assert (ref_perm >= 0).all()                                   # the dealing is a bijection
    s_indptr, s_indices, s_perm = conn._group_offsets(conn._struct(), n_pre, regroup=True)
    assert np.array_equal(s_indptr.cpu().numpy(), ref_ptr)
    assert np.array_equal(s_indices.cpu().numpy(), ref_idx)
    assert np.array_equal(s_perm.cpu().numpy(), ref_perm)
    # full stretches of a group hold one entry per bank unless a bank has more entries than stretches
    only_ptr = conn._group_offsets(conn._struct(), n_pre, regroup=False)[0]
    assert torch.equal(only_ptr, s_indptr)
    st = conn._struct()
    assert bsx.bsx_sliced_build(C.byref(st), s_indptr.data_ptr(), s_indices.data_ptr(), None, None) == _lib.BSX_ERR_INVALID_ARG


@pytest.mark.parametrize('n_post', [1000, 40001, 70003, 131072])
@pytest.mark.parametrize('hetero', [False, True])
def test_scatter_over_rows_grouped_by_slice(n_post, hetero, bsx, cuda):
    """``bsx_event_vecmat_sliced`` on the regrouped copy (and on the transposed copy with group
    offsets only) against the oracle, for every spike format and when accumulating."""
    from brainstate_b200 import _lib
    from brainstate_b200.event import pack_spikes, event_matvec
    n_pre, K, B = 777, 29, 19
    rs = np.random.RandomState(n_post % 89)
    for layout in (None, 0.7):
        conn, idx, indptr, w = make(n_pre, n_post, K, 53, hetero, cuda, layout)
        spk = rs.random_sample((B, n_pre)) < 0.15
        ref = eo.event_vecmat(spk, idx, w, n_post, indptr)
        ts = torch.from_numpy(spk).to(cuda)
        st = conn._sliced_struct(conn.data)
        stream = _lib.current_stream()

        def sliced(t, fmt, out, accumulate=0):
            _lib.check(bsx.bsx_event_vecmat_sliced(C.byref(st), t.data_ptr(), fmt, B, out.data_ptr(), accumulate, stream))
            return out

        y = sliced(ts, _lib.SPK_BOOL8, torch.full((B, n_post), 9.0, device=cuda))
        close(y, ref)
        if not hetero:      # integer hit counts times the weight, rounded once — exactly
            counts = eo.event_vecmat(spk, idx, np.float32(1.0), n_post, indptr)
            assert np.array_equal(y.cpu().numpy(), (counts * np.float32(w)).astype(np.float32))
        xf = torch.from_numpy((spk * rs.uniform(0.5, 2, spk.shape)).astype(np.float32)).to(cuda)
        close(sliced(xf, _lib.SPK_F32, torch.empty_like(y)), ref)
        close(sliced(pack_spikes(ts), _lib.SPK_BITS32, y.clone(), accumulate=1), 2 * ref)
        # W @ spikes over the transposed copy, whose sorted rows only need the group offsets
        spk_post = rs.random_sample((B, n_post)) < 0.05
        tp = torch.from_numpy(spk_post).to(cuda)
        st_t = conn._transposed_sliced_struct(conn.data)
        yt = torch.empty((B, n_pre), dtype=torch.float32, device=cuda)
        _lib.check(bsx.bsx_event_vecmat_sliced(C.byref(st_t), tp.data_ptr(), _lib.SPK_BOOL8, B, yt.data_ptr(), 0, stream))
        close(yt, eo.event_matvec(spk_post, idx, w, n_pre, indptr=indptr))


def test_large_batches_take_the_sliced_copy(cuda):
    """Batches that fill the GPU go through the copy grouped by output slice, in both directions,
    and agree with the small-batch path."""
    from brainstate_b200 import EventArray, _lib
    from brainstate_b200.event import event_matvec
    n, K, B = 3000, 41, 160
    conn, idx, _, w = make(n, n, K, 55, True, cuda)
    spk = np.random.RandomState(56).random_sample((B, n)) < 0.03
    ts = torch.from_numpy(spk).to(cuda)
    st = conn._struct()
    assert _lib.lib().bsx_event_vecmat_variant(C.byref(st), _lib.SPK_BOOL8, B) == _lib.VECMAT_SHARED_SLICES
    assert _lib.lib().bsx_event_vecmat_variant(C.byref(st), _lib.SPK_BOOL8, 8) == _lib.VECMAT_GLOBAL_ATOMICS
    y = EventArray(ts) @ conn
    assert 'sliced' in conn._derived
    close(y, eo.event_vecmat(spk, idx, w, n))
    close(y[:8], (EventArray(ts[:8]) @ conn).cpu().numpy())
    z = event_matvec(conn, ts, method='scatter')
    assert 't_groups' in conn._derived
    close(z, eo.event_matvec(spk, idx, w, n))


def test_layer_calls_build_the_derived_layouts_once(cuda):
    """``FixedNumConn.update`` goes through ``conn.with_data(weight)`` on every call
    (``brainstate/nn/_event_fixedprob.py:204``): the views share the derived layouts of the
    layer's connectivity, so the transposed and the sliced copy — and the permuted weights,
    as long as the weight tensor is unchanged — are built by the first call only."""
    from brainstate_b200.nn import EventFixedProb
    n, K, B = 3000, 41, 160
    w = np.random.RandomState(71).uniform(0.05, 0.15, (n, K)).astype(np.float32)
    layer = EventFixedProb(n, n, K, w, seed=70)
    idx = layer.conn.indices.cpu().numpy()
    spk = np.random.RandomState(72).random_sample((B, n)) < 0.03
    ts = torch.from_numpy(spk).to(cuda)
    ref = eo.event_vecmat(spk, idx, w, n)
    close(layer(ts), ref)                                   # batch fills the GPU: sliced copy
    sliced, w_s = layer.conn._derived['sliced'], layer.conn._derived['w_s'][1]
    close(layer(ts), ref)
    assert layer.conn._derived['sliced'] is sliced and layer.conn._derived['w_s'][1] is w_s
    layer.method = 'gather'                                 # deterministic form: transposed copy
    close(layer(ts[:3]), ref[:3])
    t, w_t = layer.conn._derived['transposed'], layer.conn._derived['w_t'][1]
    close(layer(ts[:3]), ref[:3])
    assert layer.conn._derived['transposed'] is t and layer.conn._derived['w_t'][1] is w_t
    layer.weight.value.mul_(2.0)                            # an in-place update refreshes the weights only
    close(layer(ts[:3]), 2 * ref[:3])
    assert layer.conn._derived['transposed'] is t and layer.conn._derived['w_t'][1] is not w_t


@pytest.mark.parametrize('layout', ['fixed', 'csr'])
def test_fixed_point_scatter_is_deterministic_and_close(layout, bsx, cuda):
    """``method='fixed'``: the batched scatter with heterogeneous weights summed in 2^-s fixed
    point (s from ``bsx_fixed_scale_log2``: the largest scale the largest column sum of |w|
    cannot overflow).  Order-free, so two runs agree bit for bit; every output within
    (its events) * 2^-(s+1) of the float64 sum, which here is well inside rtol 1e-5 / atol 1e-6;
    both products; mixed-sign weights; all-active input (the overflow bound is reached)."""
    from brainstate_b200 import _lib, EventArray
    from brainstate_b200.event import event_matvec, event_vecmat
    n, K, B = 3000, 41, 160
    conn, idx, indptr, w = make(n, n, K, 57, True, cuda, csr_ratio=0.6 if layout == 'csr' else None)
    w = (w * np.random.RandomState(58).choice([-1.0, 1.0], size=w.shape)).astype(np.float32)
    conn = conn.with_data(torch.from_numpy(w).to(cuda))
    spk = np.random.RandomState(59).random_sample((B, n)) < 0.05
    spk[3] = True                                           # every presynaptic neuron fires in this vector
    ts = torch.from_numpy(spk).to(cuda)
    y1 = event_vecmat(conn, ts, method='fixed')
    y2 = event_vecmat(conn, ts, method='fixed')
    assert torch.equal(y1, y2)
    st_s = conn._sliced_struct(conn.data)
    s = conn._fixed_scale('s', st_s, conn.data)
    col_abs = np.zeros(n)
    np.add.at(col_abs, idx.reshape(-1), np.abs(w.reshape(-1)).astype(np.float64))
    assert s == min(30, int(np.floor(np.log2(2.0 ** 30 / col_abs.max()))))
    exact = np.zeros((B, n))
    starts = np.arange(n + 1) * K if indptr is None else indptr.astype(np.int64)
    for b in range(B):
        for i in np.nonzero(spk[b])[0]:
            np.add.at(exact[b], idx.reshape(-1)[starts[i]:starts[i + 1]], w.reshape(-1)[starts[i]:starts[i + 1]].astype(np.float64))
    events = np.zeros((B, n))
    for b in range(B):
        for i in np.nonzero(spk[b])[0]:
            np.add.at(events[b], idx.reshape(-1)[starts[i]:starts[i + 1]], 1.0)
    err = np.abs(y1.cpu().numpy().astype(np.float64) - exact)
    assert np.all(err <= events * 2.0 ** -(s + 1) + np.abs(exact) * 2.0 ** -23 + 1e-12)
    np.testing.assert_allclose(y1.cpu().numpy(), exact, rtol=RTOL, atol=ATOL)
    z1 = event_matvec(conn, ts, method='fixed')
    assert torch.equal(z1, event_matvec(conn, ts, method='fixed'))
    close(z1, eo.event_matvec(spk, idx, w, n, indptr), scale=3)
    # below 16 vectors the order-fixing gather serves the request
    close(event_vecmat(conn, ts[:3], method='fixed'), exact[:3].astype(np.float32), scale=3)
    # homogeneous weights are counted, which is order-free as it is
    hom, idx_h, _, _ = make(n, n, K, 57, False, cuda)
    yh = event_vecmat(hom, ts, method='fixed')
    counts = eo.event_vecmat(spk, idx_h, np.float32(1.0), n)
    assert np.array_equal(yh.cpu().numpy(), (counts * np.float32(0.1)).astype(np.float32))


@pytest.mark.parametrize('shape', [(30, 20, 3), (513, 257, 131), (96, 1000, 7)])
@pytest.mark.parametrize('hetero', [False, True])
@pytest.mark.parametrize('layout', ['fixed', 'csc'])
def test_in_degree_layouts_match_oracle(shape, hetero, layout, cuda):
    """Connectivity stored by postsynaptic neuron (a fixed number of presynaptic partners, or CSC):
    the arrays are those of the transposed matrix in out-degree form, so the oracle products are
    the matvec / vecmat of that mirror."""
    from brainstate_b200 import EventArray, FixedPreNumConn, CSC
    n_pre, n_post, K = shape
    rs = np.random.RandomState(31)
    if layout == 'fixed':
        idx = eo.fixed_num_indices(17, n_post, n_pre, K)            # (n_post, K) presynaptic ids
        indptr = None
    else:
        idx, indptr, _ = eo.afferent_csr(17, n_post, n_pre, K, 0.6)
    w = rs.uniform(0.05, 0.15, size=idx.shape).astype(np.float32) if hetero else np.float32(0.1)
    ti, tw = torch.from_numpy(idx).to(cuda), torch.as_tensor(w, device=cuda)
    if layout == 'fixed':
        conn = FixedPreNumConn((tw, ti), shape=(n_pre, n_post))
    else:
        conn = CSC((tw, ti, torch.from_numpy(indptr).to(cuda)), shape=(n_pre, n_post))
    conn.validate()
    for batch in (None, 5):
        size = (n_pre,) if batch is None else (batch, n_pre)
        spk = rs.random_sample(size) < 0.2
        ref = np.stack([eo.event_matvec(s, idx, w, n_post, indptr) for s in np.atleast_2d(spk)]).reshape(
            size[:-1] + (n_post,))
        y = EventArray(torch.from_numpy(spk).to(cuda)) @ conn
        assert tuple(y.shape) == size[:-1] + (n_post,)
        close(y, ref)
        y2 = EventArray(torch.from_numpy(spk).to(cuda)) @ conn           # one warp per output, fixed order
        assert torch.equal(y, y2)
        conn.matvec_method = 'scatter'                                    # event-driven form, same sums
        close(EventArray(torch.from_numpy(spk).to(cuda)) @ conn, ref)
        conn.matvec_method = 'gather'
        x = rs.standard_normal(size).astype(np.float32)
        refx = np.stack([eo.float_matvec(v, idx, w, n_post, indptr) for v in np.atleast_2d(x)]).reshape(
            size[:-1] + (n_post,))
        close(torch.from_numpy(x).to(cuda) @ conn, refx, scale=float(np.abs(x).sum() / x.size * K * 10 + 1))
        v = rs.standard_normal(size[:-1] + (n_post,)).astype(np.float32)
        refv = np.stack([eo.float_vecmat(u, idx, w, n_pre, indptr) for u in np.atleast_2d(v)]).reshape(size)
        close(conn @ torch.from_numpy(v).to(cuda), refv, scale=float(K * 10 + 1))
        sp = rs.random_sample(size[:-1] + (n_post,)) < 0.3
        refe = np.stack([eo.event_vecmat(u, idx, w, n_pre, indptr) for u in np.atleast_2d(sp)]).reshape(size)
        close(conn @ EventArray(torch.from_numpy(sp).to(cuda)), refe)


@pytest.mark.parametrize('event', [True, False])
def test_in_degree_layout_reverse_and_forward_mode(event, cuda):
    from brainstate_b200 import EventArray, FixedPreNumConn
    n_pre, n_post, K = 60, 45, 7
    rs = np.random.RandomState(5)
    idx = eo.fixed_num_indices(23, n_post, n_pre, K)
    w = rs.uniform(0.05, 0.15, size=idx.shape).astype(np.float32)
    x = (rs.random_sample((3, n_pre)) < 0.4) * rs.uniform(0.5, 2.0, (3, n_pre))
    x = x.astype(np.float32)
    ct = rs.standard_normal((3, n_post)).astype(np.float32)
    tw = torch.tensor(w, device=cuda, requires_grad=True)
    tx = torch.tensor(x, device=cuda, requires_grad=True)
    conn = FixedPreNumConn((tw, torch.from_numpy(idx).to(cuda)), shape=(n_pre, n_post))
    y = (EventArray(tx) if event else tx) @ conn
    y.backward(torch.from_numpy(ct).to(cuda))
    xv = (x != 0).astype(np.float32) if event else x
    # y[b,j] = sum_k w[j,k] xv[b, idx[j,k]]
    dw = np.einsum('bj,bjk->jk', ct.astype(np.float64), xv[:, idx].astype(np.float64))
    dx = np.zeros((3, n_pre))
    for j in range(n_post):
        for k in range(K):
            dx[:, idx[j, k]] += ct[:, j].astype(np.float64) * w[j, k]
    np.testing.assert_allclose(tw.grad.cpu().numpy(), dw, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(tx.grad.cpu().numpy(), dx, rtol=1e-5, atol=1e-5)
    # forward mode: y_dot = M_w @ x_dot + M_wdot @ x
    import torch.autograd.forward_ad as fwad
    xd = rs.standard_normal((3, n_pre)).astype(np.float32)
    wd = rs.standard_normal(idx.shape).astype(np.float32)
    with fwad.dual_level():
        dxt = fwad.make_dual(torch.tensor(x, device=cuda), torch.from_numpy(xd).to(cuda))
        dwt = fwad.make_dual(torch.tensor(w, device=cuda), torch.from_numpy(wd).to(cuda))
        c2 = FixedPreNumConn((dwt, torch.from_numpy(idx).to(cuda)), shape=(n_pre, n_post))
        out = (EventArray(dxt) if event else dxt) @ c2
        tangent = fwad.unpack_dual(out).tangent
    ref = np.einsum('jk,bjk->bj', w.astype(np.float64), xd[:, idx]) + np.einsum('jk,bjk->bj', wd.astype(np.float64),
                                                                                xv[:, idx])
    np.testing.assert_allclose(tangent.cpu().numpy(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize('n_post', [1000, 40000, 70001])
@pytest.mark.parametrize('hetero', [False, True])
def test_compressed_sliced_layout_equals_the_32_bit_one(n_post, hetero, bsx, cuda):
    """16-bit column offsets inside the slice and weights stored in fixed point: the same sums, bit
    for bit, as the fixed-point (heterogeneous) / counting (homogeneous) scatter over the 32-bit
    sliced copy, and the oracle's within the float tolerance; bool, float and packed spikes;
    accumulate; both products."""
    from brainstate_b200 import _lib, event
    from brainstate_b200.event import event_matvec, event_vecmat, pack_spikes
    n_pre, K, B = 900, 53, 40
    conn, idx, _, w = make(n_pre, n_post, K, 61, hetero, cuda)
    spk = np.random.RandomState(62).random_sample((B, n_pre)) < 0.1
    ts = torch.from_numpy(spk).to(cuda)
    assert event.PACKED_SLICES
    y16 = event_vecmat(conn, ts, method='fixed')
    loc = conn._derived['loc_s']
    assert loc.dtype == torch.int16 and loc.numel() == conn.nnz
    s_idx = conn._derived['sliced'][1].cpu().numpy()
    assert np.array_equal(loc.cpu().numpy().view(np.uint16), (s_idx % 32768).astype(np.uint16))
    try:
        event.PACKED_SLICES = False
        y32 = event_vecmat(conn, ts, method='fixed')
    finally:
        event.PACKED_SLICES = True
    assert torch.equal(y16, y32)
    ref = np.stack([eo.event_vecmat(s, idx, w, n_post) for s in spk])
    close(y16, ref, scale=3)
    # the C entry point itself: float spikes, packed spikes, accumulate
    st_s = conn._sliced_struct(conn.data)
    scale = conn._fixed_scale('s', st_s, conn.data)
    loc, q = conn._packed('s', st_s, conn.data, scale)
    if hetero:
        wq = conn._derived['w_s'][1].cpu().numpy()
        assert np.array_equal(q.cpu().numpy(), np.rint(wq.astype(np.float64) * 2.0 ** scale).astype(np.int32))
    stream = torch.cuda.current_stream().cuda_stream
    for t, fmt, batch in ((ts.to(torch.float32) * 3.0, _lib.SPK_F32, B), (pack_spikes(ts), _lib.SPK_BITS32, B)):
        out = torch.full((B, n_post), 2.0, dtype=torch.float32, device=cuda)
        _lib.check(bsx.bsx_event_vecmat_sliced16(C.byref(st_s), loc.data_ptr(), None if q is None else q.data_ptr(),
                                                 t.data_ptr(), fmt, batch, out.data_ptr(), 1, scale, stream))
        assert torch.equal(out, y32 + 2.0)
    # the transposed product through the compressed copy of the transposed layout
    conn2, idx2, _, w2 = make(n_post, n_pre, 7, 63, hetero, cuda)        # (n_post x n_pre): outputs = n_post rows
    sp2 = np.random.RandomState(64).random_sample((B, n_pre)) < 0.1
    z16 = event_matvec(conn2, torch.from_numpy(sp2).to(cuda), method='fixed')
    try:
        event.PACKED_SLICES = False
        z32 = event_matvec(conn2, torch.from_numpy(sp2).to(cuda), method='fixed')
    finally:
        event.PACKED_SLICES = True
    assert torch.equal(z16, z32)
    close(z16, eo.event_matvec(sp2, idx2, w2, n_post), scale=3)
    # hetero without qweights is refused
    if hetero:
        out = torch.empty((B, n_post), dtype=torch.float32, device=cuda)
        assert bsx.bsx_event_vecmat_sliced16(C.byref(st_s), loc.data_ptr(), None, ts.data_ptr(), _lib.SPK_BOOL8, B,
                                             out.data_ptr(), 0, scale, stream) == _lib.BSX_ERR_INVALID_ARG


def test_bit_packed_spike_delay_feeds_the_event_product(cuda):
    """Ring of packed spike vectors: what was stored d steps ago comes back bit for bit, as words
    for the packed-input product and as bools."""
    from brainstate_b200.nn import SpikeDelay
    from brainstate_b200.event import event_matvec
    n, K = 1000, 11
    conn, idx, _, w = make(300, n, K, 71, True, cuda)
    d = SpikeDelay(n, entries={'syn': 0.5}, dt=0.1, device=cuda)
    assert d.max_length == 6
    d.init_state()
    rs = np.random.RandomState(72)
    past = []
    for t in range(15):
        spk = rs.random_sample(n) < 0.1
        past.append(spk)
        d.update(torch.from_numpy(spk).to(cuda))
        for k in range(min(len(past), 6)):
            assert np.array_equal(d.retrieve_at_step(k, bits=False).cpu().numpy(), past[-1 - k])
            assert np.array_equal(d.retrieve_at_step(k).cpu().numpy().view(np.uint32), eo.pack_bits(past[-1 - k]))
    y = event_matvec(conn, d.at('syn'), bits=True)
    close(y, eo.event_matvec(past[-6], idx, w, 300))
    with pytest.raises(ValueError):
        d.retrieve_at_step(6)
    db = SpikeDelay(n, time=2, device=cuda)
    db.init_state(batch_size=3)
    s3 = rs.random_sample((3, n)) < 0.2
    db.update(torch.from_numpy(s3).to(cuda))
    assert np.array_equal(db.retrieve_at_step(0, bits=False).cpu().numpy(), s3)


@pytest.mark.parametrize('hetero', [False, True])
def test_chained_single_vector_calls(hetero, bsx, cuda):
    """A loop that alternates between two output buffers: every call adds its product into one and
    clears the other for the call that follows (one launch per call, no clearing node)."""
    from brainstate_b200 import _lib
    n_pre, n_post, K = 3000, 2500, 37
    conn, idx, _, w = make(n_pre, n_post, K, 81, hetero, cuda)
    st = conn._struct()
    rs = np.random.RandomState(82)
    bufs = [torch.zeros(n_post, dtype=torch.float32, device=cuda), torch.full((n_post,), 7.0, device=cuda)]
    stream = torch.cuda.current_stream().cuda_stream
    for step in range(6):
        spk = rs.random_sample(n_pre) < 0.03
        ts = torch.from_numpy(spk).to(cuda)
        out, nxt = bufs[step % 2], bufs[(step + 1) % 2]
        _lib.check(bsx.bsx_event_vecmat_chained(C.byref(st), ts.data_ptr(), _lib.SPK_BOOL8, 1, out.data_ptr(),
                                                nxt.data_ptr(), stream))
        ref = eo.event_vecmat(spk, idx, w, n_post)
        if hetero:
            close(out, ref)
        else:
            assert np.array_equal(out.cpu().numpy(), ref)
        assert float(nxt.abs().max()) == 0.0                  # ready for the next call
    # packed words and a NULL next buffer; the product is ADDED to what the buffer holds
    spk = rs.random_sample(n_pre) < 0.03
    from brainstate_b200.event import pack_spikes
    words = pack_spikes(torch.from_numpy(spk).to(cuda))
    out = torch.full((n_post,), 1.0, device=cuda)
    _lib.check(bsx.bsx_event_vecmat_chained(C.byref(st), words.data_ptr(), _lib.SPK_BITS32, 1, out.data_ptr(), None, stream))
    close(out, eo.event_vecmat(spk, idx, w, n_post) + np.float32(1.0), scale=3)
    # refusals: the same buffer twice; an input beyond 128 KB
    assert bsx.bsx_event_vecmat_chained(C.byref(st), words.data_ptr(), _lib.SPK_BITS32, 1, out.data_ptr(), out.data_ptr(),
                                        stream) == _lib.BSX_ERR_INVALID_ARG
    big = torch.zeros((64, n_pre), dtype=torch.bool, device=cuda)
    big_out = torch.zeros((64, n_post), dtype=torch.float32, device=cuda)
    assert bsx.bsx_event_vecmat_chained(C.byref(st), big.data_ptr(), _lib.SPK_BOOL8, 64, big_out.data_ptr(), None,
                                        stream) == _lib.BSX_ERR_UNSUPPORTED
