"""CPU: pins the oracle (NumPy + C) against the golden fixtures, NumPy's own
generator and the reference's known-answer cases."""
import os

import numpy as np
import pytest

from oracle import event_oracle as eo

GOLD = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'event_golden.npz'))
CASES = [0, 1, 2, 3]


def meta(c):
    seed, n_pre, n_post, K = (int(v) for v in GOLD[f'c{c}_meta'])
    return seed, n_pre, n_post, K


@pytest.mark.parametrize('c', CASES)
def test_connectivity_bit_exact(c, c_oracle):
    seed, n_pre, n_post, K = meta(c)
    gold = GOLD[f'c{c}_indices']
    assert np.array_equal(eo.fixed_num_indices(seed, n_pre, n_post, K), gold)
    assert np.array_equal(eo.fixed_num_indices(seed, n_pre, n_post, K, chunk_rows=3), gold)
    assert np.array_equal(c_oracle.fixed_num_indices(seed, n_pre, n_post, K), gold)
    flat, indptr, sel = eo.afferent_csr(seed, n_pre, n_post, K, 0.5)
    assert np.array_equal(sel, GOLD[f'c{c}_pre_selected'])
    assert np.array_equal(flat, gold[sel].reshape(-1))
    assert indptr[0] == 0 and indptr[-1] == flat.size
    assert np.array_equal(np.diff(indptr), np.where(sel, K, 0))


@pytest.mark.parametrize('n_post', [1, 2, 3, 40, 1000, 65536, 65537, 4000, 1 << 20])
def test_c_generator_matches_numpy(n_post, c_oracle):
    for seed in (0, 1, 123, 2 ** 31 + 5):
        a = c_oracle.fixed_num_indices(seed, 37, n_post, 11)
        b = np.random.RandomState(seed).randint(0, n_post, size=(37, 11)).astype(np.int32)
        assert np.array_equal(a, b)


def test_c_stream_continues_into_random_sample(c_oracle):
    mt = c_oracle.MT(7)
    rs = np.random.RandomState(7)
    assert np.array_equal(mt.randint(40, 80), rs.randint(0, 40, 80).astype(np.int32))
    assert np.array_equal(mt.random_sample(20), rs.random_sample(20))


@pytest.mark.parametrize('c', CASES)
def test_products_match_golden(c, c_oracle):
    seed, n_pre, n_post, K = meta(c)
    idx, spk, xf, w = GOLD[f'c{c}_indices'], GOLD[f'c{c}_spk'], GOLD[f'c{c}_xf'], GOLD[f'c{c}_w_het']
    ct = GOLD[f'c{c}_ct']
    for impl_np in (True, False):
        ev = eo.event_vecmat if impl_np else (lambda s, i, ww, n: c_oracle.event_vecmat_u8(s, i, ww, n))
        fv = eo.float_vecmat if impl_np else (lambda s, i, ww, n: c_oracle.float_vecmat(s, i, ww, n))
        assert np.array_equal(ev(spk, idx, np.float32(1.5), n_post), GOLD[f'c{c}_y_event_homo'])
        assert np.array_equal(ev(spk, idx, w, n_post), GOLD[f'c{c}_y_event_het'])
        assert np.array_equal(fv(xf, idx, w, n_post), GOLD[f'c{c}_y_float_het'])
    # a float spike vector is an event wherever it is nonzero
    assert np.array_equal(eo.event_vecmat(xf, idx, w, n_post), GOLD[f'c{c}_y_event_het'])
    dx, dw = eo.vecmat_vjp(xf, ct, idx, w, event=False)
    # float32 sequential sum of K mixed-sign terms against the float64 golden sum
    np.testing.assert_allclose(dx, GOLD[f'c{c}_dx_het'], rtol=1e-5, atol=2e-5)
    assert np.array_equal(dw, GOLD[f'c{c}_dw_het_float'])
    _, dwe = eo.vecmat_vjp(xf, ct, idx, w, event=True)
    assert np.array_equal(dwe, GOLD[f'c{c}_dw_het_event'])
    _, dwh = eo.vecmat_vjp(spk, ct, idx, np.float32(1.5), event=True)
    np.testing.assert_allclose(dwh, GOLD[f'c{c}_dw_homo_event'], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(c_oracle.float_matvec(ct, idx, w, n_pre), GOLD[f'c{c}_dx_het'], rtol=1e-5, atol=2e-5)
    assert np.array_equal(c_oracle.vecmat_dw(xf, ct, idx, n_pre, n_post), GOLD[f'c{c}_dw_het_float'])


def test_vjp_matches_finite_differences_of_the_forward():
    rs = np.random.RandomState(3)
    n_pre, n_post, K = 12, 9, 4
    idx = rs.randint(0, n_post, (n_pre, K)).astype(np.int32)
    w = rs.uniform(-1, 1, (n_pre, K))
    x = rs.uniform(-1, 1, n_pre)
    ct = rs.standard_normal(n_post)

    def f(xx, ww):  # float64 dense evaluation
        y = np.zeros(n_post)
        for i in range(n_pre):
            np.add.at(y, idx[i], ww[i] * xx[i])
        return float(y @ ct)

    dx, dw = eo.vecmat_vjp(x.astype(np.float32), ct.astype(np.float32), idx, w.astype(np.float32))
    eps = 1e-6
    for i in range(n_pre):
        e = np.zeros(n_pre); e[i] = eps
        assert abs((f(x + e, w) - f(x - e, w)) / (2 * eps) - dx[i]) < 1e-4
    for (i, k) in [(0, 0), (3, 2), (11, 3)]:
        e = np.zeros((n_pre, K)); e[i, k] = eps
        assert abs((f(x, w + e) - f(x, w - e)) / (2 * eps) - dw[i, k]) < 1e-4
    # forward mode: y_dot = x_dot @ W + x @ W_dot equals the directional derivative
    xd, wd = rs.standard_normal(n_pre), rs.standard_normal((n_pre, K))
    yd = eo.vecmat_jvp(x, xd, wd, idx, w, n_post)
    num = (f(x + eps * xd, w + eps * wd) - f(x - eps * xd, w - eps * wd)) / (2 * eps)
    assert abs(float(yd @ ct.astype(np.float32)) - num) < 1e-3


def test_csr_layout_equals_masked_dense_layout():
    seed, n_pre, n_post, K = 7, 33, 50, 5
    flat, indptr, sel = eo.afferent_csr(seed, n_pre, n_post, K, 0.4)
    idx = eo.fixed_num_indices(seed, n_pre, n_post, K)
    spk = np.random.RandomState(1).random_sample(n_pre) < 0.5
    y_csr = eo.event_vecmat(spk, flat, np.float32(0.7), n_post, indptr)
    y_ref = eo.event_vecmat(spk & sel, idx, np.float32(0.7), n_post)
    assert np.array_equal(y_csr, y_ref)
    v = np.random.RandomState(2).standard_normal(n_post).astype(np.float32)
    w = np.random.RandomState(3).standard_normal(flat.size).astype(np.float32)
    m = eo.float_matvec(v, flat, w, n_pre, indptr)
    assert np.all(m[~sel] == 0)


def test_matvec_is_transpose_of_vecmat():
    rs = np.random.RandomState(5)
    n_pre, n_post, K = 40, 25, 6
    idx = rs.randint(0, n_post, (n_pre, K)).astype(np.int32)
    w = rs.standard_normal((n_pre, K)).astype(np.float32)
    dense = np.zeros((n_pre, n_post))
    for i in range(n_pre):
        np.add.at(dense[i], idx[i], w[i])
    x = rs.standard_normal(n_pre).astype(np.float32)
    v = rs.standard_normal(n_post).astype(np.float32)
    np.testing.assert_allclose(eo.float_vecmat(x, idx, w, n_post), x @ dense, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(eo.float_matvec(v, idx, w, n_pre), dense @ v, rtol=1e-4, atol=1e-5)
    s = rs.random_sample(n_post) < 0.3
    np.testing.assert_allclose(eo.event_matvec(s, idx, w, n_pre), dense @ s, rtol=1e-4, atol=1e-5)


def test_dense_event_known_answer():
    spk, w = GOLD['dense_spk'], GOLD['dense_w']
    y_true = eo.event_linear(spk, w, 6, float_as_event=True)
    y_false = eo.event_linear(spk, w, 6, float_as_event=False)
    assert np.all(y_true == GOLD['dense_event_true'])
    assert np.all(y_false == GOLD['dense_event_false'])
    W = np.random.RandomState(0).standard_normal((10, 6)).astype(np.float32)
    np.testing.assert_allclose(eo.event_linear(spk, W, 6, True), (spk != 0).astype(np.float32) @ W, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(eo.event_linear(spk, W, 6, False), spk @ W, rtol=1e-5, atol=1e-6)


def test_pack_bits_roundtrip():
    rs = np.random.RandomState(0)
    for n in (1, 31, 32, 33, 100, 4000):
        s = rs.random_sample(n) < 0.3
        words = eo.pack_bits(s)
        assert words.size == (n + 31) // 32
        assert np.array_equal(eo.unpack_bits(words, n), s)
        for i in np.nonzero(s)[0][:5]:
            assert (int(words[i // 32]) >> (i % 32)) & 1


def test_network_oracle_is_self_active_and_deterministic():
    n_exc, n_inh = 320, 80
    n = n_exc + n_inh
    idx_e = eo.fixed_num_indices(100, n_exc, n, 8)
    idx_i = eo.fixed_num_indices(101, n_inh, n, 8)
    V0 = np.random.RandomState(102).uniform(-60, -50, n).astype(np.float32)
    runs = []
    for _ in range(2):
        net = eo.EINetOracle(n_exc, n_inh, idx_e, np.float32(1.62), idx_i, np.float32(-9.0), V0=V0)
        runs.append(net.run(300))
    assert np.array_equal(runs[0], runs[1])
    assert runs[0].sum() > 0                       # V_rest above threshold: the network fires unaided
    # refractory: no neuron fires twice within tau_ref / dt = 50 steps
    t, i = np.nonzero(runs[0])
    for nid in np.unique(i)[:20]:
        ts = t[i == nid]
        assert np.all(np.diff(ts) > 50)


def test_exprel_f32_is_within_one_ulp_of_float64():
    """The exponential factor of the conductance-based step: the float32 Horner polynomial
    used for |z| <= 0.125 (on the device and in the oracle, operation for operation) and the
    float64 branch beyond stay within one float32 ulp of expm1(z)/z."""
    pieces = [np.linspace(-0.125, 0.125, 400001), np.linspace(-0.5, -0.125, 50001), np.linspace(0.125, 0.5, 50001),
              np.linspace(-30, 30, 20001), np.array([1e-8, -1e-8, 1e-4, -1e-4, 0.125, -0.125, 0.12500001, -0.12500001])]
    z = np.concatenate(pieces).astype(np.float32)
    z = z[z != 0]
    got = eo.exprel_f32(z).astype(np.float64)
    z64 = z.astype(np.float64)
    ref = np.expm1(z64) / z64
    ulp = np.spacing(ref.astype(np.float32)).astype(np.float64)
    err = np.abs(got - ref) / ulp
    assert err.max() <= 1.0, (err.max(), z[err.argmax()])
    inside = np.abs(z) <= np.float32(0.125)
    assert err[inside].max() <= 0.75            # measured 0.57
    assert err[~inside].max() <= 0.5 + 1e-9     # one rounding of the float64 value
    assert eo.exprel_f32(np.float32(0.0)) == np.float32(1.0)


@pytest.mark.parametrize('hetero', [False, True])
def test_event_vecmat_over_active_rows_equals_the_full_walk(hetero):
    """``event_vecmat_rows`` (active rows only; what the network oracle uses at 10^6 neurons)
    gives the bits of ``event_vecmat``, for both layouts; its fixed-point form agrees within
    half a float32 ulp of the sum and does not depend on the order of the entries."""
    rs = np.random.RandomState(5)
    n_pre, n_post, K = 400, 150, 21
    idx = rs.randint(0, n_post, (n_pre, K)).astype(np.int32)
    w = rs.normal(0.1, 0.3, (n_pre, K)).astype(np.float32) if hetero else np.float32(-0.7)
    spk = rs.random_sample(n_pre) < 0.15
    assert np.array_equal(eo.event_vecmat_rows(spk, idx, w, n_post), eo.event_vecmat(spk, idx, w, n_post))
    flat, indptr, _ = eo.afferent_csr(9, n_pre, n_post, K, 0.5)
    wf = rs.normal(0.1, 0.3, flat.shape).astype(np.float32) if hetero else w
    assert np.array_equal(eo.event_vecmat_rows(spk, flat, wf, n_post, indptr), eo.event_vecmat(spk, flat, wf, n_post, indptr))
    fx = eo.event_vecmat_rows(spk, idx, w, n_post, fixed_point=True)
    act = np.nonzero(spk)[0]
    ref = np.zeros(n_post, np.float64)
    np.add.at(ref, idx[act].reshape(-1), (w[act].reshape(-1) if hetero else np.full(act.size * K, w)).astype(np.float64))
    np.testing.assert_allclose(fx, ref, rtol=1e-6, atol=1e-7)
    perm = rs.permutation(K)                     # another order inside every row: same integers, same sum
    w2 = w[:, perm] if hetero else w
    assert np.array_equal(eo.event_vecmat_rows(spk, idx[:, perm], w2, n_post, fixed_point=True), fx)
