"""CPU oracle for the event-driven synaptic propagation path (NumPy).

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, what the
reference computes on this path.  It is imported by the tests, by the smoke
check and by the CPU-baseline leg of the benchmark, and by nothing else; the
product never calls it.

What is pinned and what is not
------------------------------
* Connectivity generation is the reference's own NumPy call
  (``brainstate/nn/_event_fixedprob.py:165-171`` and ``:183-190``) and is
  bit-exact by construction; ``oracle/bsx_oracle.c`` restates the generator
  (MT19937 + masked rejection) and is checked against NumPy element for element.
* Operator semantics (forward, transpose, weight cotangent, JVP) follow the
  oracles the reference's tests recompute in-test
  (``brainstate/nn/_event_fixedprob_test.py:77-81,114-118,254-259``) and the
  event semantics of ``brainstate/nn/_event_linear.py:77-102``.  The reference
  ships no golden vector files; the arithmetic itself lives in the un-vendored
  dependency ``brainevent`` (``pyproject.toml:60``, ``>=0.0.7``, no exact pin),
  which is not installed here, so operator parity is pinned through those
  in-test oracles and the known-answer case of
  ``brainstate/nn/_event_linear_test.py:126-162``.
* Neuron/synapse dynamics (``EINetOracle``): PARITY UNPINNED.  The classes the
  reference's examples use (``brainpy.state.LIFRef/Expon/CUBA/COBA``) are not in
  the reference tree; the step below follows the call order of
  ``examples/400_CUBA_2005_bpu.py:60-66`` and the exponential-Euler scheme of
  ``brainstate/nn/_exp_euler.py:226-249``.

All accumulations are float32 and sequential in (row, k) order, which is what
``np.add.at`` does on a float32 array.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32


# ----------------------------------------------------------------------------
# connectivity  (brainstate/nn/_event_fixedprob.py:142-196)
# ----------------------------------------------------------------------------

def resolve_conn_num(out_size: int, conn_num) -> int:
    """``conn_num`` as the reference resolves it (``_event_fixedprob.py:142-147``)."""
    if isinstance(conn_num, float):
        assert 0. <= conn_num <= 1., 'Connection probability must be in [0, 1].'
        conn_num = int(out_size * conn_num)
    assert isinstance(conn_num, int), 'Connection number must be an integer.'
    return conn_num


def fixed_num_indices(seed: int, n_pre: int, n_post: int, conn_num: int,
                      chunk_rows: int | None = None) -> np.ndarray:
    """Index matrix ``(n_pre, conn_num)`` int32, bit-exact to
    ``_event_fixedprob.py:165-171`` (``allow_multi_conn=True``).

    ``chunk_rows`` draws the same stream in row chunks (identical output, lower
    peak memory: NumPy returns int64 before the cast).
    """
    rng = np.random.RandomState(seed)
    if chunk_rows is None or chunk_rows >= n_pre:
        return rng.randint(0, n_post, size=(n_pre, conn_num)).astype(np.int32)
    out = np.empty((n_pre, conn_num), np.int32)
    for r0 in range(0, n_pre, chunk_rows):
        r1 = min(n_pre, r0 + chunk_rows)
        out[r0:r1] = rng.randint(0, n_post, size=(r1 - r0, conn_num))
    return out


def afferent_csr(seed: int, n_pre: int, n_post: int, conn_num: int, afferent_ratio: float):
    """CSR branch of the constructor (``_event_fixedprob.py:183-190``).

    Returns ``(indices_flat int32, indptr int32 (n_pre+1,), pre_selected bool)``.
    The row mask is drawn from the same stream, after the indices.
    """
    rng = np.random.RandomState(seed)
    indices = rng.randint(0, n_post, size=(n_pre, conn_num)).astype(np.int32)
    pre_selected = rng.random(n_pre) < afferent_ratio
    flat = indices[pre_selected].flatten()
    indptr = (np.arange(1, n_pre + 1) * conn_num - np.cumsum(~pre_selected) * conn_num)
    indptr = np.insert(indptr, 0, 0).astype(np.int32)
    return flat, indptr, pre_selected


# ----------------------------------------------------------------------------
# helpers over the two layouts
# ----------------------------------------------------------------------------

def _flat(indices, weights):
    idx = np.ascontiguousarray(indices).reshape(-1)
    w = np.asarray(weights, dtype=F32)
    hetero = w.ndim > 0 and w.size == idx.size
    if not hetero:
        assert w.size == 1, 'weights must be a scalar or match the indices'
    return idx, (w.reshape(-1) if hetero else w.reshape(()).astype(F32)), bool(hetero)


def _row_starts(indices, indptr, n_pre):
    if indptr is None:
        K = indices.size // max(n_pre, 1)
        return np.arange(n_pre + 1, dtype=np.int64) * K
    return np.asarray(indptr, dtype=np.int64)


# ----------------------------------------------------------------------------
# forward products
# ----------------------------------------------------------------------------

def float_vecmat(x, indices, weights, n_post, indptr=None):
    """``y = x @ W`` for float ``x`` (``FixedNumConn.update``,
    ``_event_fixedprob.py:202-205``): ``y[idx[i,k]] += x[i] * w[i,k]``; duplicate
    targets accumulate (``_event_fixedprob_test.py:254-259``).  Leading batch
    dimensions of ``x`` are kept."""
    x = np.asarray(x)
    n_pre = x.shape[-1]
    idx, w, hetero = _flat(indices, weights)
    starts = _row_starts(indices, indptr, n_pre)
    xb = x.reshape(-1, n_pre).astype(F32)
    out = np.zeros((xb.shape[0], n_post), F32)
    lens = np.diff(starts)
    row_of = np.repeat(np.arange(n_pre), lens)
    for b in range(xb.shape[0]):
        nz = xb[b][row_of] != 0
        vals = (w[nz] if hetero else w) * xb[b][row_of[nz]]
        np.add.at(out[b], idx[nz], vals.astype(F32))
    return out.reshape(x.shape[:-1] + (n_post,))


def event_vecmat(spk, indices, weights, n_post, indptr=None):
    """``y = EventArray(spk) @ W`` (``EventFixedNumConn.update``,
    ``_event_fixedprob.py:249-252``): every nonzero entry of ``spk`` is a unit
    event (``_event_linear.py:82-85``); ``y[idx[i,k]] += w[i,k]`` for active ``i``."""
    spk = np.asarray(spk)
    return float_vecmat((spk != 0).astype(F32), indices, weights, n_post, indptr)


def event_vecmat_rows(spk, indices, weights, n_post, indptr=None, fixed_point=False):
    """:func:`event_vecmat` for ONE spike vector, visiting the active rows only (the same
    sequential float32 sum in (row, k) order, so the same bits; usable at 10^6 rows).
    With ``fixed_point`` the sum is taken over ``round(w * 2^32)`` in int64 and converted
    once (``float32(sum) * 2^-32``): the order-free accumulation the deterministic network
    step uses."""
    spk = np.asarray(spk).reshape(-1)
    n_pre = spk.size
    idx, w, hetero = _flat(indices, weights)
    active = np.nonzero(spk != 0)[0]
    if indptr is None:
        K = idx.size // max(n_pre, 1)
        pos = (active[:, None] * K + np.arange(K)[None, :]).reshape(-1)
    else:
        ip = np.asarray(indptr, dtype=np.int64)
        lens = ip[active + 1] - ip[active]
        pos = np.repeat(ip[active] - np.concatenate([[0], np.cumsum(lens)[:-1]]), lens) + np.arange(int(lens.sum()))
    cols = idx[pos]
    vals = w[pos] if hetero else np.full(cols.size, w, F32)
    if fixed_point:
        acc = np.zeros(n_post, np.int64)
        np.add.at(acc, cols, np.rint(vals.astype(np.float64) * 4294967296.0).astype(np.int64))
        return (acc.astype(F32) * F32(2.0 ** -32)).astype(F32)
    out = np.zeros(n_post, F32)
    np.add.at(out, cols, vals.astype(F32))
    return out


def float_matvec(v, indices, weights, n_pre, indptr=None):
    """``y = W @ v``: ``y[i] = sum_k w[i,k] * v[idx[i,k]]``, sequential in ``k``.
    This is also the input cotangent of the vecmat
    (``_event_fixedprob_test.py:56-88``)."""
    v = np.asarray(v)
    n_post = v.shape[-1]
    idx, w, hetero = _flat(indices, weights)
    starts = _row_starts(indices, indptr, n_pre)
    vb = v.reshape(-1, n_post).astype(F32)
    out = np.zeros((vb.shape[0], n_pre), F32)
    lens = np.diff(starts)
    row_of = np.repeat(np.arange(n_pre), lens)
    for b in range(vb.shape[0]):
        prod = (vb[b][idx] * w).astype(F32)
        np.add.at(out[b], row_of, prod)
    return out.reshape(v.shape[:-1] + (n_pre,))


def event_matvec(spk_post, indices, weights, n_pre, indptr=None):
    """``y = W @ EventArray(s)``: ``y[i] = sum_k w[i,k] * [s[idx[i,k]] != 0]``."""
    s = np.asarray(spk_post)
    return float_matvec((s != 0).astype(F32), indices, weights, n_pre, indptr)


# ----------------------------------------------------------------------------
# autodiff products  (_event_fixedprob_test.py:56-126)
# ----------------------------------------------------------------------------

def vecmat_vjp(x, ct, indices, weights, indptr=None, event=False):
    """Cotangents of ``y = x @ W`` for output cotangent ``ct``.

    ``dx[i] = sum_k w[i,k] ct[idx[i,k]]`` (dense, also for silent inputs: the
    gradient flows through the value, ``_event_linear.py:84-91``);
    heterogeneous ``dw[i,k] = a[i] ct[idx[i,k]]``, homogeneous
    ``dw = sum_i a[i] sum_k ct[idx[i,k]]``, with ``a = x`` for the float product
    and ``a = [x != 0]`` for the event product.  Batched inputs sum ``dw`` over
    the batch.
    """
    x = np.asarray(x)
    ct = np.asarray(ct, dtype=F32)
    n_pre, n_post = x.shape[-1], ct.shape[-1]
    idx, w, hetero = _flat(indices, weights)
    starts = _row_starts(indices, indptr, n_pre)
    lens = np.diff(starts)
    row_of = np.repeat(np.arange(n_pre), lens)
    dx = float_matvec(ct, indices, weights, n_pre, indptr)
    a = ((x != 0) if event else x).astype(F32).reshape(-1, n_pre)
    ctb = ct.reshape(-1, n_post)
    if hetero:
        dw = np.zeros(idx.shape, F32)
        for b in range(a.shape[0]):
            dw += (a[b][row_of] * ctb[b][idx]).astype(F32)
        dw = dw.reshape(np.shape(weights))
    else:
        acc = F32(0)
        for b in range(a.shape[0]):
            rowsum = np.zeros(n_pre, F32)
            np.add.at(rowsum, row_of, ctb[b][idx])
            acc = F32(acc + np.sum((a[b] * rowsum).astype(np.float64)))
        dw = F32(acc)
    return dx.astype(F32), dw


def vecmat_jvp(x, x_dot, w_dot, indices, weights, n_post, indptr=None, event=False):
    """Tangent of ``y = x @ W``: ``y_dot = x_dot @ W + a @ W_dot``
    (``_event_fixedprob_test.py:90-126``), ``a`` as in :func:`vecmat_vjp`."""
    a = (np.asarray(x) != 0).astype(F32) if event else np.asarray(x, dtype=F32)
    t1 = float_vecmat(np.asarray(x_dot, dtype=F32), indices, weights, n_post, indptr)
    t2 = float_vecmat(a, indices, w_dot, n_post, indptr)
    return (t1 + t2).astype(F32)


# ----------------------------------------------------------------------------
# dense event layer  (brainstate/nn/_event_linear.py:75-102)
# ----------------------------------------------------------------------------

def event_linear(spk, weight, out_size, float_as_event=True):
    """``EventLinear.update``: scalar weight reduces by the event count
    (``float_as_event``) or the value sum and broadcasts over ``out_size``;
    a matrix weight is ``[spk != 0] @ W`` or ``spk @ W``."""
    spk = np.asarray(spk)
    w = np.asarray(weight, dtype=F32)
    if w.size == 1:
        red = np.sum(spk != 0, axis=-1) if float_as_event else np.sum(spk.astype(F32), axis=-1)
        return (np.ones(spk.shape[:-1] + (out_size,), F32)
                * (np.asarray(red, F32)[..., None] * w.reshape(()))).astype(F32)
    a = (spk != 0).astype(F32) if float_as_event else spk.astype(F32)
    out = np.zeros(a.shape[:-1] + (w.shape[1],), F32)
    ab = a.reshape(-1, a.shape[-1])
    ob = out.reshape(-1, w.shape[1])
    for b in range(ab.shape[0]):
        for i in np.nonzero(ab[b])[0]:          # sequential in i, float32 accumulate
            ob[b] += (ab[b, i] * w[i]).astype(F32)
    return out


# ----------------------------------------------------------------------------
# position-keyed heterogeneous weights (builder-specified: the reference takes any
# initializer callable for conn_weight, brainstate/nn/_event_fixedprob.py:173-175)
# ----------------------------------------------------------------------------

def _mix32(x):
    x = np.asarray(x, np.uint32).copy()
    with np.errstate(over='ignore'):
        x ^= x >> np.uint32(16); x *= np.uint32(0x7feb352d)
        x ^= x >> np.uint32(15); x *= np.uint32(0x846ca68b)
        x ^= x >> np.uint32(16)
    return x


def lognormal_weights(seed, rows, ks, mu, sigma, sign=1.0):
    """``sign * exp(mu + sigma * z)`` with ``z`` a standard normal from a 32-bit hash
    of ``(seed, row, k)`` (Box-Muller in float64, one rounding to float32)."""
    rows = np.asarray(rows, np.uint32)
    ks = np.asarray(ks, np.uint32)
    with np.errstate(over='ignore'):
        h = _mix32(_mix32(rows + np.uint32(seed) * np.uint32(0x9e3779b9))
                   ^ (ks * np.uint32(0x85ebca6b) + np.uint32(0x27d4eb2f)))
        g = _mix32(h ^ np.uint32(0x165667b1))
    u1 = (h.astype(np.float64) + 1.0) * (1.0 / 4294967296.0)
    u2 = g.astype(np.float64) * (1.0 / 4294967296.0)
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(6.283185307179586476925286766559 * u2)
    return (np.float32(sign) * np.exp(mu + sigma * z).astype(F32)).astype(F32)


# ----------------------------------------------------------------------------
# spike packing
# ----------------------------------------------------------------------------

def pack_bits(spk) -> np.ndarray:
    """Packed spike words: bit ``i % 32`` of word ``i // 32`` is ``spk[i] != 0``."""
    s = (np.asarray(spk).reshape(-1) != 0)
    n = s.size
    pad = (-n) % 32
    s = np.concatenate([s, np.zeros(pad, bool)])
    return np.packbits(s.reshape(-1, 32), axis=1, bitorder='little').view('<u4').reshape(-1)


def unpack_bits(words, n) -> np.ndarray:
    b = np.unpackbits(np.asarray(words, dtype='<u4').view(np.uint8), bitorder='little')
    return b[:n].astype(bool)


# ----------------------------------------------------------------------------
# E/I network step (parity unpinned; see the module docstring)
# ----------------------------------------------------------------------------

def exprel_f32(z):
    """``(exp(z)-1)/z``, the factor ``exp_euler_step`` uses
    (``brainstate/nn/_exp_euler.py:246``).  For ``|z| <= 0.125`` the degree-5 Taylor
    polynomial ``1 + z/2 + ... + z^5/720`` in Horner form with every multiply and add
    rounded to float32 (the first dropped term, ``z^6/5040``, is below 8e-10 there, the
    result within one float32 ulp of the float64 value; a GPU doing the same operations
    matches bit for bit); otherwise float64 and one rounding."""
    z = np.asarray(z, dtype=F32)
    p = np.full(z.shape, F32(0.0013888889), F32)
    for c in (F32(0.008333334), F32(0.041666668), F32(0.16666667), F32(0.5), F32(1.0)):
        p = ((p * z).astype(F32) + c).astype(F32)
    z64 = z.astype(np.float64)
    safe = np.where(z64 == 0, 1.0, z64)
    big = (np.expm1(safe) / safe).astype(F32)
    return np.where(np.abs(z) <= F32(0.125), p, big).astype(F32)


class EINetOracle:
    """Excitatory/inhibitory LIF network with exponential synapses.

    One step, in the order of ``examples/400_CUBA_2005_bpu.py:60-66``:

    1. ``s`` = spikes of the previous step; excitatory rows are ``[0, n_exc)``.
    2. ``dg_e = s[:n_exc] @ W_E``, ``dg_i = s[n_exc:] @ W_I`` (event vecmat).
    3. ``g <- g * exp(-dt/tau_syn) + dg`` — exponential Euler of ``dg/dt = -g/tau``
       is exact (``_exp_euler.py:246-249``).
    4. current: CUBA ``I = g_e + g_i``; COBA ``I = g_e (E_e - V) + g_i (E_i - V)``.
    5. ``f(V) = (V_rest - V + R (I + I_ext)) / tau_m``;
       ``V <- V + dt * exprel(dt * J) * f`` with ``J = df/dV``
       (CUBA: ``-1/tau_m``; COBA: ``-(1 + R (g_e + g_i))/tau_m``).  Neurons in
       their refractory period keep ``V`` unchanged.
    6. ``spike = (V >= V_th)`` and not refractory; spiking neurons are set to
       ``V_reset`` and start ``ref_steps`` refractory steps.

    Every operation is a single float32 IEEE operation (no fused multiply-add),
    transcendental factors are evaluated in float64 and rounded once, so a GPU
    implementation can reproduce the spike raster bit for bit.
    """

    def __init__(self, n_exc, n_inh, idx_e, w_e, idx_i, w_i, *, coba=False,
                 dt=0.1, tau_m=20., tau_e=5., tau_i=10., V_rest=-49., V_th=-50.,
                 V_reset=-60., tau_ref=5., R=1., I_ext=0., E_e=0., E_i=-80.,
                 V0=None, indptr_e=None, indptr_i=None, n_local=None, first=0, delay_e=0, delay_i=0,
                 ext_threshold=0, ext_seed=0, ext_weight=0., fixed_point=False):
        # n_local: number of neurons whose state this instance holds (a postsynaptic
        # shard); the index arrays then hold local column ids.  Default: the whole network.
        self.n_exc, self.n_inh = n_exc, n_inh
        self.n_global = n_exc + n_inh
        self.n = self.n_global if n_local is None else n_local
        self.idx_e, self.w_e, self.idx_i, self.w_i = idx_e, w_e, idx_i, w_i
        self.indptr_e, self.indptr_i = indptr_e, indptr_i
        self.coba = coba
        self.dt = F32(dt)
        self.decay_e = F32(np.exp(-np.float64(dt) / np.float64(tau_e)))
        self.decay_i = F32(np.exp(-np.float64(dt) / np.float64(tau_i)))
        self.inv_tau_m = F32(1.0 / np.float64(tau_m))
        self.cuba_gain = F32(-np.expm1(-np.float64(dt) / np.float64(tau_m)))  # dt*exprel(-dt/tau)/tau
        self.V_rest, self.V_th, self.V_reset = F32(V_rest), F32(V_th), F32(V_reset)
        self.R, self.I_ext = F32(R), F32(I_ext)
        self.E_e, self.E_i = F32(E_e), F32(E_i)
        self.ref_steps = int(round(float(tau_ref) / float(dt)))
        self.V = (np.full(self.n, V_reset, F32) if V0 is None else np.asarray(V0, F32).copy())
        self.g_e = np.zeros(self.n, F32)
        self.g_i = np.zeros(self.n, F32)
        self.ref = np.zeros(self.n, np.int32)       # remaining refractory steps
        self.spk = np.zeros(self.n, bool)
        # synaptic delays: a spike of step t acts at step t + 1 + delay; background drive:
        # one external excitatory event per neuron and step where the hash of
        # (seed, global id, step) is below the threshold
        self.first = first
        self.delay_e, self.delay_i = int(delay_e), int(delay_i)
        self.history = []                      # global spike vectors of past steps, oldest first
        self.t = 0
        self.ext_threshold, self.ext_seed, self.ext_weight = int(ext_threshold), int(ext_seed), F32(ext_weight)
        # fixed_point: synaptic input summed as int64 multiples of 2^-32 (order-free)
        self.fixed_point = bool(fixed_point)

    @staticmethod
    def mix32(x):
        x = x.astype(np.uint32)
        x ^= x >> np.uint32(16); x *= np.uint32(0x7feb352d)
        x ^= x >> np.uint32(15); x *= np.uint32(0x846ca68b)
        x ^= x >> np.uint32(16)
        return x

    @classmethod
    def drive_hash(cls, seed, gid, step):
        """Restates the integer hash of the device's background drive."""
        with np.errstate(over='ignore'):
            gid = np.asarray(gid, np.uint32)
            a = cls.mix32(gid + np.uint32(seed) * np.uint32(0x9e3779b9))
            b = np.uint32(step) * np.uint32(0x85ebca6b) + np.uint32(0xc2b2ae35)
            return cls.mix32(a ^ b)

    def _delayed(self, delay):
        k = len(self.history) - 1 - delay
        return self.history[k] if k >= 0 else np.zeros(self.n_global, bool)

    def step(self, s_global=None):
        """One step.  ``s_global``: spikes of the previous step of the WHOLE network
        (needed by a shard); by default the instance's own previous spikes."""
        s = self.spk if s_global is None else np.asarray(s_global, bool)
        assert s.shape == (self.n_global,)
        if self.t > 0:
            self.history.append(s.copy())
        s_e, s_i = self._delayed(self.delay_e), self._delayed(self.delay_i)
        self.history = self.history[-(max(self.delay_e, self.delay_i) + 1):]
        dg_e = event_vecmat_rows(s_e[:self.n_exc], self.idx_e, self.w_e, self.n, self.indptr_e, self.fixed_point)
        dg_i = event_vecmat_rows(s_i[self.n_exc:], self.idx_i, self.w_i, self.n, self.indptr_i, self.fixed_point)
        return self.advance(dg_e, dg_i)

    def projections(self, s_global):
        """Synaptic input one spike vector of the whole network sends to this instance's neurons:
        ``(dg_e, dg_i)``, no delay applied (the caller decides at which step it acts)."""
        s = np.asarray(s_global, bool)
        return (event_vecmat_rows(s[:self.n_exc], self.idx_e, self.w_e, self.n, self.indptr_e, self.fixed_point),
                event_vecmat_rows(s[self.n_exc:], self.idx_i, self.w_i, self.n, self.indptr_i, self.fixed_point))

    def advance(self, dg_e, dg_i):
        """The neuron update of one step for given synaptic increments (steps 3-6 of the class
        docstring, plus the background drive).  Returns ``(spikes, dg_e, dg_i)``."""
        dg_e, dg_i = np.asarray(dg_e, F32), np.asarray(dg_i, F32)
        if self.ext_threshold:
            gid = np.arange(self.first, self.first + self.n, dtype=np.uint32)
            fire = self.drive_hash(self.ext_seed, gid, self.t) < np.uint32(min(self.ext_threshold, 0xffffffff))
            dg_e = np.where(fire, (dg_e + self.ext_weight).astype(F32), dg_e).astype(F32)
        self.t += 1
        self.g_e = (self.g_e * self.decay_e).astype(F32) + dg_e
        self.g_i = (self.g_i * self.decay_i).astype(F32) + dg_i
        V = self.V
        if self.coba:
            cur = (self.g_e * (self.E_e - V)).astype(F32) + (self.g_i * (self.E_i - V)).astype(F32)
        else:
            cur = self.g_e + self.g_i
        drive = (self.R * (cur + self.I_ext).astype(F32)).astype(F32)
        f = (((self.V_rest - V).astype(F32) + drive).astype(F32) * self.inv_tau_m).astype(F32)
        if self.coba:
            gsum = (self.g_e + self.g_i).astype(F32)
            J = (-(F32(1) + (self.R * gsum).astype(F32)).astype(F32) * self.inv_tau_m).astype(F32)
            gain = (self.dt * exprel_f32((self.dt * J).astype(F32))).astype(F32)
            V_new = (V + (gain * f).astype(F32)).astype(F32)
        else:
            # dt*exprel(-dt/tau)*f == (1-exp(-dt/tau)) * (V_rest - V + R I)
            num = ((self.V_rest - V).astype(F32) + drive).astype(F32)
            V_new = (V + (self.cuba_gain * num).astype(F32)).astype(F32)
        refractory = self.ref > 0
        V_new = np.where(refractory, V, V_new).astype(F32)
        spk = (V_new >= self.V_th) & ~refractory
        self.V = np.where(spk, self.V_reset, V_new).astype(F32)
        self.ref = np.where(spk, self.ref_steps, np.maximum(self.ref - 1, 0)).astype(np.int32)
        self.spk = spk
        return spk, dg_e, dg_i

    def run(self, steps):
        raster = np.zeros((steps, self.n), bool)
        for t in range(steps):
            raster[t] = self.step()[0]
        return raster
