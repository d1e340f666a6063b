"""Excitatory/inhibitory spiking network driver over the fused step kernels.

``EINet`` stands for the model the reference's examples assemble from
``brainstate.nn.EventFixedProb`` and ``brainpy.state`` parts
(``examples/400_CUBA_2005_bpu.py:36-66``: ``LIFRef`` neurons, two
``AlignPostProj(comm=EventFixedProb, syn=Expon, out=CUBA|COBA)`` projections) and
for the loop ``brainstate.transform.for_loop(net.update, times)``
(``brainstate/transform/_loop_collect_return.py:488-572``): ``run(steps)`` advances
the network and returns the bit-packed spike raster.

On one GPU all steps of a ``run`` are one cooperative kernel launch.  With a
process group the postsynaptic neurons are split into contiguous blocks, one per
rank; every rank keeps the synapses that target its block (a CSR block drawn from
the same seeded stream as the full matrix).  The ranks exchange their spikes either
inside the step kernel (``exchange='p2p'``: compact id lists pushed over NVLink, one
launch per GPU for all steps) or with one NCCL all-gather of the packed spike words per
step (``exchange='nccl'``, split-phase launches).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import BsxLifParams, BsxNet, BsxNetLinks, BsxNetShard, check, lib
from .event import CSR, FixedPostNumConn
from .nn._event_fixedprob import EventFixedProb, _device

__all__ = ['LIFParams', 'Lognormal', 'EINet', 'shard_bounds', 'words_per_rank', 'sharded_block',
           'build_projection', 'unpack_raster', 'preset', 'from_preset', 'population_rates', 'COBA_BIAS']


@dataclass
class LIFParams:
    """Neuron and synapse constants (times in ms, potentials in mV)."""
    dt: float = 0.1
    tau_m: float = 20.
    tau_e: float = 5.
    tau_i: float = 10.
    V_rest: float = -49.
    V_th: float = -50.
    V_reset: float = -60.
    tau_ref: float = 5.
    R: float = 1.
    I_ext: float = 0.
    E_e: float = 0.
    E_i: float = -80.
    coba: bool = False
    ext_rate_hz: float = 0.      # background drive: external events per second per neuron
    ext_weight: float = 0.       # size of one external event (added to the excitatory synapse)
    ext_seed: int = 0

    @property
    def ext_threshold(self) -> int:
        """32-bit threshold of the per-step event probability ``rate * dt`` (dt in ms)."""
        p = max(0.0, min(1.0, self.ext_rate_hz * self.dt * 1e-3))
        return min(0xffffffff, int(round(p * 4294967296.0)))

    def struct(self) -> BsxLifParams:
        p = BsxLifParams()
        f32 = np.float32
        p.dt = f32(self.dt)
        p.decay_e = f32(math.exp(-self.dt / self.tau_e))
        p.decay_i = f32(math.exp(-self.dt / self.tau_i))
        p.inv_tau_m = f32(1.0 / self.tau_m)
        p.cuba_gain = f32(-math.expm1(-self.dt / self.tau_m))
        p.V_rest, p.V_th, p.V_reset = f32(self.V_rest), f32(self.V_th), f32(self.V_reset)
        p.R, p.I_ext = f32(self.R), f32(self.I_ext)
        p.E_e, p.E_i = f32(self.E_e), f32(self.E_i)
        p.ref_steps = int(round(self.tau_ref / self.dt))
        p.coba = int(self.coba)
        p.ext_threshold = self.ext_threshold
        p.ext_seed = int(self.ext_seed) & 0xffffffff
        p.ext_weight = f32(self.ext_weight)
        return p


def words_per_rank(n: int, world: int) -> int:
    """Spike words every rank contributes to the all-gather (the last ranks' share
    may be partly or wholly padding)."""
    words = (n + 31) // 32
    return (words + world - 1) // world


def shard_bounds(n: int, world: int, rank: int):
    """Contiguous block ``[first, last)`` of ``n`` neurons owned by ``rank``: whole
    32-bit spike words, ``words_per_rank`` of them per rank, clipped to ``n``."""
    wpr = words_per_rank(n, world)
    return min(n, 32 * rank * wpr), min(n, 32 * (rank + 1) * wpr)


def sharded_block(seed: int, n_pre: int, n_post: int, conn_num: int, col0: int, col1: int):
    """CSR block (host arrays) of the fixed-number matrix ``RandomState(seed).randint(0,
    n_post, (n_pre, conn_num))`` restricted to targets in ``[col0, col1)``; column
    ids are local (minus ``col0``).  Returns ``(indices int32, indptr int64)``."""
    if col1 <= col0:        # an empty shard (more ranks than spike words); an empty column range would mean "no filter"
        return np.empty(0, np.int32), np.zeros(n_pre + 1, np.int64)
    buf = np.empty(n_pre * conn_num, np.int32)
    counts = np.empty(n_pre, np.int32)
    n = lib().bsx_host_fixed_num_indices(C.c_uint32(int(seed) & 0xffffffff), n_pre, n_post, conn_num, 0, n_pre,
                                        col0, col1, buf.ctypes.data, counts.ctypes.data)
    check(int(n))
    indptr = np.zeros(n_pre + 1, np.int64)
    np.cumsum(counts, out=indptr[1:])
    return buf[:n].copy(), indptr


class PeerLost(RuntimeError):
    """A rank of the network did not answer the host-side roll call before a launch."""


def wait_for_peers(health_group, timeout_s: float = 5.0) -> None:
    """Roll call of the ranks on the host, before a launch whose kernels wait for one another:
    every rank must answer within ``timeout_s`` (``torch.distributed.monitored_barrier`` on a
    ``gloo`` group over the same ranks).  A rank that has exited, hangs or is later than that
    raises :class:`PeerLost` on the others — on the host, with no kernel in flight — instead
    of a device-side wait running out.  The reference has no counterpart (a single-process
    library)."""
    import datetime
    import torch.distributed as dist
    try:
        dist.monitored_barrier(group=health_group, timeout=datetime.timedelta(seconds=float(timeout_s)),
                               wait_all_ranks=True)
    except RuntimeError as exc:
        raise PeerLost(f'a rank did not answer within {timeout_s} s: {exc}') from exc


@dataclass
class Lognormal:
    """Heterogeneous weights ``scale * exp(mu + sigma * z)``, ``z`` standard normal keyed by
    the synapse's position ``(row, k)`` and ``seed`` (so every shard can fill its own)."""
    mu: float = -2.0
    sigma: float = 0.5
    seed: int = 0
    scale: float = 1.0


def build_projection(seed: int, n_pre: int, n_post: int, conn_num: int, weight, device, col0: int = 0,
                     col1: Optional[int] = None, chunk_rows: Optional[int] = None):
    """One projection's connectivity on the device, drawn from the reference's seeded
    stream (``RandomState(seed).randint(0, n_post, (n_pre, conn_num))``,
    ``brainstate/nn/_event_fixedprob.py:165-171``) in row chunks, so that neither the
    host nor the device ever holds more than a chunk beyond the final arrays.

    With ``[col0, col1)`` narrower than ``[0, n_post)`` the result is the CSR block of
    one postsynaptic shard (local column ids); otherwise the full fixed-number matrix.
    ``weight``: a float (homogeneous) or :class:`Lognormal`.
    """
    l = lib()
    col1 = n_post if col1 is None else col1
    if col1 <= col0:        # an empty shard (more ranks than spike words): no synapse targets it
        if isinstance(weight, Lognormal):
            return CSR((torch.empty(0, dtype=torch.float32, device=device), torch.empty(0, dtype=torch.int32, device=device),
                        torch.zeros(n_pre + 1, dtype=torch.int64, device=device)), shape=(n_pre, 0))
        return CSR((float(weight), torch.empty(0, dtype=torch.int32, device=device),
                    torch.zeros(n_pre + 1, dtype=torch.int64, device=device)), shape=(n_pre, 0))
    filtered = not (col0 == 0 and col1 == n_post)
    if chunk_rows is None:
        chunk_rows = max(1, (1 << 26) // max(conn_num, 1))          # 64 Mi entries per chunk
    gen = l.bsx_host_gen_new(C.c_uint32(int(seed) & 0xffffffff))
    if not gen:
        raise MemoryError('bsx_host_gen_new failed')
    hetero = isinstance(weight, Lognormal)
    try:
        if not filtered:
            idx = torch.empty((n_pre, conn_num), dtype=torch.int32, device=device)
            buf = torch.empty((min(chunk_rows, n_pre), conn_num), dtype=torch.int32).pin_memory()
            for r0 in range(0, n_pre, chunk_rows):
                rows = min(chunk_rows, n_pre - r0)
                n = l.bsx_host_gen_rows(gen, rows, n_post, conn_num, 0, 0, buf.data_ptr(), None, None)
                check(int(n))
                idx[r0:r0 + rows].copy_(buf[:rows])
            kpos, indptr = None, None
        else:
            pieces, kpieces, counts = [], [], np.empty(n_pre, np.int32)
            buf = np.empty(min(chunk_rows, n_pre) * conn_num, np.int32)
            kbuf = np.empty(buf.size, np.int16) if hetero else None
            for r0 in range(0, n_pre, chunk_rows):
                rows = min(chunk_rows, n_pre - r0)
                n = l.bsx_host_gen_rows(gen, rows, n_post, conn_num, col0, col1, buf.ctypes.data,
                                        None if kbuf is None else kbuf.ctypes.data, counts[r0:].ctypes.data)
                check(int(n))
                pieces.append(torch.from_numpy(buf[:n].copy()).to(device))
                if hetero:
                    kpieces.append(torch.from_numpy(kbuf[:n].copy()).to(device))
            idx = torch.cat(pieces) if pieces else torch.empty(0, dtype=torch.int32, device=device)
            kpos = torch.cat(kpieces) if hetero and kpieces else None
            ip = np.zeros(n_pre + 1, np.int64)
            np.cumsum(counts, out=ip[1:])
            indptr = torch.from_numpy(ip).to(device)
    finally:
        l.bsx_host_gen_free(gen)
    n_cols = col1 - col0
    if hetero:
        w = torch.empty(idx.shape, dtype=torch.float32, device=device)
        conn = (FixedPostNumConn((w, idx), shape=(n_pre, n_cols)) if indptr is None
                else CSR((w, idx, indptr), shape=(n_pre, n_cols)))
        st = conn._struct()
        check(l.bsx_lognormal_weights(C.byref(st), _lib.ptr(kpos), 0, C.c_uint32(int(weight.seed) & 0xffffffff),
                                      float(weight.mu), float(weight.sigma), float(weight.scale), w.data_ptr(),
                                      _lib.current_stream()))
        torch.cuda.synchronize(device)
        return conn
    if indptr is None:
        return FixedPostNumConn((float(weight), idx), shape=(n_pre, n_cols))
    return CSR((float(weight), idx, indptr), shape=(n_pre, n_cols))


def build_projection_in_degree(seed: int, n_pre: int, n_post: int, k_in: int, weight, device, row0: int = 0,
                               row1: Optional[int] = None):
    """One projection with a fixed IN-degree: every postsynaptic neuron draws ``k_in`` presynaptic
    partners, ``RandomState(seed).randint(0, n_pre, (n_post, k_in))`` — the same generator call as
    ``brainstate/nn/_event_fixedprob.py:165-171`` with the roles exchanged.  ``[row0, row1)`` selects
    the postsynaptic shard (its rows of the one seeded stream).  The step kernels scatter along
    presynaptic rows, so the result is the presynaptic-major CSR copy (built on the device by
    ``bsx_transpose_build``), local column ids.  Homogeneous weights only."""
    if not isinstance(weight, (int, float)):
        raise NotImplementedError('fixed in-degree projections take one weight per projection')
    row1 = n_post if row1 is None else row1
    n_local = row1 - row0
    buf = np.empty(max(n_local * k_in, 1), np.int32)
    n = lib().bsx_host_fixed_num_indices(C.c_uint32(int(seed) & 0xffffffff), n_post, n_pre, k_in, row0, row1, 0, 0,
                                        buf.ctypes.data, None)
    check(int(n))
    idx_in = torch.from_numpy(buf[:n_local * k_in].reshape(n_local, k_in)).to(device)
    mirror = FixedPostNumConn((float(weight), idx_in), shape=(n_local, n_pre))     # rows: local postsynaptic neurons
    t = mirror.transposed()
    return CSR((float(weight), t.indices, t.indptr), shape=(n_pre, n_local))


class EINet:
    """E/I network of LIF neurons with exponential synapses.

    Parameters
    ----------
    n_exc, n_inh : population sizes; global ids ``[0, n_exc)`` are excitatory.
    conn_num : connection probability (float) or number of targets per neuron (int),
        as in ``EventFixedProb``.
    w_e, w_i : synaptic weights of the two projections: a float (homogeneous) or
        :class:`Lognormal` (heterogeneous, generated on the device).
    seed_e, seed_i : connectivity seeds (``EventFixedProb(..., seed=...)``).
    V0 : initial membrane potentials, ``(n_exc + n_inh,)``.
    delay_e, delay_i : synaptic delays in steps beyond the next step (0: a spike of
        step t acts at step t+1).  The spikes wait in a ring of bit-packed-by-index
        lists, the counterpart of the reference's delay ring buffer
        (``brainstate/nn/_delay.py:768-958``) for spike vectors.
    group : optional ``torch.distributed`` process group; with more than one rank
        the postsynaptic neurons are sharded.
    exchange : ``'p2p'`` — the spike exchange is part of the step kernel (one launch per
        GPU for all steps of a ``run``); ``'nccl'`` — one all-gather per step between
        split-phase launches.
    deterministic : accumulate the synaptic input in 2^-32 fixed point (64-bit integer
        adds).  The sums are then independent of the order in which the GPU adds them, so
        the raster of a network with heterogeneous weights is the same on every run, grid
        and number of GPUs.  Uses the kernel of ``exchange='p2p'`` also on one GPU.
    slack : with ``exchange='p2p'`` and both delays at least ``slack`` steps, spikes are
        consumed ``slack`` steps after they were sent, which takes the NVLink latency off
        the critical path.  Default: ``min(delay_e, delay_i)``.
    conn : ``(conn_e, conn_i)`` of an ``EINet`` of the same network and shard: the projections
        are shared instead of drawn again (a second network over the same synapses).
    shard_kernel : on one GPU, ``True`` runs the kernel of ``exchange='p2p'`` (increment rows,
        one grid-wide barrier per step whatever the delays) instead of the spike-list kernels.
    degree : ``'out'`` — every neuron has ``conn_num`` targets (the reference's ``efferent_target='post'``
        layout); ``'in'`` — every neuron has ``conn_num`` presynaptic partners, ``conn_num * n_exc / n`` of
        them excitatory (fixed in-degree; homogeneous weights).
    health_group, health_timeout : a ``gloo`` process group over the same ranks and a patience in
        seconds: every ``run`` on several GPUs starts with :func:`wait_for_peers`, so a lost or late
        rank is noticed on the host (``PeerLost``) before anything is launched.
    overlap : with ``exchange='nccl'``, run the all-gather of a step on the process group's stream
        while the rank's own spikes are scattered for the next step, instead of the strictly
        sequential scatter -> update -> all-gather -> list.  It doubles the launches per step, so it
        pays only when the steps are replayed from a CUDA graph (``run(..., graph_steps=)``:
        32 against 36 us per step on two GPUs at 10^6 neurons; eager 69 against 41).
    """

    def __init__(self, n_exc: int, n_inh: int, conn_num, w_e, w_i, *, seed_e: int, seed_i: int,
                 V0, params: Optional[LIFParams] = None, device=None, group=None, delay_e: int = 0,
                 delay_i: int = 0, exchange: str = 'p2p', deterministic: bool = False,
                 slack: Optional[int] = None, shard_kernel: Optional[bool] = None, conn=None,
                 overlap: bool = False, degree: str = 'out', health_group=None, health_timeout: float = 5.0):
        if exchange not in ('nccl', 'p2p'):
            raise ValueError("exchange must be 'nccl' or 'p2p'")
        self.exchange = exchange
        self.overlap = bool(overlap)
        self.health_group, self.health_timeout = health_group, float(health_timeout)
        self.deterministic = bool(deterministic)
        self._links = None
        self._seq = 0
        self.link_flags = _lib.LINK_DEFAULT
        self.delay_e, self.delay_i = int(delay_e), int(delay_i)
        self.ring = max(self.delay_e, self.delay_i) + 2
        self.n_exc, self.n_inh = int(n_exc), int(n_inh)
        self.n = self.n_exc + self.n_inh
        self.params = params or LIFParams()
        self.dev = _device(device)
        self.group = group
        self.world, self.rank = 1, 0
        if group is not None:
            import torch.distributed as dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.first, self.last = shard_bounds(self.n, self.world, self.rank) if self.world > 1 else (0, self.n)
        self.n_local = self.last - self.first
        K = conn_num if isinstance(conn_num, int) else int(self.n * conn_num)
        self.conn_num = K
        dev = self.dev
        hetero = isinstance(w_e, Lognormal) or isinstance(w_i, Lognormal)
        if degree not in ('out', 'in'):
            raise ValueError("degree must be 'out' or 'in'")
        self.degree = degree
        if conn is not None:
            self.conn_e, self.conn_i = conn
            if self.conn_e.shape != (self.n_exc, self.n_local) or self.conn_i.shape != (self.n_inh, self.n_local):
                raise ValueError('conn: projections of another network or shard')
        elif degree == 'in':
            k_e = int(round(K * self.n_exc / self.n))
            self.in_degree = (k_e, K - k_e)                 # presynaptic partners per neuron: excitatory, inhibitory
            self.conn_e = build_projection_in_degree(seed_e, self.n_exc, self.n, k_e, w_e, dev, self.first, self.last)
            self.conn_i = build_projection_in_degree(seed_i, self.n_inh, self.n, K - k_e, w_i, dev, self.first, self.last)
        elif self.world == 1 and not hetero and self.n * K < (1 << 31):
            self.E = EventFixedProb(self.n_exc, self.n, K, float(w_e), seed=seed_e, device=dev)
            self.I = EventFixedProb(self.n_inh, self.n, K, float(w_i), seed=seed_i, device=dev)
            self.conn_e, self.conn_i = self.E.conn, self.I.conn
        else:
            c0, c1 = (0, self.n) if self.world == 1 else (self.first, self.last)
            self.conn_e = build_projection(seed_e, self.n_exc, self.n, K, w_e, dev, c0, c1)
            self.conn_i = build_projection(seed_i, self.n_inh, self.n, K, w_i, dev, c0, c1)
        V0 = np.asarray(V0, np.float32)
        assert V0.shape == (self.n,)
        self.V = torch.from_numpy(V0[self.first:self.last].copy()).to(dev)
        z = lambda dt: torch.zeros(self.n_local, dtype=dt, device=dev)
        self.g_e, self.g_i, self.delta_e, self.delta_i = z(torch.float32), z(torch.float32), z(torch.float32), z(torch.float32)
        self.ref = z(torch.int32)
        self.words = (self.n + 31) // 32
        self.wpr = words_per_rank(self.n, self.world)
        self.bits = torch.zeros(self.wpr * self.world, dtype=torch.int32, device=dev)
        self.step_count = 0
        self._graphs = {}
        self._warmed = False
        self._pstruct = self.params.struct()
        # which kernel family runs the steps: the shard kernel (state: ring of increment rows)
        # or the spike-list kernels (state: ring of spike lists)
        self.shard_kernel = (self.world > 1 and exchange == 'p2p') or self.deterministic
        if shard_kernel is not None and self.world == 1 and not self.deterministic:
            self.shard_kernel = bool(shard_kernel)       # one GPU: either family can run the network
        if self.world > 1 and self.deterministic and exchange != 'p2p':
            raise ValueError("deterministic=True on several GPUs needs exchange='p2p'")
        dmin = min(self.delay_e, self.delay_i)
        self.slack = dmin if slack is None else int(slack)
        if not 0 <= self.slack <= dmin:
            raise ValueError(f'slack must lie in [0, min(delay_e, delay_i)] = [0, {dmin}]')
        if self.shard_kernel:
            acc = torch.int64 if self.deterministic else torch.float32
            self.incr_e = torch.zeros((self.ring, self.n_local), dtype=acc, device=dev)
            self.incr_i = torch.zeros((self.ring, self.n_local), dtype=acc, device=dev)
            self.lists = None
            self._shard = self._make_shard_struct()
            self._net = None
        else:
            self.lists = torch.zeros((self.ring, self.n + 1), dtype=torch.int32, device=dev)
            self.marks = torch.zeros(self.ring, dtype=torch.int32, device=dev)
            self._net = self._make_struct()

    def _make_struct(self) -> BsxNet:
        s = BsxNet()
        s.n_global, s.n_exc, s.first, s.n_local = self.n, self.n_exc, self.first, self.n_local
        self._se, self._si = self.conn_e._struct(), self.conn_i._struct()
        s.exc, s.inh = self._se, self._si
        s.V, s.g_e, s.g_i, s.ref = self.V.data_ptr(), self.g_e.data_ptr(), self.g_i.data_ptr(), self.ref.data_ptr()
        s.delta_e, s.delta_i = self.delta_e.data_ptr(), self.delta_i.data_ptr()
        s.bits = self.bits.data_ptr()
        s.lists = self.lists.data_ptr()
        s.ring, s.delay_e, s.delay_i = self.ring, self.delay_e, self.delay_i
        return s

    def _make_shard_struct(self) -> BsxNetShard:
        s = BsxNetShard()
        s.n_global, s.n_exc, s.first, s.n_local = self.n, self.n_exc, self.first, self.n_local
        self._se, self._si = self.conn_e._struct(), self.conn_i._struct()
        s.exc, s.inh = self._se, self._si
        s.V, s.g_e, s.g_i, s.ref = self.V.data_ptr(), self.g_e.data_ptr(), self.g_i.data_ptr(), self.ref.data_ptr()
        s.incr_e, s.incr_i = self.incr_e.data_ptr(), self.incr_i.data_ptr()
        s.bits = self.bits.data_ptr() + 4 * self.rank * self.wpr
        s.ring, s.delay_e, s.delay_i = self.ring, self.delay_e, self.delay_i
        s.fixed_point = int(self.deterministic)
        return s

    # ------------------------------------------------------------------
    def run(self, steps: int, record: bool = True, blocks: int = 0, graph_steps: int = 0):
        """Advances ``steps`` steps.  Returns ``(raster, counts)``: the packed spike
        words ``(steps, ceil(n/32))`` int32 (``None`` without ``record``) and the
        number of spikes of every step ``(steps,)`` int32.  ``graph_steps`` (only with
        ``exchange='nccl'`` on several GPUs): replay chunks of that many steps from a captured
        CUDA graph."""
        if self.world > 1 and self.health_group is not None:
            wait_for_peers(self.health_group, self.health_timeout)
        if self.shard_kernel:
            return self._run_shard_kernel(steps, record)
        if self.world > 1:
            return self._run_sharded(steps, record, graph_steps)
        dev = self.dev
        raster = torch.empty((steps, self.words), dtype=torch.int32, device=dev) if record else None
        counts = torch.empty(steps, dtype=torch.int32, device=dev)
        check(lib().bsx_net_run(C.byref(self._net), C.byref(self._pstruct), steps, self.step_count,
                                _lib.ptr(raster), counts.data_ptr(), blocks, _lib.current_stream()))
        self.step_count += steps
        return raster, counts

    def _sharded_step(self, t: int, counts, raster_rows):
        """Enqueues one step on the current stream: scatter the delayed spikes (all ranks'
        spikes, this rank's targets), update the local neurons, all-gather the packed spike
        words, rebuild the spike list.

        With ``overlap`` the all-gather runs on the process group's own stream while the
        current stream scatters this rank's OWN spikes of the lists the next step reads (they
        are known without the exchange: the list's first section, ``marks`` holds its length);
        the other ranks' section of each list is scattered at the start of the next step.
        Between steps the increments ``delta_e`` / ``delta_i`` then already hold the own-spike
        part of the next step's input, which is why a checkpoint records the mode."""
        import torch.distributed as dist
        l = lib()
        stream = _lib.current_stream()
        net, ps = C.byref(self._net), C.byref(self._pstruct)
        step = self.step_count
        if not self.overlap:
            check(l.bsx_net_scatter(net, step, stream))
            check(l.bsx_net_update(net, ps, step, counts[t:t + 1].data_ptr(), stream))
            dist.all_gather_into_tensor(self.bits, self._mine, group=self.group)
            check(l.bsx_net_list_from_bits(net, step, stream))
        else:
            w0 = self.rank * self.wpr
            w1 = min(w0 + self.wpr, self.words)
            marks = self.marks.data_ptr()
            check(l.bsx_net_scatter_part(net, step, marks, 1, stream))            # the other ranks' spikes
            check(l.bsx_net_update(net, ps, step, counts[t:t + 1].data_ptr(), stream))
            check(l.bsx_net_list_from_bits_part(net, step, w0, w1, 0, marks, stream))
            work = dist.all_gather_into_tensor(self.bits, self._mine, group=self.group, async_op=True)
            check(l.bsx_net_scatter_part(net, step + 1, marks, 0, stream))        # own spikes, during the exchange
            work.wait()
            check(l.bsx_net_list_from_bits_part(net, step, w0, w1, 1, marks, stream))
        if raster_rows is not None:
            raster_rows[t].copy_(self.bits[:self.words])
        self.step_count += 1

    def _run_sharded(self, steps: int, record: bool, graph_steps: int = 0):
        """Multi-rank run.  With ``graph_steps`` > 0, whole chunks of that many (even)
        steps are replayed from a captured CUDA graph, which removes the per-launch
        host cost; the rest, and everything by default, runs eagerly."""
        import torch.distributed as dist
        dev = self.dev
        self._mine = self.bits[self.rank * self.wpr:(self.rank + 1) * self.wpr]
        raster = torch.empty((steps, self.words), dtype=torch.int32, device=dev) if record else None
        counts = torch.zeros(steps, dtype=torch.int32, device=dev)
        t = 0
        S = graph_steps - (graph_steps % self.ring)      # a whole number of turns of the list ring
        # A captured launch carries its step number by value.  Replays are right only where the
        # step enters through ``step % ring`` alone: no background drive (hashed from the step),
        # and every delayed list already exists (the step - 1 - delay >= 0 tests are past).
        if S >= self.ring and self.params.ext_threshold != 0:
            raise ValueError('CUDA-graph replay of the sharded step is not available with a background drive')
        if S >= self.ring and steps >= 2 * S:
            if not self._warmed:       # NCCL and lazy module loading must have run before a capture
                c0 = torch.zeros(2, dtype=torch.int32, device=dev)
                r0 = torch.empty((2, self.words), dtype=torch.int32, device=dev) if record else None
                for k in range(2):
                    self._sharded_step(k, c0, r0)
                counts[0:2].copy_(c0)
                if record:
                    raster[0:2].copy_(r0)
                t = 2
                self._warmed = True
                torch.cuda.synchronize()
            while self.step_count <= max(self.delay_e, self.delay_i) + 1 and t < steps:   # eager until every list exists
                c0 = torch.zeros(1, dtype=torch.int32, device=dev)
                r0 = torch.empty((1, self.words), dtype=torch.int32, device=dev) if record else None
                self._sharded_step(0, c0, r0)
                counts[t:t + 1].copy_(c0)
                if record:
                    raster[t:t + 1].copy_(r0)
                t += 1
            key = (S, record, self.step_count % self.ring)
            if key not in self._graphs:
                gc = torch.zeros(S, dtype=torch.int32, device=dev)
                gr = torch.empty((S, self.words), dtype=torch.int32, device=dev) if record else None
                step_before = self.step_count
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    gc.zero_()
                    for k in range(S):
                        self._sharded_step(k, gc, gr)
                self.step_count = step_before          # capture enqueues nothing: no step was taken
                self._graphs[key] = (g, gc, gr)
            g, gc, gr = self._graphs[key]
            while steps - t >= S:
                g.replay()
                self.step_count += S
                counts[t:t + S].copy_(gc)
                if record:
                    raster[t:t + S].copy_(gr)
                t += S
        if t < steps:
            rest = steps - t
            c1 = torch.zeros(rest, dtype=torch.int32, device=dev)
            r1 = torch.empty((rest, self.words), dtype=torch.int32, device=dev) if record else None
            for k in range(rest):
                self._sharded_step(k, c1, r1)
            counts[t:].copy_(c1)
            if record:
                raster[t:].copy_(r1)
        dist.all_reduce(counts, group=self.group)
        return raster, counts


    # ------------------------------------------------------------------
    def spikes(self) -> torch.Tensor:
        """Spikes of the latest step as a bool vector over the whole network."""
        w = self.bits[:self.words].cpu().numpy().view(np.uint32)
        b = np.unpackbits(w.view(np.uint8), bitorder='little')[:self.n].astype(bool)
        return torch.from_numpy(b)

    # -- shard kernel: exchange inside the step kernel (peer stores over NVLink) --------
    def _setup_links(self):
        """Launch geometry, the two synchronisation words and — with more than one rank — this
        rank's inbox, exported to the other ranks of the node and theirs mapped (CUDA IPC;
        one-time)."""
        l = lib()
        blocks, wpb = C.c_int32(0), C.c_int32(0)
        check(l.bsx_net_shard_geometry(self.wpr, C.byref(blocks), C.byref(wpb)))
        links = BsxNetLinks()
        links.world, links.rank = self.world, self.rank
        links.blocks, links.words_per_block, links.words_per_rank = blocks.value, wpb.value, self.wpr
        links.slack, links.slots = (self.slack if self.world > 1 else 0), 2 * self.slack + 2
        links.spin_limit = 0
        links.flags = self.link_flags
        sync = torch.zeros(2, dtype=torch.int32, device=self.dev)
        links.sync = sync.data_ptr()
        state = {'links': links, 'sync': sync, 'base': None, 'opened': []}
        if self.world > 1:
            import torch.distributed as dist
            nbytes = l.bsx_net_inbox_bytes(self.world, blocks.value, wpb.value, links.slots)
            base = C.c_void_p()
            handle = C.create_string_buffer(64)
            check(l.bsx_ipc_alloc(nbytes, C.byref(base), handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=self.group)
            for r in range(self.world):
                if r == self.rank:
                    links.inbox[r] = base.value
                else:
                    q = C.c_void_p()
                    check(l.bsx_ipc_open(C.create_string_buffer(handles[r], 64), C.byref(q)))
                    links.inbox[r] = q.value
                    state['opened'].append(q.value)
            state['base'] = base.value
            dist.barrier(group=self.group)                # every rank has mapped every inbox
        self._links = state
        self._seq = 0

    def prepare(self):
        """One-time set-up that would otherwise happen inside the first ``run``: the launch
        geometry and, with several ranks, the inboxes and their peer mappings (collective)."""
        if self.shard_kernel and self._links is None:
            self._setup_links()
        return self

    def _run_shard_kernel(self, steps: int, record: bool):
        """All steps in one cooperative launch per GPU; the spike ids travel by peer stores
        inside the kernel.  The raster of the whole network is assembled from the ranks'
        words after the launch."""
        if self._links is None:
            self._setup_links()
        dev = self.dev
        if self.world > 1:
            import torch.distributed as dist
            # the kernels of all ranks wait for one another with a bounded patience (about a
            # second): line the hosts up first so that none of them launches much later
            dist.barrier(group=self.group)
        words_local = (self.n_local + 31) // 32
        mine = torch.empty((steps, words_local), dtype=torch.int32, device=dev) if record else None
        counts = torch.empty(steps, dtype=torch.int32, device=dev)
        links = self._links['links']
        links.seq0 = self._seq
        check(lib().bsx_net_run_sharded(C.byref(self._shard), C.byref(self._pstruct), C.byref(links), steps,
                                        self.step_count, _lib.ptr(mine), counts.data_ptr(), _lib.current_stream()))
        host = C.c_int32(0)
        check(lib().bsx_read_status(self._links['sync'].data_ptr(), C.byref(host), _lib.current_stream()))
        if host.value == _lib.BSX_ERR_NONFINITE:
            self._links['sync'].zero_()
            raise FloatingPointError('a neuron state became NaN or infinite; the run stopped at the end of '
                                     'that step (BSX_ERR_NONFINITE)')
        if host.value != 0:
            self._drop_links()
            raise RuntimeError('the multi-GPU step kernel gave up waiting for a peer '
                               f'({lib().bsx_status_name(host.value).decode()}); the run stopped early and '
                               'the exchange buffers were dropped')
        self.step_count += steps
        self._seq += steps
        if self.world == 1:
            return mine, counts
        import torch.distributed as dist
        mine_bits = self.bits[self.rank * self.wpr:(self.rank + 1) * self.wpr]
        dist.all_gather_into_tensor(self.bits, mine_bits.clone(), group=self.group)   # latest step, whole network
        raster = None
        if record:
            padded = torch.zeros((steps, self.wpr), dtype=torch.int32, device=dev)
            padded[:, :words_local] = mine
            parts = torch.empty((self.world, steps, self.wpr), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(parts, padded, group=self.group)
            raster = parts.permute(1, 0, 2).reshape(steps, self.world * self.wpr)[:, :self.words].contiguous()
        return raster, counts

    def _drop_links(self):
        if self._links is None:
            return
        for q in self._links['opened']:
            lib().bsx_ipc_close(q)
        if self._links['base'] is not None:
            lib().bsx_ipc_free(self._links['base'])
        self._links = None

    def close(self):
        """Drops the captured CUDA graphs and the peer mappings.  Call it before the
        process group is destroyed: a live graph that holds captured collectives keeps
        the communicator busy and the teardown waits for it."""
        if self._links is not None and self.world > 1:
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=self.group)                # nobody still writes into a buffer about to go
            for q in self._links['opened']:
                lib().bsx_ipc_close(q)
            self._links['opened'] = []
            dist.barrier(group=self.group)
        self._drop_links()
        self._graphs.clear()
        import gc
        gc.collect()
        torch.cuda.synchronize()

    # -- checkpoint / resume --------------------------------------------------
    _STATE = ('V', 'g_e', 'g_i', 'ref', 'delta_e', 'delta_i', 'bits', 'lists', 'marks', 'incr_e', 'incr_i')

    def _meta(self) -> dict:
        return {'n_exc': self.n_exc, 'n_inh': self.n_inh, 'conn_num': self.conn_num, 'ring': self.ring,
                'first': self.first, 'n_local': self.n_local, 'shard_kernel': self.shard_kernel,
                'deterministic': self.deterministic, 'degree': self.degree,
                'own_spikes_scattered_ahead': bool(self.world > 1 and not self.shard_kernel and self.overlap)}

    def state_dict(self) -> dict:
        """Everything a resumed run needs that cannot be regenerated: the rank's neuron
        state, the pending synaptic input (spike lists, or increment rows with the shard
        kernel) and the step counter.  The connectivity is not stored; like the reference
        (whose index arrays are plain attributes, not states,
        ``brainstate/nn/_event_fixedprob.py:181``) it is rebuilt from the seeds."""
        sd = {k: getattr(self, k).clone() for k in self._STATE if getattr(self, k, None) is not None}
        sd['step'] = self.step_count
        sd['meta'] = self._meta()
        return sd

    def load_state_dict(self, sd: dict):
        """Restores a checkpoint of the same network, shard and kernel family.  The exchange
        sequence number of the inboxes is NOT rewound: it counts what went through them, not
        the simulation step."""
        if sd['meta'] != self._meta():
            raise ValueError(f"checkpoint of a different network or shard: {sd['meta']} vs {self._meta()}")
        for k in self._STATE:
            if getattr(self, k, None) is not None:
                getattr(self, k).copy_(sd[k])
        self.step_count = int(sd['step'])


# Constant bias current of the 'coba' preset (same unit as a conductance times a potential:
# with R = 0.1 the membrane sees R * I = 16.8 mV above rest).  Found by bisection on the full
# 10^6-neuron network on a B200: mean rate over the configuration's 1000 steps (100 ms) from
# the seeded start 10.02 Hz (9.92 Hz at 166, 10.26 Hz at 172); 9.1 Hz once the initial
# transient of the first 200 steps is left out.
COBA_BIAS = 168.0


def preset(name: str) -> dict:
    """The three network recipes, as keyword material for :class:`EINet`:

    cuba   4 000 current-based LIF neurons, p = 0.02 (80 targets), weights +1.62 / -9 mV,
           V_rest -49 mV above V_th -50 mV (self-active), V0 ~ U(-60, -50), seeds 100-102
           (``examples/400_CUBA_2005_bpu.py:36-58`` with its constants)
    coba   1 000 000 conductance-based LIF neurons (800k E / 200k I), 100 targets per neuron,
           g 0.6 / 6.7, E_e 0, E_i -80 mV, V_rest -60 mV, constant bias ``COBA_BIAS`` giving
           about 10 Hz, V0 ~ U(-60, -50), seeds 300-302
    large  8 000 000 LIF neurons, 1000 targets per neuron (8e9 synapses), lognormal(-2, 0.5)
           weights signed by population (inhibition x6), hashed background drive giving
           about 5 Hz, seeds 400-405
    """
    if name == 'cuba':
        return dict(n_exc=3200, n_inh=800, conn_num=80, w_e=1.62, w_i=-9.0, params=LIFParams(), seed_e=100,
                    seed_i=101, seed_v=102, v0=(-60., -50.))
    if name == 'coba':
        return dict(n_exc=800000, n_inh=200000, conn_num=100, w_e=0.6, w_i=6.7,
                    params=LIFParams(coba=True, R=0.1, V_rest=-60., E_e=0., E_i=-80., tau_e=5., tau_i=10.,
                                     I_ext=COBA_BIAS),
                    seed_e=300, seed_i=301, seed_v=302, v0=(-60., -50.))
    if name == 'large':
        return dict(n_exc=6400000, n_inh=1600000, conn_num=1000, w_e=Lognormal(-2.0, 0.5, 402, 1.0),
                    w_i=Lognormal(-2.0, 0.5, 403, -6.0),
                    params=LIFParams(V_rest=-60., ext_rate_hz=9000., ext_weight=0.3, ext_seed=405),
                    seed_e=400, seed_i=401, seed_v=404, v0=(-65., -52.))
    raise ValueError(f'unknown preset {name!r}')


def from_preset(name: str, device=None, group=None, scale: float = 1.0, **kw) -> 'EINet':
    """Builds the network of :func:`preset` (``scale`` shrinks both populations)."""
    p = preset(name)
    n_exc, n_inh = int(p['n_exc'] * scale), int(p['n_inh'] * scale)
    V0 = np.random.RandomState(p['seed_v']).uniform(p['v0'][0], p['v0'][1], n_exc + n_inh).astype(np.float32)
    return EINet(n_exc, n_inh, p['conn_num'], p['w_e'], p['w_i'], seed_e=p['seed_e'], seed_i=p['seed_i'], V0=V0,
                 params=p['params'], device=device, group=group, **kw)


def population_rates(counts_or_raster, n_exc: int, n_inh: int, dt_ms: float):
    """Mean firing rates in Hz of the excitatory and the inhibitory population from a packed
    raster ``(steps, words)`` (ids below ``n_exc`` are excitatory)."""
    r = unpack_raster(counts_or_raster, n_exc + n_inh)
    seconds = r.shape[0] * dt_ms * 1e-3
    return float(r[:, :n_exc].sum() / max(n_exc, 1) / seconds), float(r[:, n_exc:].sum() / max(n_inh, 1) / seconds)


def unpack_raster(raster: torch.Tensor, n: int) -> np.ndarray:
    """``(steps, words)`` packed words -> ``(steps, n)`` bool array (host)."""
    w = raster.cpu().numpy().view(np.uint32)
    bits = np.unpackbits(w.view(np.uint8).reshape(w.shape[0], -1), axis=1, bitorder='little')
    return bits[:, :n].astype(bool)
