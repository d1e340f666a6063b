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
the same seeded stream as the full matrix) and the ranks exchange one all-gather of
the packed spike words per step.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import BsxLifParams, BsxNet, check, lib
from .event import CSR, FixedPostNumConn
from .nn._event_fixedprob import EventFixedProb, _device

__all__ = ['LIFParams', 'Lognormal', 'EINet', 'shard_bounds', 'words_per_rank', 'sharded_block',
           'build_projection', 'unpack_raster']


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
    buf = np.empty(n_pre * conn_num, np.int32)
    counts = np.empty(n_pre, np.int32)
    n = lib().bsx_host_fixed_num_indices(C.c_uint32(int(seed) & 0xffffffff), n_pre, n_post, conn_num, 0, n_pre,
                                        col0, col1, buf.ctypes.data, counts.ctypes.data)
    check(int(n))
    indptr = np.zeros(n_pre + 1, np.int64)
    np.cumsum(counts, out=indptr[1:])
    return buf[:n].copy(), indptr


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
    """

    def __init__(self, n_exc: int, n_inh: int, conn_num, w_e, w_i, *, seed_e: int, seed_i: int,
                 V0, params: Optional[LIFParams] = None, device=None, group=None, delay_e: int = 0,
                 delay_i: int = 0, exchange: str = 'nccl'):
        if exchange not in ('nccl', 'p2p'):
            raise ValueError("exchange must be 'nccl' or 'p2p'")
        self.exchange = exchange
        self._p2p = None
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
        if self.world == 1 and not hetero and self.n * K < (1 << 31):
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
        self.lists = torch.zeros((self.ring, self.n + 1), dtype=torch.int32, device=dev)
        self.step_count = 0
        self._graphs = {}
        self._warmed = False
        self._pstruct = self.params.struct()
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

    # ------------------------------------------------------------------
    def run(self, steps: int, record: bool = True, blocks: int = 0):
        """Advances ``steps`` steps.  Returns ``(raster, counts)``: the packed spike
        words ``(steps, ceil(n/32))`` int32 (``None`` without ``record``) and the
        number of spikes of every step ``(steps,)`` int32."""
        if self.world > 1 and self.exchange == 'p2p':
            return self._run_p2p(steps, record, blocks)
        if self.world > 1:
            return self._run_sharded(steps, record)
        dev = self.dev
        raster = torch.empty((steps, self.words), dtype=torch.int32, device=dev) if record else None
        counts = torch.empty(steps, dtype=torch.int32, device=dev)
        check(lib().bsx_net_run(C.byref(self._net), C.byref(self._pstruct), steps, self.step_count,
                                _lib.ptr(raster), counts.data_ptr(), blocks, _lib.current_stream()))
        self.step_count += steps
        return raster, counts

    def _sharded_step(self, t: int, counts, raster_rows):
        """Enqueues one step on the current stream: scatter the previous step's spikes
        (all ranks' spikes, this rank's targets), update the local neurons, all-gather
        the packed spike words, rebuild the spike list."""
        import torch.distributed as dist
        l = lib()
        stream = _lib.current_stream()
        net, ps = C.byref(self._net), C.byref(self._pstruct)
        step = self.step_count
        check(l.bsx_net_scatter(net, step, stream))
        check(l.bsx_net_update(net, ps, step, counts[t:t + 1].data_ptr(), stream))
        dist.all_gather_into_tensor(self.bits, self._mine, group=self.group)
        check(l.bsx_net_list_from_bits(net, step, stream))
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

    # -- exchange inside the kernel (peer stores over NVLink) ---------------------
    def _setup_p2p(self):
        """Allocates this rank's exchange buffer and progress counters, exports them to
        the other ranks of the node and maps theirs (CUDA IPC; one-time)."""
        import torch.distributed as dist
        from ._lib import BsxNetPeers
        l = lib()
        words = self.wpr * self.world
        bits_bytes = 2 * words * 4
        flags_off = (bits_bytes + 255) // 256 * 256
        total = flags_off + 256 + 256                     # counters (world x int64), status word
        base = C.c_void_p()
        handle = C.create_string_buffer(64)
        check(l.bsx_ipc_alloc(total, C.byref(base), handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=self.group)
        ptrs, opened = [], []
        for r in range(self.world):
            if r == self.rank:
                ptrs.append(base.value)
            else:
                q = C.c_void_p()
                check(l.bsx_ipc_open(C.create_string_buffer(handles[r], 64), C.byref(q)))
                ptrs.append(q.value)
                opened.append(q.value)
        peers = BsxNetPeers()
        peers.world, peers.rank, peers.words_per_rank, peers.spin_limit = self.world, self.rank, self.wpr, 0
        for r in range(self.world):
            peers.bits[r] = ptrs[r]
            peers.flags[r] = ptrs[r] + flags_off
        peers.status = base.value + flags_off + 256
        self._p2p = {'peers': peers, 'base': base.value, 'opened': opened, 'status_ptr': base.value + flags_off + 256}
        dist.barrier(group=self.group)                    # every rank has mapped every buffer

    def _run_p2p(self, steps: int, record: bool, blocks: int = 0):
        """All steps of all ranks in one cooperative launch per GPU; the spike words
        travel by peer stores inside the kernel."""
        import torch.distributed as dist
        if self._p2p is None:
            self._setup_p2p()
        # the kernels of all ranks wait for one another with a bounded patience (about a
        # second): line the hosts up first so that none of them launches much later
        dist.barrier(group=self.group)
        dev = self.dev
        raster = torch.empty((steps, self.words), dtype=torch.int32, device=dev) if record else None
        counts = torch.empty(steps, dtype=torch.int32, device=dev)
        check(lib().bsx_net_run_p2p(C.byref(self._net), C.byref(self._pstruct), C.byref(self._p2p['peers']), steps,
                                    self.step_count, _lib.ptr(raster), counts.data_ptr(), blocks,
                                    _lib.current_stream()))
        host = C.c_int32(0)
        check(lib().bsx_read_status(self._p2p['status_ptr'], C.byref(host), _lib.current_stream()))
        if host.value != 0:
            raise RuntimeError('the multi-GPU step kernel gave up waiting for a peer '
                               f'({lib().bsx_status_name(host.value).decode()}); the run stopped early')
        self.step_count += steps
        return raster, counts

    def close(self):
        """Drops the captured CUDA graphs and the peer mappings.  Call it before the
        process group is destroyed: a live graph that holds captured collectives keeps
        the communicator busy and the teardown waits for it."""
        if self._p2p is not None:
            import torch.distributed as dist
            torch.cuda.synchronize()
            dist.barrier(group=self.group)                # nobody still writes into a buffer about to go
            for q in self._p2p['opened']:
                lib().bsx_ipc_close(q)
            dist.barrier(group=self.group)
            lib().bsx_ipc_free(self._p2p['base'])
            self._p2p = None
        self._graphs.clear()
        import gc
        gc.collect()
        torch.cuda.synchronize()

    # -- checkpoint / resume --------------------------------------------------
    def state_dict(self) -> dict:
        """Everything a resumed run needs that cannot be regenerated: the rank's neuron
        state, the pending spike lists and the step counter.  The connectivity is not
        stored; like the reference (whose index arrays are plain attributes, not
        states, ``brainstate/nn/_event_fixedprob.py:181``) it is rebuilt from the seeds."""
        return {'V': self.V.clone(), 'g_e': self.g_e.clone(), 'g_i': self.g_i.clone(), 'ref': self.ref.clone(),
                'delta_e': self.delta_e.clone(), 'delta_i': self.delta_i.clone(), 'bits': self.bits.clone(),
                'lists': self.lists.clone(), 'step': self.step_count,
                'meta': {'n_exc': self.n_exc, 'n_inh': self.n_inh, 'conn_num': self.conn_num, 'ring': self.ring,
                         'first': self.first, 'n_local': self.n_local}}

    def load_state_dict(self, sd: dict):
        m = sd['meta']
        mine = {'n_exc': self.n_exc, 'n_inh': self.n_inh, 'conn_num': self.conn_num, 'ring': self.ring,
                'first': self.first, 'n_local': self.n_local}
        if m != mine:
            raise ValueError(f'checkpoint of a different network or shard: {m} vs {mine}')
        for k in ('V', 'g_e', 'g_i', 'ref', 'delta_e', 'delta_i', 'bits', 'lists'):
            getattr(self, k).copy_(sd[k])
        self.step_count = int(sd['step'])


def unpack_raster(raster: torch.Tensor, n: int) -> np.ndarray:
    """``(steps, words)`` packed words -> ``(steps, n)`` bool array (host)."""
    w = raster.cpu().numpy().view(np.uint32)
    bits = np.unpackbits(w.view(np.uint8).reshape(w.shape[0], -1), axis=1, bitorder='little')
    return bits[:, :n].astype(bool)
