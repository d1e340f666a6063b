#!/usr/bin/env python
"""Benchmark of the event-driven synaptic propagation path on B200.

Workload (the standalone event-matvec microbenchmark): a 65 536 x 65 536 sparse
matrix with fixed-probability connectivity p = 0.01 (655 int32 targets per row,
seed 200), heterogeneous float32 weights ~ N(0.1, 0.01) (seed 201), and T
distinct Bernoulli(1 %) spike vectors (seed 211).  One step = one pass of the hot
path over that batch: the forward product ``spike @ W`` of all T vectors (one
batched scatter launch) and the event matvec ``W @ spike`` of all T vectors in
the variant the firing rate selects — at 1 % the event-driven one, in which the
active columns scatter along the transposed copy of the matrix (one launch);
above 3 % it would be the deterministic gather (one pass per 16 vectors), which
is timed beside the step for its own roofline.  ``value`` = synaptic events per
second = (events of both products over the batch) / time, with everything
resident in HBM.  ``e2e`` is the
same pass through the public layer API starting from pinned host spikes and
ending with the results back in host memory.  Data are synthetic, generated from
the seeds above; the matrix (343 MB) is larger than the 126 MB L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--vectors T] [--no-cases] [--no-network] [--no-large]

With N > 1 (torchrun, one rank per GPU) every rank runs the same pass on its own
T spike vectors against its own replica of the matrix: the batch of spike vectors
is data-parallel, no collective is on the data path (weak scaling).

Reported beside the headline, in the same JSON line (none of them part of ``value``):
``cases`` — the microbenchmark grid (firing rates 0.1 / 1 / 10 %, homogeneous and
heterogeneous weights, both products) with the HBM fraction of each; ``single_vector_us``
— one spike vector per call, calls replayed back to back from a CUDA graph;
``training_step`` — the batched event matmul with its reverse mode (64 x 65 536 spikes at
2 %); ``network`` — the 10^6-neuron conductance-based network and ``network_large`` — the
8 * 10^6-neuron / 8 * 10^9-synapse network, both postsynaptic-sharded over the N ranks,
their per-step spike counts compared with the committed one-GPU record.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_NEURONS = 65536
PROB = 0.01
RATE = 0.01
SEED_CONN, SEED_W, SEED_SPK = 200, 201, 211


# ----------------------------------------------------------------------------
# workload
# ----------------------------------------------------------------------------

def build_workload(vectors, rank=0, rate=RATE, seed_spk=SEED_SPK, use_numpy=False):
    n = N_NEURONS
    K = int(n * PROB)
    if use_numpy:       # the reference arm must not touch the product: NumPy's own generator call
        idx = np.random.RandomState(SEED_CONN).randint(0, n, size=(n, K)).astype(np.int32)
    else:
        from brainstate_b200.nn import fixed_num_indices
        idx = fixed_num_indices(SEED_CONN, n, n, K)
    w = np.random.RandomState(SEED_W).normal(0.1, 0.01, (n, K)).astype(np.float32)
    spk = np.random.RandomState(seed_spk + 1000 * rank).random_sample((vectors, n)) < rate
    return n, K, idx, w, spk


def measured_hbm_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        try:
            return float(json.load(open(path))['hbm_gbs']), 'measured'
        except Exception:
            pass
    return 6650.0, 'fallback'


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.QUERY}', '--format=csv,noheader,nounits', '-lms', '100',
                 '-i', str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for ln in self.lines:
            f = [x.strip() for x in ln.split(',')]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        if not sm:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['no samples']}
        return {'sm_mhz': float(np.median(sm)), 'sm_max_mhz': float(max(smax)), 'reasons': sorted(reasons),
                'samples': len(sm)}


# ----------------------------------------------------------------------------
# CPU baseline (oracle port), bounded sample
# ----------------------------------------------------------------------------

class CpuPath:
    """The same hot path on the host cores (C/OpenMP restatement under oracle/): spike@W as
    a scatter over the active rows, W@spike either as the row gather the reference's CPU
    kernels do or as the event-driven scatter over a column-major copy (built once, like the
    device's transposed copy) — whichever is faster on this host."""

    def __init__(self, idx, w, probe):
        from oracle import c_oracle as co
        co.build()
        self.co = co
        self.cores = co.use_all_cores()
        self.idx, self.w = idx, w
        self.n = idx.shape[0]
        t_indptr, t_rows, t_perm = co.transpose(idx, self.n, self.n)
        self.t_indptr, self.t_rows = t_indptr, t_rows
        self.t_w = np.ascontiguousarray(w.reshape(-1)[t_perm])
        self.reverse = 'scatter over the column-major copy'
        t0 = time.perf_counter(); self.matvec(probe); a = time.perf_counter() - t0
        self.reverse = 'row gather'
        t0 = time.perf_counter(); self.matvec(probe); b = time.perf_counter() - t0
        if a < b:
            self.reverse = 'scatter over the column-major copy'

    def vecmat(self, spk):
        return self.co.event_vecmat_u8(spk, self.idx, self.w, self.n, split_rows=True)

    def matvec(self, spk):
        if self.reverse == 'row gather':
            return self.co.event_matvec_u8(spk, self.idx, self.w, self.n)
        return self.co.event_vecmat_u8(spk, self.t_rows, self.t_w, self.n, self.t_indptr, split_rows=True)

    def run(self, spk):
        self.vecmat(spk)
        self.matvec(spk)


def cpu_baseline(idx, w, spk, sample_s=12.0, sample_vectors=32):
    sample = np.ascontiguousarray(spk[:sample_vectors]).astype(np.uint8)
    cpu = CpuPath(idx, w, sample)
    K = idx.shape[1]
    events = 2 * int(sample.sum()) * K
    cpu.run(sample)                                    # warm-up (page-in, thread start)
    passes, t0 = 0, time.perf_counter()
    while True:
        cpu.run(sample)
        passes += 1
        el = time.perf_counter() - t0
        if el >= sample_s and passes >= 2:
            break
    return {'value': events * passes / el, 'unit': 'synaptic events/s', 'cores': cpu.cores, 'kind': 'port',
            'sample': f'{passes} passes over {sample.shape[0]} spike vectors (both products each), {el:.1f} s, '
                      f'C/OpenMP restatement of the reference CPU path, W@spike as {cpu.reverse}'}


def run_reference_arm(args):
    """``--impl reference``: the reference's CPU implementation of the path.  The
    reference's own kernels live in the un-vendored package brainevent, which is not
    installed and cannot be (no network), so the timed code is the C/OpenMP
    restatement under oracle/ (kind "port"), on all host threads, on the same
    workload: the same matrix (drawn here with NumPy, the reference's own call), the same
    ``--vectors`` spike vectors per step, both products."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return 0
    n, K, idx, w, spk = build_workload(args.vectors, use_numpy=True)
    sample = np.ascontiguousarray(spk).astype(np.uint8)
    cpu = CpuPath(idx, w, sample[:min(16, len(sample))])
    events = 2 * int(sample.sum()) * K
    for _ in range(max(min(args.warmup, 2), 1)):       # a pass takes about a second: two warm-up passes
        cpu.run(sample)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.run(sample)
    el = time.perf_counter() - t0
    value = events * args.steps / el
    unit = 'synaptic events/s'
    line = {
        'impl': 'reference', 'metric': 'synaptic events/s (event matvec microbenchmark, both products)',
        'value': value, 'unit': unit, 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': 1e3 * el / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'f32', 'data': 'synthetic',
        'config': workload_config(args.vectors, 'inputs larger than L2 (343 MB matrix vs 126 MB L2), no flush'),
        'cpu_baseline': {'value': value, 'unit': unit, 'cores': cpu.cores, 'kind': 'port',
                         'sample': f'the full step: {args.vectors} spike vectors, both products, W@spike as '
                                   f'{cpu.reverse}; brainevent (the reference\'s kernel package) is not '
                                   'installable here, so the C/OpenMP restatement is timed'},
        'e2e': {'value': value, 'unit': unit, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))
    return 0


def workload_config(vectors, l2_note):
    return {'workload': 'standalone event matvec microbenchmark: n_pre=n_post=65536, fixed-prob p=0.01 '
                        '(655 int32 targets/row), heterogeneous f32 weights N(0.1,0.01), Bernoulli 1% spikes, '
                        'products spike@W and W@spike',
            'vectors_per_step': vectors, 'firing_rate': RATE,
            'l2': l2_note, 'parallelism': 'spike vectors data-parallel, one matrix replica per GPU'}


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

class DevicePass:
    """Pre-allocated buffers and raw C-ABI calls for one pass of the hot path."""

    def __init__(self, torch, dev, n, K, idx, w, vectors):
        from brainstate_b200 import _lib, FixedPostNumConn
        self.torch, self._lib, self.lib = torch, _lib, _lib.lib()
        self.n, self.K, self.T = n, K, vectors
        self.ti = torch.from_numpy(idx).to(dev)
        self.tw = torch.from_numpy(w).to(dev)
        self.conn = FixedPostNumConn((self.tw, self.ti), shape=(n, n))
        self.st = self.conn._struct()
        self.y_vecmat = torch.empty((vectors, n), dtype=torch.float32, device=dev)
        self.y_matvec = torch.empty((vectors, n), dtype=torch.float32, device=dev)
        self.ws_bytes = self.lib.bsx_event_vecmat_workspace_bytes(vectors, n)
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.words = (n + 31) // 32
        self.bits = torch.empty((vectors, self.words), dtype=torch.int32, device=dev)   # used by --cases
        self.mv_ws_bytes = self.lib.bsx_event_matvec_workspace_bytes(vectors, n)
        self.mv_ws = torch.empty(self.mv_ws_bytes, dtype=torch.uint8, device=dev)
        self.passes = (vectors + 15) // 16
        # W@spike: below ~3 % firing the event-driven form (the active columns scatter along the
        # transposed copy) beats the gather over all rows; above it the gather wins
        self.matvec_method = 'scatter' if RATE <= 0.03 else 'gather'
        self.st_t = self.conn._transposed_struct(self.tw) if self.matvec_method == 'scatter' else None
        # which scatter kernel the library picks for this batch: output slices in shared memory
        # (one launch per product) or global atomics (compaction + scatter launch)
        self.scatter_variant = self.lib.bsx_event_vecmat_variant(C.byref(self.st), self._lib.SPK_BOOL8, vectors)
        self.sliced = self.scatter_variant == self._lib.VECMAT_SHARED_SLICES
        per_scatter = 1 if self.sliced else 2
        self.scale_s = self.scale_t = None
        if self.sliced:       # copies whose rows are grouped by output slice, built once like the matrix
            self.st_s = self.conn._sliced_struct(self.tw)
            self.scale_s = self.conn._fixed_scale('s', self.st_s, self.tw)       # fixed-point sums: order-free, faster
            # compressed form: 16-bit column offsets inside the slice, weights stored in fixed point
            self.loc_s, self.q_s = self.conn._packed('s', self.st_s, self.tw, self.scale_s)
            if self.matvec_method == 'scatter':
                self.st_t = self.conn._transposed_sliced_struct(self.tw)
                self.scale_t = self.conn._fixed_scale('ts', self.st_t, self.tw)
                self.loc_t, self.q_t = self.conn._packed('ts', self.st_t, self.tw, self.scale_t)
        # for the gather: transpose-pack + one pass per 16 vectors
        self.launches_per_pass = per_scatter + (per_scatter if self.matvec_method == 'scatter' else 1 + self.passes)

    def vecmat(self, spk_dev, stream):
        if self.sliced:
            self._lib.check(self.lib.bsx_event_vecmat_sliced16(C.byref(self.st_s), self.loc_s.data_ptr(),
                                                               self.q_s.data_ptr(), spk_dev.data_ptr(),
                                                               self._lib.SPK_BOOL8, self.T, self.y_vecmat.data_ptr(),
                                                               0, self.scale_s, stream))
            return
        self._lib.check(self.lib.bsx_event_vecmat(C.byref(self.st), spk_dev.data_ptr(), self._lib.SPK_BOOL8,
                                                  self.T, self.y_vecmat.data_ptr(), 0, self.ws.data_ptr(),
                                                  self.ws_bytes, stream))

    def matvec(self, spk_dev, stream):
        if self.matvec_method == 'scatter' and self.sliced:
            self._lib.check(self.lib.bsx_event_vecmat_sliced16(C.byref(self.st_t), self.loc_t.data_ptr(),
                                                               self.q_t.data_ptr(), spk_dev.data_ptr(),
                                                               self._lib.SPK_BOOL8, self.T, self.y_matvec.data_ptr(),
                                                               0, self.scale_t, stream))
        elif self.matvec_method == 'scatter':
            self._lib.check(self.lib.bsx_event_vecmat(C.byref(self.st_t), spk_dev.data_ptr(), self._lib.SPK_BOOL8,
                                                      self.T, self.y_matvec.data_ptr(), 0, self.ws.data_ptr(),
                                                      self.ws_bytes, stream))
        else:
            self.matvec_gather(spk_dev, stream)

    def matvec_gather(self, spk_dev, stream):
        self._lib.check(self.lib.bsx_event_matvec(C.byref(self.st), spk_dev.data_ptr(), self._lib.SPK_BOOL8,
                                                  self.T, self.y_matvec.data_ptr(), self.mv_ws.data_ptr(),
                                                  self.mv_ws_bytes, stream))

    def run(self, spk_dev, stream):
        self.vecmat(spk_dev, stream)
        self.matvec(spk_dev, stream)


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    if not torch.cuda.is_available():
        print(json.dumps({'error': 'no CUDA device: bench.py times the CUDA path only'}))
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        import datetime
        # a rank that fails must not keep the others waiting for the default ten minutes
        dist.init_process_group('nccl', device_id=dev, timeout=datetime.timedelta(seconds=420))

    from brainstate_b200 import _lib
    from brainstate_b200.nn import EventFixedProb
    T = args.vectors
    n, K, idx, w, spk = build_workload(T, rank)
    events_pass = 2 * int(spk.sum()) * K
    dp = DevicePass(torch, dev, n, K, idx, w, T)
    spk_dev = torch.from_numpy(spk).to(dev)
    stream = torch.cuda.current_stream().cuda_stream

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------
    # at least 3 warm-up steps, and enough of them for the SM clock to leave idle
    # nvidia-smi delivers a sample every 100 ms and the timed region may be a few milliseconds long, so
    # the sampler starts before the warm-up (the same kernels, back to back) and runs through the timed region
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_w, n_w = time.perf_counter(), 0
    while n_w < (args.warmup if args.profile else max(args.warmup, 3)) or (not args.profile and time.perf_counter() - t_w < 0.5):
        dp.run(spk_dev, stream)
        n_w += 1
        if n_w % 8 == 0:
            torch.cuda.synchronize()
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    mv = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    e_start.record()
    for s in range(args.steps):
        dp.vecmat(spk_dev, stream)
        mv[s][0].record()
        dp.matvec(spk_dev, stream)
        mv[s][1].record()
    e_end.record()
    barrier()
    ms_total = e_start.elapsed_time(e_end)
    ms_matvec = sum(a.elapsed_time(b) for a, b in mv)
    # the deterministic gather, timed on its own for the roofline of W@spike as an HBM stream
    # (it is the step's W@spike only when the firing rate selects it)
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g_steps = 0 if args.profile else max(3, min(args.steps, 10))
    g0.record()
    for _ in range(g_steps):
        dp.matvec_gather(spk_dev, stream)
    g1.record()
    torch.cuda.synchronize()
    ms_gather = g0.elapsed_time(g1) / max(g_steps, 1)
    clocks = sampler.stop() if rank == 0 else None
    if dp.matvec_method == 'scatter' and rank == 0 and not args.profile:   # the two forms of W@spike agree
        y_gather = dp.y_matvec.clone()
        dp.matvec(spk_dev, stream)
        torch.cuda.synchronize()
        assert torch.allclose(dp.y_matvec, y_gather, rtol=1e-5, atol=1e-6)
    t_dev = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_dev, op=dist.ReduceOp.MAX)
    ms_total_max = float(t_dev.item())
    ev_all = torch.tensor([float(events_pass)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ev_all, op=dist.ReduceOp.SUM)
    events_all = float(ev_all.item())
    value = events_all * args.steps / (ms_total_max * 1e-3)

    if args.only:             # one leg, for the profiler
        peak, _ = measured_hbm_peak()
        if args.only == 'training':
            out = run_training_step(torch, dev, dp, peak)
        elif args.only == 'single':
            out = run_single_vector(torch, dev, dp, peak, calls=8)
        else:
            out = [c for c in run_cases(torch, dev, dp, peak, rates=(0.01,)) if c['weights'] == 'homogeneous']
        if rank == 0:
            print(json.dumps({'only': args.only, 'result': out}))
        if world > 1:
            dist.destroy_process_group()
        return 0

    if args.profile:          # device loop only: what the profiler captures
        if rank == 0:
            print(json.dumps({'profile_run': True, 'value': value, 'ms_per_step': ms_total_max / args.steps}))
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- end to end through the layer API, host buffers ---------------------------
    layer = EventFixedProb(n, n, PROB, dp.tw, seed=SEED_CONN)
    assert torch.equal(layer.conn.indices, dp.ti)
    host_spk = torch.from_numpy(spk).pin_memory()
    host_y1 = torch.empty((T, n), dtype=torch.float32).pin_memory()
    host_y2 = torch.empty((T, n), dtype=torch.float32).pin_memory()

    from brainstate_b200.host import HostEventProducts
    # public host-buffer API: upload, products, download overlap
    pipe = HostEventProducts(layer.conn, chunk=64, reverse_method=dp.matvec_method)

    def e2e_pass():
        pipe(host_spk, host_y1, host_y2)               # spike @ W and W @ spike, host memory in and out
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        e2e_pass()
    if rank == 0:      # the host-buffer path returns what the device-resident path computes
        dp.run(spk_dev, stream)
        torch.cuda.synchronize()
        assert torch.allclose(host_y1.to(dev), dp.y_vecmat, rtol=1e-5, atol=1e-6)
        assert torch.allclose(host_y2.to(dev), dp.y_matvec, rtol=1e-5, atol=1e-6)
    barrier()
    e2e_steps = max(3, min(args.steps, 8))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_pass()
    barrier()
    e2e_s = time.perf_counter() - t0
    t_e2e = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    e2e_value = events_all * e2e_steps / float(t_e2e.item())

    peak, peak_kind = measured_hbm_peak()
    facts = {'passes': dp.passes, 'matvec_method': dp.matvec_method, 'scatter_variant': dp.scatter_variant,
             'launches_per_pass': dp.launches_per_pass}
    cases = single = training = None
    if rank == 0 and not args.no_cases:
        cases = run_cases(torch, dev, dp, peak)
        single = run_single_vector(torch, dev, dp, peak)
        training = run_training_step(torch, dev, dp, peak)
    # the network legs build their own connectivity: release the microbenchmark's buffers first
    idx_host, w_host = idx, w
    del dp, pipe, layer, spk_dev, host_spk, host_y1, host_y2
    torch.cuda.empty_cache()
    network = network_large = None
    if not args.no_network:
        network = run_network(torch, dist, dev, world, rank, 'coba', steps=1000, warm=200)
        if not args.no_large:
            network_large = run_network(torch, dist, dev, world, rank, 'large', steps=500, warm=0)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---- roofline of the two kernels of a step; the dominant one is reported first --
    nnz = n * K
    events_vec = float(spk.sum()) * K                      # events of one product over the batch
    # gather: one launch = one pass over the indices for 16 vectors
    g_bytes = nnz * 4 + (events_vec / facts['passes']) * 4 + n * 2 + min(T, 16) * 4 * n
    g_launch_s = (ms_gather * 1e-3) / facts['passes']                  # includes the transpose-pack launch (~2 %)
    # scatter: one launch = all T vectors of one product
    s_bytes = events_vec * 8 + T * (n + 4 * n)
    if facts['matvec_method'] == 'scatter':
        s_launches, ms_scatter = 2 * args.steps, ms_total
    else:
        s_launches, ms_scatter = args.steps, ms_total - ms_matvec
    s_launch_s = (ms_scatter * 1e-3) / s_launches

    def roof(kernel, nbytes, sec, share, note):
        a = nbytes / sec / 1e9
        return {'bound': 'hbm', 'kernel': kernel, 'achieved': a, 'peak': peak, 'peak_kind': peak_kind,
                'unit': 'GB/s', 'frac': a / peak, 'bytes_per_launch': nbytes, 'avg_launch_us': sec * 1e6,
                'share_of_step': share, 'traffic': None, 'frac_dram': None, 'note': note}

    smem_variant = facts['scatter_variant'] == _lib.VECMAT_SHARED_SLICES
    what = 'spike@W over the rows' + (' and W@spike over the transposed copy' if facts['matvec_method'] == 'scatter' else '')
    if smem_variant:
        r_s = roof('scatter_smem_kernel<hetero, fixed-point, 16-bit offsets>', s_bytes, s_launch_s, ms_scatter / ms_total,
                   what + '; one block per (spike vector, 32768-column slice of the output held in shared memory) '
                   'over the copy whose rows are grouped by slice, columns stored as 16-bit offsets inside the slice '
                   'and weights as 2^-s fixed point (6 bytes per synapse read; the algorithmic bytes count 8), summed '
                   'with native shared-memory integer atomics (order-free: deterministic); algorithmic bytes can '
                   'exceed the DRAM traffic also because rows shared between vectors are served by L2')
    else:
        r_s = roof('scatter_queue_kernel<hetero> (+compact)', s_bytes, s_launch_s, ms_scatter / ms_total,
                   what + '; limited by the L2 rate of red.global.add.f32 (about 190 G adds/s in a stand-alone '
                   'probe), not by HBM')
    r_s['atomic_adds_per_s'] = events_vec / s_launch_s
    if facts['matvec_method'] == 'scatter':
        r_g = roof('event_matvec_b16_kernel<hetero>', g_bytes, g_launch_s, 0.0,
                   'the deterministic W@spike (16 vectors per pass over the indices), timed in its own loop after '
                   'the steps: at this firing rate the step uses the event-driven form, which is '
                   f'{ms_gather / (ms_matvec / args.steps):.2f}x faster; limited by shared-memory bit tests and '
                   'instruction issue')
        roofline, roofline_2 = r_s, r_g
    else:
        r_g = roof('event_matvec_b16_kernel<hetero>', g_bytes, g_launch_s, ms_matvec / ms_total,
                   'W@spike, 16 vectors per pass over the indices; limited by shared-memory bit tests and '
                   'instruction issue')
        roofline, roofline_2 = (r_g, r_s) if ms_matvec >= ms_scatter else (r_s, r_g)
    prof = os.path.join(ROOT, 'profiles', 'traffic.json')
    if os.path.exists(prof):
        try:
            tr = json.load(open(prof))
            r_g['traffic'] = float(tr['event_matvec_b16_kernel'])                      # captured at this launch size
            if smem_variant:
                # L2 serves rows that several vectors share, so DRAM traffic does not grow in proportion
                # to the vectors: the capture is of this launch size and is used for no other
                r_s['traffic'] = float(tr['scatter_smem_kernel_packed_296_vectors']) if T == 296 and 'scatter_smem_kernel_packed_296_vectors' in tr else None
            else:
                r_s['traffic'] = float(tr['scatter_queue_kernel_per_16_vectors']) * T / 16  # grows with the events
        except Exception:
            pass
    for r in (r_s, r_g):      # what actually crossed the HBM interface (ncu), as a fraction of the peak
        if r['traffic']:
            r['frac_dram'] = r['traffic'] / (r['avg_launch_us'] * 1e-6) / 1e9 / peak

    cpu = cpu_baseline(idx_host, w_host, spk)

    line = {
        'metric': 'synaptic events/s (event matvec microbenchmark, both products)',
        'value': value, 'unit': 'synaptic events/s', 'n_gpus': world, 'steps': args.steps, 'warmup': max(args.warmup, 3),
        'ms_per_step': ms_total_max / args.steps, 'higher_is_better': True, 'scaling': 'weak',
        'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': workload_config(T, 'inputs larger than L2 (343 MB matrix vs 126 MB L2), no flush'),
        'clocks': clocks,
        'e2e': {'value': e2e_value, 'unit': 'synaptic events/s', 'h2d_bytes_per_step': int(spk.nbytes),
                'd2h_bytes_per_step': int(2 * T * n * 4), 'steps': e2e_steps},
        'gpu_launches': int(facts['launches_per_pass'] * args.steps),
        'roofline': roofline,
        'roofline_other_kernel': roofline_2,
        'cpu_baseline': cpu,
        'events_per_step': events_all,
        'variants': {'spike@W': 'scatter', 'scatter_kernel': 'shared-memory slices, fixed-point sums' if smem_variant else 'global atomics', 'W@spike': facts['matvec_method'] + (' over the transposed copy' if facts['matvec_method'] == 'scatter' else ''),
                     'chosen_for_rate': RATE},
        'cases': cases,
        'single_vector_us': single,
        'training_step': training,
        'network': network,
        'network_large': network_large,
    }
    records = {}
    for leg in (network, network_large):
        if leg:
            records.update(leg.pop('_records'))
    if args.write_fixtures and world == 1 and records:
        os.makedirs(os.path.dirname(os.path.abspath(args.write_fixtures)), exist_ok=True)
        np.savez_compressed(args.write_fixtures, **{k: v.astype(np.int32) for k, v in records.items()})
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


FIXTURE = os.path.join(ROOT, 'tests', 'golden', 'network_counts.npz')


def run_network(torch, dist, dev, world, rank, name, steps, warm):
    """One of the network recipes (``brainstate_b200.sim.preset``), postsynaptic-sharded over
    the ranks: all steps in one cooperative launch per GPU with the spike exchange inside the
    kernel.  Timed with CUDA events, maximum over ranks.  The per-step spike counts are
    compared with the committed record of the one-GPU run (``tests/golden/network_counts.npz``,
    written by ``--write-fixtures FILE``).  The large recipe has heterogeneous weights: it is timed
    with float32 sums and run once more with fixed-point sums, whose counts do not depend on
    the order of the adds and so must equal the record at any number of GPUs."""
    from brainstate_b200.sim import from_preset, preset
    p = preset(name)
    n = p['n_exc'] + p['n_inh']
    K = p['conn_num']
    group = dist.group.WORLD if world > 1 else None
    hetero = not isinstance(p['w_e'], float)
    t0 = time.perf_counter()
    net = from_preset(name, dev, group, shard_kernel=True)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0

    def timed(net):
        net.prepare()                           # inboxes and peer mappings: set-up, not part of a step
        pre = net.run(warm, record=False)[1] if warm else None
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _, counts = net.run(steps, record=False)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        all_counts = counts if pre is None else torch.cat([pre, counts])
        return float(t.item()), counts, all_counts.cpu().numpy()

    net.run(50, record=False)                  # module load, clocks; then start again from the seeded state
    fresh = from_preset(name, dev, group, shard_kernel=True, conn=(net.conn_e, net.conn_i))
    ms, counts, record = timed(fresh)
    fresh.close()
    spikes = int(counts.sum().item())
    out = {'workload': {'coba': 'COBA E/I LIF network, 1e6 neurons (800k E / 200k I), 100 targets per neuron, g_exc 0.6, '
                                'g_inh 6.7, E_exc 0 mV, E_inh -80 mV, constant bias tuned to ~10 Hz, dt 0.1 ms',
                        'large': 'LIF network, 8e6 neurons (80% E / 20% I), 1000 targets per neuron (8e9 synapses, int32), '
                                 'lognormal(-2, 0.5) f32 weights signed by population, hashed background drive (~5 Hz), '
                                 'dt 0.1 ms'}[name] + '; postsynaptic neurons sharded over the GPUs',
           'steps': steps, 'warmup_steps': warm, 'us_per_step': ms * 1e3 / steps, 'spikes': spikes,
           'mean_rate_hz': spikes / n / (steps * 1e-4), 'synaptic_events_per_s': spikes * K / (ms * 1e-3),
           'build_s': build_s, 'launches': 1,
           'kernel': 'net_run_sharded_kernel (state in shared memory)' if net._links['links'].words_per_block <= 432
                     else 'net_run_sharded_kernel (state in global memory)',
           'exchange': 'spike-id lists pushed by peer stores inside the step kernel' if world > 1 else 'none (one GPU)',
           'accumulation': 'float32 atomics'}
    # algorithmic bytes of the whole network per step: neuron state (4 words read + 4 written per
    # neuron), the packed spike words, 4 (+4 with per-synapse weights) bytes per synaptic event;
    # against the HBM peak of the N GPUs together (state kept in shared memory moves none of these
    # bytes through HBM: the figure says how the step compares with a kernel that streams its state)
    alg = n * 32 + n / 8 + (spikes / steps) * K * (8 if hetero else 4)
    peak_gbs, _ = measured_hbm_peak()
    out['algorithmic_bytes_per_step'] = alg
    out['algorithmic_GBps'] = alg / (ms * 1e-3 / steps) / 1e9
    out['frac_of_hbm_peak_all_gpus'] = out['algorithmic_GBps'] / (peak_gbs * world)
    if world > 1 and not hetero:
        # the plain-library form of the same step, for comparison: split-phase launches and one NCCL
        # all-gather of the packed spike words per step (launch-bound; 200 steps)
        def time_nccl(overlap, graph_steps):
            lib_net = from_preset(name, dev, group, exchange='nccl', overlap=overlap, conn=(net.conn_e, net.conn_i))
            lib_net.run(100, record=False, graph_steps=graph_steps)       # warm-up; captures the graph
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            lib_net.run(200, record=False, graph_steps=graph_steps)
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            lib_net.close()
            return float(t.item()) * 1e3 / 200

        # (a comparison beside the measurement: a failure here is recorded, it does not end the run)
        for key, overlap, graph_steps in (('nccl_all_gather_us_per_step', False, 0),             # eager: bound by the host's launches
                                          ('nccl_graph_replay_us_per_step', False, 50),          # 50 captured steps per replay
                                          ('nccl_graph_replay_overlapped_us_per_step', True, 50)):  # own-spike scatter during the all-gather
            try:
                out[key] = time_nccl(overlap, graph_steps)
            except Exception as exc:        # noqa: BLE001
                out[key] = None
                out.setdefault('nccl_errors', []).append(f'{key}: {type(exc).__name__}: {exc}'[:200])
    fixture = dict(np.load(FIXTURE)) if os.path.exists(FIXTURE) else {}
    written = {}
    if hetero:
        det = from_preset(name, dev, group, deterministic=True, conn=(net.conn_e, net.conn_i))
        ms_d, counts_d, record_d = timed(det)
        out['deterministic'] = {'us_per_step': ms_d * 1e3 / steps, 'spikes': int(counts_d.sum().item()),
                                'accumulation': '2^-32 fixed point, 64-bit integer atomics'}
        written[name + '_deterministic'] = record_d
        if name + '_deterministic' in fixture:
            out['matches_n1'] = bool(np.array_equal(fixture[name + '_deterministic'], record_d))
        else:
            out['matches_n1'] = None
        if name in fixture:        # float sums: equal only as long as no sum met a different rounding
            same = fixture[name] == record
            out['float_counts_equal_n1_for_steps'] = int(len(same) if same.all() else np.argmin(same))
        det.close()
    else:
        out['matches_n1'] = bool(np.array_equal(fixture[name], record)) if name in fixture else None
    written[name] = record
    out['_records'] = written
    net.close()
    return out


def _time(torch, fn, reps=5, warm=3):
    for _ in range(warm):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e-3 / reps


def run_cases(torch, dev, dp, peak, rates=(0.001, 0.01, 0.1)):
    """The microbenchmark grid: firing rates 0.1 / 1 / 10 %, homogeneous (0.1) and
    heterogeneous weights, both products — ``spike@W`` as the batched scatter, ``W@spike``
    both event-driven (scatter over the transposed copy) and as the deterministic gather
    (16 vectors per pass) — each timed on its own with CUDA events after warm-up.
    ``frac`` = algorithmic bytes / time / measured HBM peak."""
    from brainstate_b200 import _lib, FixedPostNumConn
    lib = _lib.lib()
    n, K, T = dp.n, dp.K, dp.T
    stream = torch.cuda.current_stream().cuda_stream
    homo = FixedPostNumConn((0.1, dp.ti), shape=(n, n))
    homo._derived = dp.conn._derived           # same connectivity: share the derived layouts
    out = []
    for rate in rates:
        r_id = (0.001, 0.01, 0.1).index(rate)
        spk = np.random.RandomState(210 + r_id).random_sample((T, n)) < rate
        sd = torch.from_numpy(spk).to(dev)
        events = float(spk.sum()) * K
        for name, conn in (('homogeneous', homo), ('heterogeneous', dp.conn)):
            st = conn._struct()
            h = int(conn.hetero)
            st_s, st_ts = conn._sliced_struct(conn.data), conn._transposed_sliced_struct(conn.data)

            def vecmat_sliced():
                _lib.check(lib.bsx_event_vecmat_sliced(C.byref(st_s), sd.data_ptr(), _lib.SPK_BOOL8, T,
                                                       dp.y_vecmat.data_ptr(), 0, stream))

            def matvec_sliced():
                _lib.check(lib.bsx_event_vecmat_sliced(C.byref(st_ts), sd.data_ptr(), _lib.SPK_BOOL8, T,
                                                       dp.y_matvec.data_ptr(), 0, stream))

            def matvec_b16():
                _lib.check(lib.bsx_event_matvec(C.byref(st), sd.data_ptr(), _lib.SPK_BOOL8, T, dp.y_matvec.data_ptr(),
                                                dp.mv_ws.data_ptr(), dp.mv_ws_bytes, stream))

            scale_s, scale_ts = conn._fixed_scale('s', st_s, conn.data), conn._fixed_scale('ts', st_ts, conn.data)

            def vecmat_fixed():
                _lib.check(lib.bsx_event_vecmat_sliced_fixed(C.byref(st_s), sd.data_ptr(), _lib.SPK_BOOL8, T,
                                                             dp.y_vecmat.data_ptr(), 0, scale_s, stream))

            def matvec_fixed():
                _lib.check(lib.bsx_event_vecmat_sliced_fixed(C.byref(st_ts), sd.data_ptr(), _lib.SPK_BOOL8, T,
                                                             dp.y_matvec.data_ptr(), 0, scale_ts, stream))

            loc_s, q_s = conn._packed('s', st_s, conn.data, scale_s)
            loc_ts, q_ts = conn._packed('ts', st_ts, conn.data, scale_ts)

            def vecmat_packed():
                _lib.check(lib.bsx_event_vecmat_sliced16(C.byref(st_s), loc_s.data_ptr(), _lib.ptr(q_s), sd.data_ptr(),
                                                         _lib.SPK_BOOL8, T, dp.y_vecmat.data_ptr(), 0, scale_s, stream))

            def matvec_packed():
                _lib.check(lib.bsx_event_vecmat_sliced16(C.byref(st_ts), loc_ts.data_ptr(), _lib.ptr(q_ts),
                                                         sd.data_ptr(), _lib.SPK_BOOL8, T, dp.y_matvec.data_ptr(), 0,
                                                         scale_ts, stream))

            scatter_bytes = events * (4 + 4 * h) + T * (n + 4 * n)
            packed = (('spike@W, scatter over 16-bit offsets' + (' and fixed-point weights (deterministic)' if h else ''),
                       vecmat_packed, scatter_bytes),
                      ('W@spike, scatter over 16-bit offsets of the transposed copy' + (' (deterministic)' if h else ''),
                       matvec_packed, scatter_bytes))
            fixed = (('spike@W, fixed-point scatter (deterministic)', vecmat_fixed, scatter_bytes),
                     ('W@spike, fixed-point scatter over the transposed copy (deterministic)', matvec_fixed,
                      scatter_bytes)) if h else ()
            for prod, fn, alg in packed + fixed + (('spike@W, scatter (output slices in shared memory)', vecmat_sliced, scatter_bytes),
                                  ('W@spike, event-driven scatter over the transposed copy', matvec_sliced, scatter_bytes),
                                  ('W@spike, deterministic gather (16 vectors per pass)', matvec_b16,
                                   dp.passes * (n * K * 4 + 2 * n) + T * 4 * n + events * 4 * h)):
                sec = _time(torch, fn)
                out.append({'rate': rate, 'weights': name, 'product': prod, 'vectors': T,
                            'events_per_s': events / sec, 'us_per_vector': sec / T * 1e6,
                            'algorithmic_GBps': alg / sec / 1e9, 'frac': alg / sec / 1e9 / peak})
    return out


def run_single_vector(torch, dev, dp, peak, calls=64):
    """One spike vector per call — what ``EventFixedProb.update(spk)`` sees inside a
    simulation loop: ``calls`` back-to-back ``bsx_event_vecmat`` calls on distinct spike
    vectors, captured in a CUDA graph and replayed; microseconds per call."""
    from brainstate_b200 import _lib, FixedPostNumConn
    lib = _lib.lib()
    n, K = dp.n, dp.K
    homo = FixedPostNumConn((0.1, dp.ti), shape=(n, n))
    ws_bytes = lib.bsx_event_vecmat_workspace_bytes(1, n)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    y = torch.empty((calls + 1, n), dtype=torch.float32, device=dev)
    out = []

    def replayed(burst):
        burst()
        torch.cuda.synchronize()
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                burst()
        torch.cuda.current_stream().wait_stream(side)
        sec = _time(torch, g.replay, reps=10) / calls
        del g
        return sec

    for r_id, rate in enumerate((0.001, 0.01, 0.1)):
        spk = np.random.RandomState(230 + r_id).random_sample((calls, n)) < rate
        sd = torch.from_numpy(spk).to(dev)
        events = float(spk.sum()) * K / calls
        for name, conn in (('homogeneous', homo), ('heterogeneous', dp.conn)):
            st = conn._struct()
            h = int(conn.hetero)

            def burst():
                stream = torch.cuda.current_stream().cuda_stream
                for c in range(calls):
                    _lib.check(lib.bsx_event_vecmat(C.byref(st), sd.data_ptr() + c * n, _lib.SPK_BOOL8, 1,
                                                    y.data_ptr() + 4 * c * n, 0, ws.data_ptr(), ws_bytes, stream))

            def chained():
                # one launch per call: every call adds into its own output row and clears the next call's
                # (row 0 is cleared by the last call of the previous replay: the chain closes on itself)
                stream = torch.cuda.current_stream().cuda_stream
                for c in range(calls):
                    nxt = (c + 1) % calls
                    _lib.check(lib.bsx_event_vecmat_chained(C.byref(st), sd.data_ptr() + c * n, _lib.SPK_BOOL8, 1,
                                                            y.data_ptr() + 4 * c * n, y.data_ptr() + 4 * nxt * n, stream))

            sec = replayed(burst)
            ref_rows = y[:calls].clone()
            y[0].zero_()
            sec_chained = replayed(chained)
            if h == 0:      # identical addends: the chained calls give the same bits as the plain ones
                g_check = y[1:calls]                       # row 0 was cleared again by the last call of the chain
                assert torch.equal(g_check, ref_rows[1:calls]), 'chained single-vector calls differ from the plain calls'
            alg = events * (4 + 4 * h) + n + 4 * n
            out.append({'rate': rate, 'weights': name, 'us_per_call': sec * 1e6, 'events_per_s': events / sec,
                        'algorithmic_GBps': alg / sec / 1e9, 'frac': alg / sec / 1e9 / peak,
                        'launches_per_call': int(lib.bsx_event_vecmat_launches(C.byref(st), _lib.SPK_BOOL8, 1)),
                        'us_per_call_chained': sec_chained * 1e6, 'frac_chained': alg / sec_chained / 1e9 / peak})
    return out


def run_training_step(torch, dev, dp, peak):
    """The batched event matmul with its reverse mode: 64 x 65 536 spikes at 2 %, the
    heterogeneous matrix, cotangent N(0, 1).  Forward, input cotangent, weight cotangent and
    the whole step, with the algorithmic bytes of each (reverse mode reads every index and
    weight once and writes one float per synapse)."""
    from brainstate_b200 import _lib
    lib = _lib.lib()
    n, K, B = dp.n, dp.K, 64
    nnz = n * K
    spk = np.random.RandomState(220).random_sample((B, n)) < 0.02
    ct = np.random.RandomState(221).standard_normal((B, n)).astype(np.float32)
    sd, ctd = torch.from_numpy(spk).to(dev), torch.from_numpy(ct).to(dev)
    events = float(spk.sum()) * K
    y = torch.empty((B, n), dtype=torch.float32, device=dev)
    dx = torch.empty((B, n), dtype=torch.float32, device=dev)
    dw = torch.empty((n, K), dtype=torch.float32, device=dev)
    st, st_s = dp.conn._struct(), dp.conn._sliced_struct(dp.conn.data)
    ws_bytes = lib.bsx_vecmat_vjp_batched_workspace_bytes(B, n)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream

    def fwd():
        _lib.check(lib.bsx_event_vecmat_sliced(C.byref(st_s), sd.data_ptr(), _lib.SPK_BOOL8, B, y.data_ptr(), 0, stream))

    def bwd(want_dx, want_dw):
        _lib.check(lib.bsx_vecmat_vjp_batched(C.byref(st), sd.data_ptr(), _lib.SPK_BOOL8, 1, ctd.data_ptr(), B,
                                              dx.data_ptr() if want_dx else None, dw.data_ptr() if want_dw else None,
                                              ws.data_ptr(), ws_bytes, stream))

    def step():
        fwd()
        bwd(True, True)

    t_f, t_dx, t_dw = _time(torch, fwd), _time(torch, lambda: bwd(True, False)), _time(torch, lambda: bwd(False, True))
    t_b, t_s = _time(torch, lambda: bwd(True, True)), _time(torch, step)
    b_fwd = events * 8 + B * (n + 4 * n)
    b_dx = nnz * 8 + 2 * B * n * 4
    b_dw = nnz * 4 + nnz * 4 + B * n * 4 + B * n
    b_bwd = nnz * 8 + nnz * 4 + 2 * B * n * 4
    leg = lambda t, nb: {'us': t * 1e6, 'algorithmic_bytes': nb, 'algorithmic_GBps': nb / t / 1e9, 'frac': nb / t / 1e9 / peak}
    return {'workload': '64 x 65536 Bernoulli(2 %) spikes, heterogeneous 65536 x 655 matrix, cotangent N(0,1)',
            'forward': leg(t_f, b_fwd), 'dx': leg(t_dx, b_dx), 'dw': leg(t_dw, b_dw), 'backward': leg(t_b, b_bwd),
            'step_us': t_s * 1e6, 'events_per_s_forward': events / t_f,
            'l2_gathered_bytes_dx': nnz * B * 4,
            'kernels': {'forward': 'scatter_smem_kernel', 'dx': 'vjp_dx_batched_kernel', 'dw': 'vjp_dw_batched_kernel'},
            'note': 'dx gathers 64 cotangent values per synapse from L2 (nnz x 64 x 4 B = 11 GB): its bound is the L2 '
                    'gather rate, not HBM'}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--vectors', type=int, default=296,
                    help='spike vectors per step (per GPU); 296 vectors x 2 output slices = 4 blocks on each of the 148 SMs')
    ap.add_argument('--no-cases', action='store_true', help='skip the rate x weight x product grid, the single-vector '
                    'calls and the training step')
    ap.add_argument('--no-network', action='store_true', help='skip the sharded network runs reported beside the headline')
    ap.add_argument('--no-large', action='store_true', help='skip the 8e6-neuron network')
    ap.add_argument('--write-fixtures', default=None, metavar='FILE.npz',
                    help='one GPU: write the per-step spike counts of the network runs to this file (the record '
                         'committed as tests/golden/network_counts.npz was made this way)')
    ap.add_argument('--profile', action='store_true',
                    help='run only the device-resident loop (for ncu); prints no bench line')
    ap.add_argument('--only', default=None, choices=['training', 'single', 'homogeneous'],
                    help='for ncu: build the workload, run that one leg (training step; single-vector calls; the '
                         'batched scatter with homogeneous weights) and exit')
    args = ap.parse_args()
    if args.only:
        args.profile = True           # no long warm-up, no gather loop: only what the profiler should see
    if args.impl == 'reference':
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == '__main__':
    sys.exit(main())
