"""Runs an E/I spiking network on one or more GPUs and prints one JSON line.

    python -m brainstate_b200.run_network --preset large --steps 500
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m brainstate_b200.run_network --preset large --steps 500 --exchange p2p

Presets
  cuba   4 000 LIF neurons, p = 0.02, homogeneous weights +1.62 / -9 (current-based)
  coba   1 000 000 conductance-based LIF neurons, 100 targets per neuron, 0.6 / 6.7, constant bias
         tuned to about 10 Hz
  large  8 000 000 LIF neurons, 1000 targets per neuron (8e9 synapses), lognormal(-2, 0.5)
         weights signed by population (inhibition x6), hashed background drive
``--neurons`` / ``--targets`` override the preset's size.  With several ranks the
postsynaptic neurons are sharded; every rank draws the one seeded index stream and
keeps its columns.  Times are CUDA-event times, the maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--preset', default='coba', choices=['cuba', 'coba', 'large'])
    ap.add_argument('--neurons', type=int, default=0)
    ap.add_argument('--targets', type=int, default=0)
    ap.add_argument('--steps', type=int, default=1000)
    ap.add_argument('--warmup', type=int, default=100)
    ap.add_argument('--exchange', default='p2p', choices=['p2p', 'nccl'])
    ap.add_argument('--shard-kernel', action='store_true',
                    help='one GPU: run the kernel the sharded runs use (increment rows, one barrier per step)')
    ap.add_argument('--deterministic', action='store_true', help='fixed-point synaptic sums: order-free rasters')
    ap.add_argument('--degree', default='out', choices=['out', 'in'],
                    help="'in': every neuron draws its presynaptic partners (fixed in-degree) instead of its targets")
    ap.add_argument('--record', action='store_true', help='keep the bit-packed raster (memory: steps * n / 8 bytes)')
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from brainstate_b200.sim import EINet, preset

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local_rank)
    dev = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)

    p = preset(args.preset)
    params = p['params']
    n = args.neurons or (p['n_exc'] + p['n_inh'])
    K = args.targets or p['conn_num']
    n_exc = n * 4 // 5
    n_inh = n - n_exc
    V0 = np.random.RandomState(p['seed_v']).uniform(p['v0'][0], p['v0'][1], n).astype(np.float32)

    t0 = time.perf_counter()
    net = EINet(n_exc, n_inh, K, p['w_e'], p['w_i'], seed_e=p['seed_e'], seed_i=p['seed_i'], V0=V0, params=params,
                device=dev, group=dist.group.WORLD if world > 1 else None, exchange=args.exchange,
                deterministic=args.deterministic, shard_kernel=True if args.shard_kernel else None,
                degree=args.degree)
    torch.cuda.synchronize()
    build_s = time.perf_counter() - t0
    mem_gb = torch.cuda.max_memory_allocated(dev) / 1e9

    net.run(args.warmup, record=False)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    raster, counts = net.run(args.steps, record=args.record)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    spikes = int(counts.sum().item())
    out = {'preset': args.preset, 'n_gpus': world, 'neurons': n, 'targets_per_neuron': K, 'degree': args.degree,
           'synapses': n * K,
           'steps': args.steps, 'warmup': args.warmup, 'exchange': args.exchange if world > 1 else 'none',
           'build_s': build_s, 'device_memory_gb_rank0': mem_gb, 'ms_total': ms,
           'us_per_step': ms * 1e3 / args.steps, 'spikes': spikes,
           'mean_rate_hz': spikes / n / (args.steps * params.dt * 1e-3),
           'synaptic_events_per_s': spikes * K / (ms * 1e-3)}
    if args.record and raster is not None and rank == 0:       # per-population rates need the raster
        from brainstate_b200.sim import population_rates
        out['rate_exc_hz'], out['rate_inh_hz'] = population_rates(raster, n_exc, n_inh, params.dt)
    net.close()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == '__main__':
    sys.exit(main())
