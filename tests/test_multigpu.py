"""GPU (2 or more devices): the postsynaptic-sharded network, one rank per GPU,
reproduces the single-GPU raster bit for bit.  Skipped on a one-GPU box.

Every case runs its ranks as child processes on separate GPUs (never two ranks on one
GPU: their kernels wait for one another), with NVLS off, and leaves between steps only.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _init(rank, world, port):
    import torch.distributed as dist
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=dev)
    return dev, dist


def _small_net(dev, group, coba, exchange='p2p', delay_e=1, delay_i=0, **kw):
    from brainstate_b200.sim import EINet, LIFParams
    n_exc, n_inh, K = 3200, 800, 80
    V0 = np.random.RandomState(102).uniform(-60, -50, n_exc + n_inh).astype(np.float32)
    w_e, w_i, R = (0.6, 6.7, 0.1) if coba else (1.62, -9.0, 1.0)
    return EINet(n_exc, n_inh, K, w_e, w_i, seed_e=100, seed_i=101, V0=V0, params=LIFParams(coba=coba, R=R),
                 device=dev, group=group, exchange=exchange, delay_e=delay_e, delay_i=delay_i, **kw)


def _variant(exchange):
    """Constructor keywords of the test variants named after the exchange."""
    return {'nccl-overlap': {'overlap': True}, 'p2p-indegree': {'degree': 'in'}}.get(exchange, {})


def _rank_main(rank, world, port, steps, coba, exchange, delays, slack, out_dir):
    dev, dist = _init(rank, world, port)
    try:
        net = _small_net(dev, dist.group.WORLD, coba, exchange.split('-')[0], delays[0], delays[1], slack=slack,
                         **_variant(exchange))
        r1, c1 = net.run(steps // 2)
        r2, c2 = net.run(steps - steps // 2)
        raster, counts = torch.cat([r1, r2]), torch.cat([c1, c2])
        torch.cuda.synchronize()
        if rank == 0:
            torch.save({'raster': raster.cpu(), 'counts': counts.cpu(), 'spikes': net.spikes()},
                       os.path.join(out_dir, 'sharded.pt'))
        dist.barrier()
        net.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('exchange,delays,slack', [('nccl', (1, 0), None), ('nccl-overlap', (1, 0), None), ('nccl-overlap', (0, 0), None),
                                                   ('nccl-overlap', (3, 2), None), ('p2p', (1, 0), None), ('p2p', (0, 0), None),
                                                   ('p2p', (3, 2), None), ('p2p', (3, 2), 0), ('p2p', (3, 2), 1),
                                                   ('p2p-indegree', (1, 0), None)])
@pytest.mark.parametrize('coba', [False, True])
def test_sharded_network_equals_single_gpu(coba, exchange, delays, slack, tmp_path):
    """In-kernel exchange with and without slack (spikes consumed `slack` steps after they
    were pushed; default = the smaller delay), and the NCCL all-gather path with the own-spike
    scatter strictly in sequence with the all-gather, or overlapping it ('nccl-overlap'); 'p2p-indegree':
    every neuron draws its presynaptic partners, each rank its own rows of the one seeded stream."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs at least two GPUs')
    import torch.multiprocessing as mp
    world = 2 if torch.cuda.device_count() < 4 else 4
    steps = 200
    mp.spawn(_rank_main, args=(world, _free_port(), steps, coba, exchange, delays, slack, str(tmp_path)), nprocs=world,
             join=True)
    got = torch.load(tmp_path / 'sharded.pt')
    net = _small_net('cuda:0', None, coba, delay_e=delays[0], delay_i=delays[1],
                     **{k: v for k, v in _variant(exchange).items() if k == 'degree'})
    raster, counts = net.run(steps)
    assert int(counts.sum()) > 50
    assert torch.equal(raster.cpu(), got['raster'])
    assert torch.equal(counts.cpu(), got['counts'])
    assert torch.equal(net.spikes(), got['spikes'])


def _rank_large(rank, world, port, steps, exchange, deterministic, out_dir):
    dev, dist = _init(rank, world, port)
    try:
        net = _large_net(dev, dist.group.WORLD, exchange, deterministic)
        raster, counts = net.run(steps)
        torch.cuda.synchronize()
        if rank == 0:
            torch.save({'raster': raster.cpu(), 'counts': counts.cpu()}, os.path.join(out_dir, 'large.pt'))
        dist.barrier()
        net.close()
    finally:
        dist.destroy_process_group()


def _large_net(dev, group, exchange='p2p', deterministic=False):
    from brainstate_b200.sim import EINet, LIFParams, Lognormal
    n_exc, n_inh, K = 16000, 4000, 1000
    V0 = np.random.RandomState(404).uniform(-65, -52, n_exc + n_inh).astype(np.float32)
    params = LIFParams(V_rest=-60., ext_rate_hz=9000., ext_weight=0.3, ext_seed=405)
    return EINet(n_exc, n_inh, K, Lognormal(-2.0, 0.5, 402, 1.0), Lognormal(-2.0, 0.5, 403, -6.0),
                 seed_e=400, seed_i=401, V0=V0, params=params, device=dev, group=group, exchange=exchange,
                 deterministic=deterministic)


@pytest.mark.parametrize('exchange', ['nccl', 'p2p'])
def test_sharded_heterogeneous_network_equals_single_gpu(exchange, tmp_path):
    """The large-network recipe (1000 targets per neuron, lognormal weights, hashed drive):
    a shard's rows hold hundreds of entries.  Float accumulation: same raster as one GPU
    for the first 350 steps (the drive needs about 200 to start the activity), same rate
    afterwards within 1 %."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs at least two GPUs')
    import torch.multiprocessing as mp
    steps = 700
    mp.spawn(_rank_large, args=(2, _free_port(), steps, exchange, False, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / 'large.pt')
    raster, counts = _large_net(torch.device('cuda:0'), None).run(steps)
    assert int(counts[:350].sum()) > 100
    assert torch.equal(raster[:350].cpu(), got['raster'][:350])
    a, b = float(counts[350:].sum()), float(got['counts'][350:].sum())
    assert abs(a - b) <= 0.01 * a


def test_deterministic_sharded_network_equals_single_gpu_for_all_steps(tmp_path):
    """Fixed-point accumulation: the heterogeneous network gives the SAME raster on two GPUs
    and on one for every one of 700 steps."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs at least two GPUs')
    import torch.multiprocessing as mp
    steps = 700
    mp.spawn(_rank_large, args=(2, _free_port(), steps, 'p2p', True, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / 'large.pt')
    raster, counts = _large_net(torch.device('cuda:0'), None, deterministic=True).run(steps)
    assert int(counts[350:].sum()) > 1000
    assert torch.equal(raster.cpu(), got['raster'])
    assert torch.equal(counts.cpu(), got['counts'])


def _rank_restore(rank, world, port, out_dir):
    dev, dist = _init(rank, world, port)
    try:
        net = _small_net(dev, dist.group.WORLD, True, 'p2p', 2, 1)
        first, _ = net.run(60)
        sd = net.state_dict()
        net.run(50)                                       # go on, then return to step 60
        net.load_state_dict(sd)
        rest, _ = net.run(90)
        torch.cuda.synchronize()
        if rank == 0:
            torch.save({'raster': torch.cat([first, rest]).cpu()}, os.path.join(out_dir, 'restored.pt'))
        dist.barrier()
        net.close()
    finally:
        dist.destroy_process_group()


def test_restoring_an_earlier_checkpoint_on_two_gpus(tmp_path):
    """The exchange sequence number keeps growing when the simulation step is set back, so
    stale inbox words of the abandoned steps are never taken for current ones."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs at least two GPUs')
    import torch.multiprocessing as mp
    mp.spawn(_rank_restore, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / 'restored.pt')
    raster, _ = _small_net('cuda:0', None, True, delay_e=2, delay_i=1).run(150)
    assert int(raster.ne(0).sum()) > 0
    assert torch.equal(raster.cpu(), got['raster'])


def _rank_graph(rank, world, port, overlap, out_dir):
    dev, dist = _init(rank, world, port)
    try:
        net = _small_net(dev, dist.group.WORLD, False, 'nccl', 2, 0, overlap=overlap)
        raster, counts = net.run(120, graph_steps=24)                     # ring of 4 lists: 24 steps per replay
        torch.cuda.synchronize()
        if rank == 0:
            torch.save({'raster': raster.cpu(), 'counts': counts.cpu()}, os.path.join(out_dir, 'graph.pt'))
        dist.barrier()
        net.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('overlap', [False, True])
def test_graph_replay_of_the_all_gather_path_equals_eager(overlap, tmp_path):
    """Replaying captured split-phase steps (the launches carry their step number by value)
    gives the eager raster: the capture starts only after every delayed list exists, and a
    network with a background drive refuses it.  With ``overlap`` the captured all-gather runs
    on the process group's stream beside the scatter of the rank's own spikes."""
    if torch.cuda.device_count() < 2:
        pytest.skip('needs at least two GPUs')
    import torch.multiprocessing as mp
    mp.spawn(_rank_graph, args=(2, _free_port(), overlap, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(tmp_path / 'graph.pt')
    raster, counts = _small_net('cuda:0', None, False, delay_e=2, delay_i=0).run(120)
    assert int(counts.sum()) > 50
    assert torch.equal(raster.cpu(), got['raster'])
    assert torch.equal(counts.cpu(), got['counts'])
