"""CPU: host-side logic of the postsynaptic sharding — block bounds, the shard's
CSR block drawn from the one seeded stream, and the per-step exchange of packed
spike words, run as two gloo ranks whose arithmetic is the CPU oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import event_oracle as eo


@pytest.mark.parametrize('n,world', [(4000, 1), (4000, 2), (4000, 8), (1000000, 8), (96, 4), (33, 2), (31, 3)])
def test_shard_bounds_partition_whole_words(n, world):
    from brainstate_b200.sim import shard_bounds, words_per_rank
    wpr = words_per_rank(n, world)
    assert wpr * world * 32 >= n
    prev = 0
    for r in range(world):
        a, b = shard_bounds(n, world, r)
        assert a == prev and a <= b <= n and a % 32 == 0 or a == n
        assert b - a <= 32 * wpr
        prev = b
    assert prev == n


def test_sharded_block_is_the_column_filter_of_the_full_matrix(bsx):
    from brainstate_b200.sim import sharded_block, shard_bounds
    seed, n_pre, n_post, K = 300, 257, 1000, 23
    full = np.random.RandomState(seed).randint(0, n_post, size=(n_pre, K)).astype(np.int32)
    total = 0
    for world in (2, 3):
        for r in range(world):
            c0, c1 = shard_bounds(n_post, world, r)
            idx, indptr = sharded_block(seed, n_pre, n_post, K, c0, c1)
            keep = (full >= c0) & (full < c1)
            assert np.array_equal(np.diff(indptr), keep.sum(axis=1))
            assert np.array_equal(idx, full[keep] - c0)            # row-major order is preserved
            total += idx.size
    assert total == 2 * full.size


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, steps, out_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from brainstate_b200.sim import shard_bounds, sharded_block, words_per_rank
        n_exc, n_inh, K = 320, 96, 12
        n = n_exc + n_inh
        first, last = shard_bounds(n, world, rank)
        ie, pe = sharded_block(100, n_exc, n, K, first, last)
        ii, pi = sharded_block(101, n_inh, n, K, first, last)
        V0 = np.random.RandomState(102).uniform(-60, -50, n).astype(np.float32)
        net = eo.EINetOracle(n_exc, n_inh, ie, np.float32(1.62), ii, np.float32(-9.0), V0=V0[first:last],
                             indptr_e=pe, indptr_i=pi, n_local=last - first)
        wpr = words_per_rank(n, world)
        words = (n + 31) // 32
        bits = torch.zeros(wpr * world, dtype=torch.int32)
        s_global = np.zeros(n, bool)
        raster = np.zeros((steps, n), bool)
        for t in range(steps):
            spk_local, _, _ = net.step(s_global)
            mine = np.zeros(wpr, np.uint32)
            packed = eo.pack_bits(spk_local)
            mine[:packed.size] = packed
            dist.all_gather_into_tensor(bits, torch.from_numpy(mine.view(np.int32)))
            s_global = eo.unpack_bits(bits.numpy().view(np.uint32)[:words], n)
            raster[t] = s_global
        if rank == 0:
            np.save(os.path.join(out_dir, 'raster.npy'), raster)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_raster(tmp_path, bsx):
    steps = 150
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), steps, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / 'raster.npy')
    n_exc, n_inh, K = 320, 96, 12
    n = n_exc + n_inh
    V0 = np.random.RandomState(102).uniform(-60, -50, n).astype(np.float32)
    ref = eo.EINetOracle(n_exc, n_inh, eo.fixed_num_indices(100, n_exc, n, K), np.float32(1.62),
                         eo.fixed_num_indices(101, n_inh, n, K), np.float32(-9.0), V0=V0).run(steps)
    assert ref.sum() > 20
    assert np.array_equal(got, ref)


def _rank_lists(rank, world, port, steps, delays, slack, cuts, out_dir):
    """One rank of the id-list exchange, restated on the CPU: every step a rank updates its
    neurons from row ``s % ring`` of its increment ring, sends the ids of its spiking neurons
    tagged with the exchange sequence number, adds its own spikes to the rows of the steps at
    which they act and does the same for the lists of step ``s - slack`` of the other ranks;
    the last ``slack`` lists are drained at the end of every launch (``cuts``)."""
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from brainstate_b200.sim import shard_bounds, sharded_block
        n_exc, n_inh, K = 320, 96, 12
        n = n_exc + n_inh
        de, di = delays
        ring = max(de, di) + 2
        first, last = shard_bounds(n, world, rank)
        n_local = last - first
        ie, pe = sharded_block(100, n_exc, n, K, first, last)
        ii, pi = sharded_block(101, n_inh, n, K, first, last)
        V0 = np.random.RandomState(102).uniform(-60, -50, n).astype(np.float32)
        net = eo.EINetOracle(n_exc, n_inh, ie, np.float32(1.62), ii, np.float32(-9.0), V0=V0[first:last],
                             indptr_e=pe, indptr_i=pi, n_local=n_local, first=first)
        incr_e = np.zeros((ring, n_local), np.float32)
        incr_i = np.zeros((ring, n_local), np.float32)
        inbox = {}                                     # (sequence number, source rank) -> ids

        def scatter(ids, fired):
            s = np.zeros(n, bool)
            s[ids] = True
            dg_e, dg_i = net.projections(s)
            incr_e[(fired + 1 + de) % ring] += dg_e
            incr_i[(fired + 1 + di) % ring] += dg_i

        def consume(seq, fired):
            for src in range(world):
                if src != rank:
                    scatter(inbox.pop((seq, src)), fired)

        raster = np.zeros((steps, n), bool)
        step = seq = 0
        for launch in cuts:
            for t in range(launch):
                row = step % ring
                spk, _, _ = net.advance(incr_e[row].copy(), incr_i[row].copy())
                incr_e[row] = 0
                incr_i[row] = 0
                mine = first + np.nonzero(spk)[0]
                lists = [None] * world
                dist.all_gather_object(lists, (seq, mine))          # the push: tag + ids to every peer
                for src, (tag, ids) in enumerate(lists):
                    assert tag == seq
                    inbox[(seq, src)] = ids
                    raster[step, ids] = True
                inbox.pop((seq, rank))
                scatter(mine, step)                                  # own spikes, at once
                if t >= slack:
                    consume(seq - slack, step - slack)               # received spikes, `slack` steps late
                step += 1
                seq += 1
            for back in range(min(slack, launch), 0, -1):            # drain before the launch ends
                consume(seq - back, step - back)
            assert not inbox
        if rank == 0:
            np.save(os.path.join(out_dir, 'raster_lists.npy'), raster)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('delays,slack,world', [((0, 0), 0, 2), ((1, 2), 1, 2), ((3, 2), 2, 2), ((3, 2), 0, 2),
                                                ((1, 2), 1, 8)])
def test_id_list_exchange_with_increment_ring_and_slack(delays, slack, world, tmp_path, bsx):
    """The protocol of the sharded step kernel (spike-id lists instead of packed words, delays by
    the row a spike is added to, lists consumed `slack` steps late, drained at launch ends) gives
    the unsharded oracle's raster on two gloo ranks, and on eight (13 spike words over 8 ranks: the
    last shards are short or empty)."""
    cuts = (1, 40, 2, 77)
    steps = sum(cuts)
    mp.spawn(_rank_lists, args=(world, _free_port(), steps, delays, slack, cuts, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / 'raster_lists.npy')
    n_exc, n_inh, K = 320, 96, 12
    n = n_exc + n_inh
    V0 = np.random.RandomState(102).uniform(-60, -50, n).astype(np.float32)
    ref = eo.EINetOracle(n_exc, n_inh, eo.fixed_num_indices(100, n_exc, n, K), np.float32(1.62),
                         eo.fixed_num_indices(101, n_inh, n, K), np.float32(-9.0), V0=V0,
                         delay_e=delays[0], delay_i=delays[1]).run(steps)
    assert ref.sum() > 20
    assert np.array_equal(got, ref)


def _rank_roll_call(rank, world, port, scenario, out_dir):
    """Host-side failure detection, with no GPU involved: ``lost`` — the last rank leaves between two
    runs and never answers again; ``late`` — it answers late but within the patience."""
    import time
    from brainstate_b200.sim import PeerLost, wait_for_peers
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    result = 'ok'
    wait_for_peers(dist.group.WORLD, 10.0)                   # everybody is there
    if scenario == 'lost' and rank == world - 1:
        os._exit(0)                                          # gone between steps, without a goodbye
    if scenario == 'late' and rank == world - 1:
        time.sleep(1.0)
    t0 = time.monotonic()
    try:
        wait_for_peers(dist.group.WORLD, 4.0)
    except PeerLost as exc:
        result = f'lost after {time.monotonic() - t0:.1f} s: {exc}'
    with open(os.path.join(out_dir, f'rank{rank}.txt'), 'w') as f:
        f.write(result)
    os._exit(0)                                              # no collective shutdown with a dead peer


@pytest.mark.parametrize('scenario', ['lost', 'late'])
def test_lost_and_late_ranks_are_noticed_on_the_host(scenario, tmp_path):
    """Before a launch whose kernels wait for one another the ranks call the roll on the host: a rank
    that left between two runs raises ``PeerLost`` on the others within the patience (no kernel is
    in flight, no GPU is involved); a rank that is merely late passes."""
    world = 3
    ctx = mp.get_context('spawn')
    port = _free_port()
    procs = [ctx.Process(target=_rank_roll_call, args=(r, world, port, scenario, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    survivors = range(world - 1) if scenario == 'lost' else range(world)
    for r in survivors:
        text = (tmp_path / f'rank{r}.txt').read_text()
        if scenario == 'lost':
            assert text.startswith('lost after') and float(text.split()[2]) < 20.0, text
        else:
            assert text == 'ok', text
    if scenario == 'lost':
        assert 'Ranks 2' in (tmp_path / 'rank0.txt').read_text()             # rank 0 names the missing rank
