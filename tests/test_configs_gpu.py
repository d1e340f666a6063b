"""GPU: the network configurations at their full size against the CPU oracle.

``cuba``: the 4 000-neuron current-based E/I network for its full 1 000 steps.
``coba``: the 1 000 000-neuron conductance-based network (10^8 synapses, constant bias
tuned to about 10 Hz) for 300 steps.  Homogeneous weights make every synaptic sum
independent of the order of the adds, so the rasters must be identical step for step
(the bar is 200 identical steps) and the per-population rates equal (the bar is 1 %).
The dynamics oracle itself is builder-specified: parity with the reference is unpinned.
"""
import numpy as np
import pytest
import torch

from oracle import event_oracle as eo

pytestmark = pytest.mark.gpu


def _oracle(name, p):
    n = p['n_exc'] + p['n_inh']
    K = p['conn_num']
    ie = eo.fixed_num_indices(p['seed_e'], p['n_exc'], n, K, chunk_rows=100000)
    ii = eo.fixed_num_indices(p['seed_i'], p['n_inh'], n, K, chunk_rows=100000)
    V0 = np.random.RandomState(p['seed_v']).uniform(p['v0'][0], p['v0'][1], n).astype(np.float32)
    q = p['params']
    orc = eo.EINetOracle(p['n_exc'], p['n_inh'], ie, np.float32(p['w_e']), ii, np.float32(p['w_i']), coba=q.coba,
                         dt=q.dt, tau_m=q.tau_m, tau_e=q.tau_e, tau_i=q.tau_i, V_rest=q.V_rest, V_th=q.V_th,
                         V_reset=q.V_reset, tau_ref=q.tau_ref, R=q.R, I_ext=q.I_ext, E_e=q.E_e, E_i=q.E_i, V0=V0)
    return orc, ie, ii


def test_cuba_network_full_1000_steps(cuda):
    from brainstate_b200.sim import from_preset, preset, unpack_raster, population_rates
    p = preset('cuba')
    n = p['n_exc'] + p['n_inh']
    orc, ie, ii = _oracle('cuba', p)
    ref = orc.run(1000)
    assert ref.sum() > 2000
    one_block = from_preset('cuba', cuda)                       # 4 000 neurons: single-block kernel
    shard = from_preset('cuba', cuda, shard_kernel=True)        # increment rows, one barrier per step
    coop = from_preset('cuba', cuda)
    assert np.array_equal(one_block.conn_e.indices.cpu().numpy(), ie)
    assert np.array_equal(one_block.conn_i.indices.cpu().numpy(), ii)
    r1, c1 = one_block.run(1000)
    r2, c2 = shard.run(1000)
    r3, _ = coop.run(1000, blocks=16)                           # cooperative kernel, state in global memory
    got = unpack_raster(r1, n)
    diff = np.nonzero((got != ref).any(axis=1))[0]
    assert diff.size == 0, f'rasters diverge at step {diff[0]}'
    assert torch.equal(r1, r2) and torch.equal(r1, r3) and torch.equal(c1, c2)
    assert np.array_equal(c1.cpu().numpy(), ref.sum(axis=1))
    re, ri = population_rates(r1, p['n_exc'], p['n_inh'], 0.1)
    assert re == pytest.approx(ref[:, :p['n_exc']].sum() / p['n_exc'] / 0.1, rel=1e-12)
    assert ri == pytest.approx(ref[:, p['n_exc']:].sum() / p['n_inh'] / 0.1, rel=1e-12)
    np.testing.assert_allclose(one_block.V.cpu().numpy(), orc.V, rtol=1e-5, atol=1e-6)


def test_coba_network_one_million_neurons_300_steps(cuda):
    from brainstate_b200.sim import from_preset, preset
    p = preset('coba')
    n = p['n_exc'] + p['n_inh']
    orc, ie, ii = _oracle('coba', p)
    lists = from_preset('coba', cuda)                           # spike-list kernel, state resident on chip
    assert np.array_equal(lists.conn_e.indices.cpu().numpy(), ie)
    assert np.array_equal(lists.conn_i.indices.cpu().numpy(), ii)
    del ie, ii
    steps = 300
    raster, counts = lists.run(steps)
    words = raster.cpu().numpy().view(np.uint32)
    total = 0
    for t in range(steps):
        spk, dg_e, dg_i = orc.step()
        total += int(spk.sum())
        assert np.array_equal(eo.pack_bits(spk), words[t]), f'rasters diverge at step {t}'
    assert total > 100000                                       # about 10 Hz: 10^6 neurons x 30 ms
    assert int(counts.sum()) == total
    np.testing.assert_allclose(lists.V.cpu().numpy(), orc.V, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(lists.g_e.cpu().numpy(), orc.g_e, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(lists.g_i.cpu().numpy(), orc.g_i, rtol=1e-5, atol=1e-6)
    assert np.array_equal(lists.ref.cpu().numpy(), orc.ref)
    del lists
    shard = from_preset('coba', cuda, shard_kernel=True)        # the kernel the sharded runs use, world of one
    r2, c2 = shard.run(steps)
    assert torch.equal(raster, r2) and torch.equal(counts, c2)


def test_coba_preset_fires_at_about_ten_hertz(cuda):
    """The bias of the preset: mean rate over the configuration's 1000 steps within 5 % of 10 Hz."""
    from brainstate_b200.sim import from_preset, preset
    p = preset('coba')
    net = from_preset('coba', cuda)
    _, counts = net.run(1000, record=False)
    rate = float(counts.sum()) / (p['n_exc'] + p['n_inh']) / 0.1
    assert 9.5 <= rate <= 10.5, rate
