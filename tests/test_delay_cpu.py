"""The delay ring buffer against a plain list of past values (the semantics of
``brainstate/nn/_delay.py:768-817,903-958``: slot ``(write_ptr - 1 - delay) mod max_length``,
one write per ``update``, ``update_every`` cadence), on CPU tensors."""
import numpy as np
import pytest
import torch

from brainstate_b200.nn import Delay, StateWithDelay, State


def test_retrieve_at_step_equals_list_of_past_values():
    rs = np.random.RandomState(0)
    d = Delay(torch.zeros(5), time=0.7, dt=0.1, init=-1.0)
    assert d.max_length == 8
    d.init_state()
    past = []
    for t in range(30):
        v = torch.from_numpy(rs.standard_normal(5).astype(np.float32))
        d.update(v)
        past.append(v)
        for k in range(8):
            want = past[-1 - k] if k < len(past) else torch.full((5,), -1.0)
            assert torch.equal(d.retrieve_at_step(k), want)
    with pytest.raises(ValueError, match='less than the maximum delay 7'):
        d.retrieve_at_step(8)


def test_entries_vector_delays_and_batches():
    d = Delay(torch.zeros(4), entries={'a': 0.3, 'b': (torch.tensor([0.0, 0.1, 0.2, 0.5]), torch.arange(4))}, dt=0.1)
    assert d.max_length == 6                       # grew to hold the 0.5 tap
    with pytest.raises(KeyError, match='has been registered'):
        d.register_entry('a', 0.1)
    d.init_state(batch_size=None)
    past = []
    for t in range(12):
        v = torch.arange(4, dtype=torch.float32) + 10 * t
        d.update(v)
        past.append(v)
    assert torch.equal(d.at('a'), past[-4])
    steps = [0, 1, 2, 5]
    assert torch.equal(d.at('b'), torch.stack([past[-1 - s][i] for i, s in enumerate(steps)]))
    with pytest.raises(KeyError, match='Does not find delay entry'):
        d.at('c')
    db = Delay(torch.zeros(3), time=2, dt=1.0)
    db.init_state(batch_size=2)
    assert db.history.shape == (3, 2, 3)
    db.update(torch.ones(2, 3))
    assert torch.equal(db.retrieve_at_step(0), torch.ones(2, 3)) and torch.equal(db.retrieve_at_step(1), torch.zeros(2, 3))


def test_retrieve_at_time_interpolates():
    d = Delay(torch.zeros(1), time=1.0, dt=0.25, interpolation='linear')
    d.init_state()
    for t in range(6):                                       # value = time of the sample
        d.update(torch.tensor([0.25 * t]))
    now = 1.25
    assert torch.allclose(d.retrieve_at_time(1.0, now), torch.tensor([1.0]))
    assert torch.allclose(d.retrieve_at_time(0.9, now), torch.tensor([0.9]))
    dn = Delay(torch.zeros(1), time=1.0, dt=0.25, interpolation='round')
    dn.init_state()
    for t in range(6):
        dn.update(torch.tensor([0.25 * t]))
    assert torch.allclose(dn.retrieve_at_time(0.9, now), torch.tensor([1.0]))
    with pytest.raises(ValueError, match='should be within'):
        d.retrieve_at_time(1.5, now)
    with pytest.raises(ValueError, match='Unknown interpolation'):
        Delay(torch.zeros(1), interpolation='spline')


def test_update_every_writes_one_slot_per_interval():
    d = Delay(torch.zeros(1), time=4.0, dt=1.0, update_every=2.0)
    assert d.update_every_step == 2 and d.max_length == 3
    d.init_state()
    for t in range(9):
        d.update(torch.tensor([float(t)]))
    # slots were written at calls 0, 2, 4 (wrap) 6, 8: the newest slot holds call 8, one back call 6
    assert d.retrieve_at_step(0).item() == 8.0 and d.retrieve_at_step(1).item() == 6.0 and d.retrieve_at_step(2).item() == 4.0
    with pytest.raises(ValueError, match='update_every must be >= dt'):
        Delay(torch.zeros(1), dt=1.0, update_every=0.5)


def test_state_with_delay_reads_the_target_state():
    class Cell:
        def __init__(self):
            self.V = State(torch.zeros(3))
    c = Cell()
    d = StateWithDelay(c, 'V', time=2, dt=1.0)
    d.init_state()
    for t in range(4):
        c.V.value = torch.full((3,), float(t))
        d.update()
    assert torch.equal(d.retrieve_at_step(2), torch.full((3,), 1.0))


def _filled(method, fn, length=12, dt=0.5):
    d = Delay(torch.zeros(2, dtype=torch.float64), time=(length - 1) * dt, dt=dt, interpolation=method)
    d.init_state()
    for k in range(length):                                   # sample k holds fn(k * dt)
        d.update(torch.tensor([fn(k * dt), 2 * fn(k * dt)], dtype=torch.float64))
    return d, (length - 1) * dt


@pytest.mark.parametrize('method', ['cubic', 'hermite', 'polynomial2', 'polynomial3'])
def test_higher_order_interpolation(method):
    """Each method reproduces the polynomials it must: all four are exact on straight lines, the 3- and
    4-point Lagrange forms on parabolas, the 4-point form on cubics; Catmull-Rom and the Hermite form
    with central-difference tangents are the same spline."""
    line = lambda t: 3.0 - 2.0 * t
    para = lambda t: 1.0 + t - 0.5 * t * t
    cube = lambda t: 0.25 * t ** 3 - t + 2.0
    for t_query in (2.1, 3.25, 3.5, 4.9):
        d, now = _filled(method, line)
        assert torch.allclose(d.retrieve_at_time(t_query, now), torch.tensor([line(t_query), 2 * line(t_query)], dtype=torch.float64))
        if method.startswith('polynomial'):
            d, now = _filled(method, para)
            assert torch.allclose(d.retrieve_at_time(t_query, now)[0], torch.tensor(para(t_query), dtype=torch.float64))
        if method == 'polynomial3':
            d, now = _filled(method, cube)
            assert torch.allclose(d.retrieve_at_time(t_query, now)[0], torch.tensor(cube(t_query), dtype=torch.float64))
    a, now = _filled('cubic', cube)
    b, _ = _filled('hermite', cube)
    assert torch.allclose(a.retrieve_at_time(3.3, now), b.retrieve_at_time(3.3, now))
    # at a sample every method returns the sample
    assert torch.allclose(a.retrieve_at_time(3.0, now)[0], torch.tensor(cube(3.0), dtype=torch.float64))


def test_custom_interpolation_callable():
    seen = {}

    def pick(history, indices, slot, max_length):
        seen['slot'] = slot
        return history[(int(round(slot)) % max_length,) + indices]
    d = Delay(torch.zeros(1), time=3.0, dt=1.0, interpolation=pick)
    d.init_state()
    for k in range(4):
        d.update(torch.tensor([float(k)]))
    assert d.retrieve_at_time(1.0, 3.0).item() == 1.0 and seen['slot'] % 4 == 1.0       # the ring position, up to whole turns
    with pytest.raises(TypeError, match='str or callable'):
        Delay(torch.zeros(1), interpolation=3)
