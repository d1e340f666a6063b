"""Delay ring buffers for the values the event layers consume.

``Delay`` follows ``brainstate.nn.Delay`` (``brainstate/nn/_delay.py:399-958``): a ring of
``max_length = ceil(max delay / dt) + 1`` past values with a write pointer that counts
``update`` calls, named entries, retrieval by step (``:768-817``: slot
``(write_ptr - 1 - delay_step) mod max_length``), retrieval by time with nearest, linear, cubic,
Hermite or Lagrange interpolation (``:163-350,819-901``), per-element delays through index arguments, and a slower write
cadence (``update_every``, ``:903-958``).  Values are CUDA tensors; time is a plain float in the
unit of ``dt`` (physical units are not modelled).

``SpikeDelay`` is the same ring for spike vectors, bit-packed (one bit per neuron and step,
packed on the device by ``bsx_pack_spikes``): ``at`` returns packed words, which the event
products take directly (``event_matvec(..., bits=True)``), or unpacked bools on request.
"""
from __future__ import annotations

import math

import numpy as np
from typing import Callable, Dict, Optional, Union

import torch

from ._module import Module

__all__ = ['Delay', 'SpikeDelay', 'StateWithDelay']

_NEAREST = ('nearest', 'round')
_LINEAR = ('linear', 'linear_interp')


def _tap_weights(method: str, t: float):
    """Weights of the ring slots ``floor(f) + (-1, 0, 1, 2)`` for a fractional slot position
    ``f = floor(f) + t`` (a larger slot position is a more recent sample), for the four
    higher-order methods of ``brainstate/nn/_delay.py:193-350``: Catmull-Rom spline, cubic
    Hermite with central-difference tangents, and the Lagrange polynomials through 3 and 4
    neighbouring samples."""
    t2, t3 = t * t, t * t * t
    if method == 'cubic':
        return (-0.5 * t3 + t2 - 0.5 * t, 1.5 * t3 - 2.5 * t2 + 1.0, -1.5 * t3 + 2.0 * t2 + 0.5 * t, 0.5 * t3 - 0.5 * t2)
    if method == 'hermite':
        h00, h10, h01, h11 = 2 * t3 - 3 * t2 + 1, t3 - 2 * t2 + t, -2 * t3 + 3 * t2, t3 - t2
        # value = h00 v0 + h10 (v1 - v-1)/2 + h01 v1 + h11 (v2 - v0)/2
        return (-0.5 * h10, h00 - 0.5 * h11, h01 + 0.5 * h10, 0.5 * h11)
    if method == 'polynomial2':
        return (0.5 * t * (t - 1), (1 - t) * (1 + t), 0.5 * t * (t + 1), 0.0)
    if method == 'polynomial3':
        return (-t * (t - 1) * (t - 2) / 6, (t + 1) * (t - 1) * (t - 2) / 2, -t * (t + 1) * (t - 2) / 2,
                t * (t + 1) * (t - 1) / 6)
    raise ValueError(method)


_HIGHER = ('cubic', 'hermite', 'polynomial2', 'polynomial3')


def _delay_steps(time, dt: float):
    """``ceil(time / dt)`` as the reference's ``_get_delay`` (``_delay.py:351-360``), whose ceiling is
    taken in float32 (so 0.3 / 0.1 and 0.9 / 0.3 give 3, not 3 and 4); tensors give tensors."""
    if time is None:
        return 0
    if isinstance(time, (list, tuple)):
        time = torch.as_tensor(time, dtype=torch.float32)
    if isinstance(time, torch.Tensor):
        if time.dtype == torch.float64:
            q = (time / dt).to(torch.float32)
        else:
            q = time.to(torch.float32) / torch.tensor(dt, dtype=torch.float32)
        return torch.ceil(q).to(torch.int64)
    return int(math.ceil(float(np.float32(float(time) / dt))))


class Delay(Module):
    """Ring buffer of the last ``max_length`` values of one tensor.

    target : a tensor (only its shape, dtype and device are used).
    time : the largest delay to hold, in the unit of ``dt`` (more can be registered later, before
        ``init_state``).
    init : number, tensor or ``callable(shape, dtype=..., device=...)`` filling the history before t0.
    entries : ``{name: delay_time}`` or ``{name: (delay_time, *indices)}``.
    interpolation : for ``retrieve_at_time``: ``'nearest'`` (``'round'``), ``'linear'``, ``'cubic'``,
        ``'hermite'``, ``'polynomial2'``, ``'polynomial3'``, or a callable
        ``f(history, indices, float_slot, max_length)`` as the reference's registry takes.
    update_every : write a slot only every that much time (a multiple of ``dt``); ``update`` is
        still called every step.
    """

    def __init__(self, target: torch.Tensor, time=None, init=None, entries: Optional[Dict] = None,
                 interpolation: str = 'linear', update_every: Optional[float] = None, *, dt: float = 1.0,
                 name: Optional[str] = None):
        super().__init__(name=name)
        if isinstance(interpolation, str):
            if interpolation not in _NEAREST + _LINEAR + _HIGHER:
                raise ValueError(f'Unknown interpolation method: {interpolation}. Available methods: '
                                 f'{list(_NEAREST + _LINEAR + _HIGHER)}')
        elif not callable(interpolation):
            raise TypeError(f'interpolation must be str or callable, got {type(interpolation)}')
        if init is not None and not isinstance(init, (int, float, torch.Tensor)) and not callable(init):
            raise TypeError(f'init should be Array, Callable, or None. But got {init}')
        self.dt = float(dt)
        self.target_shape, self.dtype, self.device = tuple(target.shape), target.dtype, target.device
        self.interp_method = interpolation
        self._init = init
        if update_every is not None and update_every < self.dt:
            raise ValueError(f'update_every must be >= dt ({self.dt}), got {update_every}')
        self.update_every = update_every
        self.update_every_step = 1 if update_every is None else int(update_every / self.dt)
        self._slot_dt = self.dt if update_every is None else float(update_every)
        self.max_time = 0.0 if time is None else float(time)
        self.max_length = _delay_steps(time, self._slot_dt) + 1
        self._registered_entries = {}
        self.history = None
        self.write_ptr = 0
        if entries is not None:
            for entry, time_and_idx in entries.items():
                if isinstance(time_and_idx, (tuple, list)):
                    self.register_entry(entry, *time_and_idx)
                else:
                    self.register_entry(entry, time_and_idx)

    # -- state -----------------------------------------------------------------------------------
    def _new_history(self, batch_size):
        shape = (self.max_length,) + (() if batch_size is None else (int(batch_size),)) + self.target_shape
        if callable(self._init):
            return self._init(shape, dtype=self.dtype, device=self.device)
        h = torch.zeros(shape, dtype=self.dtype, device=self.device)
        if self._init is not None:
            h += torch.as_tensor(self._init, dtype=self.dtype, device=self.device)
        return h

    def init_state(self, batch_size: Optional[int] = None, **kwargs):
        self.write_ptr = 0
        self.history = self._new_history(batch_size)

    reset_state = init_state

    # -- registration ------------------------------------------------------------------------------
    def register_delay(self, *time_and_idx):
        assert len(time_and_idx) >= 1, 'You should provide at least one delay time.'
        for ix in time_and_idx[1:]:
            ok = isinstance(ix, int) or (isinstance(ix, torch.Tensor) and not ix.dtype.is_floating_point)
            assert ok, f'The index should be integer. But got {ix}.'
        if time_and_idx[0] is None:
            return None
        t = time_and_idx[0]
        step = _delay_steps(t, self._slot_dt)
        top = int(step.max()) if isinstance(step, torch.Tensor) else step
        if isinstance(step, torch.Tensor) and step.dim() > 1:
            raise ValueError('delay times are scalars or one-dimensional')
        tmax = float(torch.as_tensor(t, dtype=torch.float64).max()) if not isinstance(t, (int, float)) else float(t)
        self.max_time = max(self.max_time, tmax)
        if self.max_length <= top + 1:
            if self.history is not None:
                raise RuntimeError('a longer delay cannot be registered after init_state')
            self.max_length = top + 1
        if isinstance(step, torch.Tensor):
            step = step.to(self.device)
        return (step,) + tuple(time_and_idx[1:])

    def register_entry(self, entry: str, *time_and_idx):
        if entry in self._registered_entries:
            raise KeyError(f'Entry {entry} has been registered. The existing delay for the key {entry} is '
                           f'{self._registered_entries[entry]}. The new delay for the key {entry} is '
                           f'{time_and_idx}. You can use another key. ')
        info = self.register_delay(*time_and_idx)
        self._registered_entries[entry] = info
        return info

    def at(self, entry: str):
        assert isinstance(entry, str), f'entry should be a string for describing the entry of the delay data. But we got {entry}.'
        if entry not in self._registered_entries:
            raise KeyError(f'Does not find delay entry "{entry}".')
        info = self._registered_entries[entry]
        if info is None:
            info = (0,)
        return self.retrieve_at_step(*info)

    # -- retrieval -----------------------------------------------------------------------------------
    def _slot(self, delay_step):
        current = (self.write_ptr - 1) // self.update_every_step
        if isinstance(delay_step, torch.Tensor):
            if delay_step.dtype.is_floating_point:
                raise ValueError(f'"delay_len" must be integer, but we got {delay_step}')
            return torch.remainder(current - delay_step, self.max_length)
        if not isinstance(delay_step, int):
            raise ValueError(f'"delay_len" must be integer, but we got {delay_step}')
        if delay_step >= self.max_length:
            raise ValueError(f'The request delay length should be less than the maximum delay '
                             f'{self.max_length - 1}. But we got {delay_step}')
        return (current - delay_step) % self.max_length

    def retrieve_at_step(self, delay_step, *indices):
        assert self.history is not None, 'The delay history is not initialized.'
        assert delay_step is not None, 'The delay step should be given.'
        slot = self._slot(delay_step)
        if isinstance(slot, torch.Tensor) and int(delay_step.max()) >= self.max_length:
            raise ValueError(f'The request delay length should be less than the maximum delay '
                             f'{self.max_length - 1}. But we got {int(delay_step.max())}')
        return self.history[(slot,) + tuple(indices)]

    def retrieve_at_time(self, delay_time: float, current_time: float, *indices):
        """The value at absolute time ``delay_time`` when the newest slot holds ``current_time``."""
        assert self.history is not None, 'The delay history is not initialized.'
        if delay_time > current_time + 1e-9 or delay_time < current_time - self.max_time - self.dt - 1e-9:
            raise ValueError(f'The request delay time should be within '
                             f'[{current_time - self.max_time - self.dt}, {current_time}], but we got {delay_time}')
        f = (current_time - delay_time) / self._slot_dt
        if callable(self.interp_method) or self.interp_method in _HIGHER:
            slot = (self.write_ptr - 1) // self.update_every_step - f        # fractional position in the ring
            if callable(self.interp_method):
                return self.interp_method(self.history, tuple(indices), slot, self.max_length)
            i0 = math.floor(slot)
            out = None
            for k, wk in zip((-1, 0, 1, 2), _tap_weights(self.interp_method, slot - i0)):
                if wk != 0.0:
                    term = self.history[((i0 + k) % self.max_length,) + tuple(indices)] * wk
                    out = term if out is None else out + term
            return out
        if self.interp_method in _NEAREST:
            return self.retrieve_at_step(int(round(f)), *indices)
        lo, hi = int(math.floor(f + 1e-12)), int(math.ceil(f - 1e-12))
        a = self.retrieve_at_step(lo, *indices)
        if hi == lo:
            return a
        b = self.retrieve_at_step(hi, *indices)
        t = f - lo
        return a * (1 - t) + b * t

    # -- update -----------------------------------------------------------------------------------------
    def update(self, current: torch.Tensor) -> None:
        assert self.history is not None, 'The delay history is not initialized.'
        if self.write_ptr % self.update_every_step == 0:
            self.history[self.write_ptr // self.update_every_step].copy_(current)
        self.write_ptr = (self.write_ptr + 1) % (self.max_length * self.update_every_step)


class StateWithDelay(Delay):
    """A ``Delay`` that reads the delayed value from ``getattr(target, item).value`` on every
    ``update()`` (``brainstate/nn/_delay.py:960-1079``)."""

    def __init__(self, target, item: str, init: Union[Callable, None] = None, interpolation: str = 'round', **kwargs):
        self._target, self._target_term = target, item
        super().__init__(self.state.value, init=init, interpolation=interpolation, **kwargs)

    @property
    def state(self):
        r = getattr(self._target, self._target_term)
        if not hasattr(r, 'value'):
            raise TypeError(f'The term "{self._target_term}" in the module "{self._target}" is not a State.')
        return r

    def update(self, *args) -> None:
        return super().update(self.state.value)


class SpikeDelay(Module):
    """Ring of the last ``max_length`` spike vectors, one bit per neuron and step.

    ``update(spk)`` packs a bool / uint8 / float32 CUDA vector (``(n,)`` or ``(batch, n)``) into
    32-bit words on the device; ``retrieve_at_step(d)`` / ``at(entry)`` return the packed words of
    ``d`` steps ago (``bits=True``, what ``event_matvec(..., bits=True)`` and the C ABI's
    ``BSX_SPK_BITS32`` take) or the bool vector.  Slot arithmetic as in ``Delay``.
    """

    def __init__(self, n: int, time=None, entries: Optional[Dict] = None, *, dt: float = 1.0, device='cuda',
                 name: Optional[str] = None):
        super().__init__(name=name)
        self.n, self.words = int(n), (int(n) + 31) // 32
        self.dt, self.device = float(dt), torch.device(device)
        self.max_length = _delay_steps(time, self.dt) + 1
        self._registered_entries = {}
        self.history = None
        self.write_ptr = 0
        for entry, t in (entries or {}).items():
            self.register_entry(entry, t)

    def register_entry(self, entry: str, time):
        if entry in self._registered_entries:
            raise KeyError(f'Entry {entry} has been registered.')
        step = _delay_steps(time, self.dt)
        if self.max_length <= step + 1:
            if self.history is not None:
                raise RuntimeError('a longer delay cannot be registered after init_state')
            self.max_length = step + 1
        self._registered_entries[entry] = step
        return step

    def init_state(self, batch_size: Optional[int] = None, **kwargs):
        shape = (self.max_length,) + (() if batch_size is None else (int(batch_size),)) + (self.words,)
        self.history = torch.zeros(shape, dtype=torch.int32, device=self.device)
        self.write_ptr = 0

    reset_state = init_state

    def update(self, spk: torch.Tensor) -> None:
        from ..event import pack_spikes
        assert self.history is not None, 'The delay history is not initialized.'
        self.history[self.write_ptr].copy_(pack_spikes(spk))
        self.write_ptr = (self.write_ptr + 1) % self.max_length

    def retrieve_at_step(self, delay_step: int, bits: bool = True):
        assert self.history is not None, 'The delay history is not initialized.'
        if not 0 <= delay_step < self.max_length:
            raise ValueError(f'The request delay length should be less than the maximum delay '
                             f'{self.max_length - 1}. But we got {delay_step}')
        w = self.history[(self.write_ptr - 1 - delay_step) % self.max_length]
        if bits:
            return w
        shifts = torch.arange(32, device=w.device, dtype=torch.int32)
        b = (w.unsqueeze(-1) >> shifts) & 1
        return b.reshape(w.shape[:-1] + (self.words * 32,))[..., :self.n].to(torch.bool)

    def at(self, entry: str, bits: bool = True):
        if entry not in self._registered_entries:
            raise KeyError(f'Does not find delay entry "{entry}".')
        return self.retrieve_at_step(self._registered_entries[entry], bits=bits)
