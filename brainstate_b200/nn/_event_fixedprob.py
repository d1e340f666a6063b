"""Sparse event-connection layers with the reference's constructor and ``update``
signatures (``brainstate/nn/_event_fixedprob.py:102-115,202-209,249-255``).

``FixedNumConn`` takes a float input, ``EventFixedNumConn`` (alias
``EventFixedProb``) a spike vector.  The connectivity is generated exactly as the
reference generates it — ``RandomState(seed).randint(0, n_post, (n_pre, K))`` cast
to int32, then the ``afferent_ratio`` row mask from the same stream — by the
library's host generator, which reproduces NumPy's stream bit for bit.  Inputs
and outputs are CUDA tensors; every product runs in ``libbsx.so``.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Union

import numpy as np
import torch

from .. import _lib
from ..event import CSR, EventArray, FixedPostNumConn
from ._module import Module, Size
from ._state import FakeState, ParamState

__all__ = ['FixedNumConn', 'EventFixedNumConn', 'EventFixedProb', 'init_indices_without_replace',
           'fixed_num_indices']


def _device(device=None) -> torch.device:
    if device is not None:
        return torch.device(device)
    if not torch.cuda.is_available():
        raise RuntimeError('no CUDA device: the event layers compute on the GPU only')
    return torch.device('cuda', torch.cuda.current_device())


def fixed_num_indices(seed: int, n_pre: int, n_post: int, conn_num: int) -> np.ndarray:
    """Host index matrix ``(n_pre, conn_num)`` int32, equal element for element to
    ``np.random.RandomState(seed).randint(0, n_post, size=(n_pre, conn_num))``
    (``_event_fixedprob.py:165-171``), produced by the library's host generator
    without NumPy's int64 intermediate."""
    out = np.empty((n_pre, conn_num), np.int32)
    n = _lib.lib().bsx_host_fixed_num_indices(C.c_uint32(int(seed) & 0xffffffff), n_pre, n_post, conn_num,
                                              0, n_pre, 0, 0, out.ctypes.data, None)
    _lib.check(int(n))
    assert n == out.size
    return out


def fixed_num_indices_skip(rng: np.random.RandomState, count: int, n_post: int, chunk: int = 1 << 22):
    """Advances ``rng`` past ``count`` bounded draws (the index matrix), in chunks."""
    while count > 0:
        n = min(count, chunk)
        rng.randint(0, n_post, size=n)
        count -= n


def init_indices_without_replace(conn_num: int, n_pre: int, n_post: int, seed: Optional[int], method: str):
    """Per-row sampling without replacement (``_event_fixedprob.py:39-62``).

    The reference draws these from JAX's threefry generator, which is not
    available here, so this sampler is NOT bit-compatible with the reference: it
    honours the same contract (shape ``(n_pre, conn_num)``, values in
    ``[0, n_post)``, distinct within a row, reproducible from ``seed``) with the
    library's host generator (MT19937 draws, repeats within a row dropped).
    ``method`` is validated as in the reference; both methods give the same result.
    """
    if method not in ('vmap', 'for_loop'):
        raise ValueError(f"Unknown method: {method}")
    if conn_num > n_post:
        raise ValueError('cannot draw more distinct targets than there are postsynaptic neurons')
    if seed is None:
        seed = int(np.random.randint(0, 2 ** 31 - 1))
    out = np.empty((n_pre, conn_num), np.int32)
    n = _lib.lib().bsx_host_distinct_indices(C.c_uint32(int(seed) & 0xffffffff), n_pre, n_post, conn_num,
                                             out.ctypes.data)
    _lib.check(int(n))
    return out


def _init_weight(conn_weight, shape, device):
    """``init.param(conn_weight, shape)`` (``brainstate/nn/init.py:144-226``): a
    scalar passes through as a 0-d value (homogeneous weight, ``:188-189``); a
    callable is called with the shape; an array must have the shape."""
    if conn_weight is None:
        raise ValueError('conn_weight must not be None')
    if isinstance(conn_weight, torch.Tensor):
        w = conn_weight
        if w.device != device:
            w = w.to(device)
        if w.dtype != torch.float32:
            w = w.to(torch.float32)
    elif callable(conn_weight):
        w = conn_weight(shape)
        w = w if isinstance(w, torch.Tensor) else torch.as_tensor(np.asarray(w, np.float32))
        w = w.to(device=device, dtype=torch.float32)
    else:
        w = torch.as_tensor(np.asarray(conn_weight, np.float32), device=device)
    if w.numel() == 1 and tuple(w.shape) != tuple(shape):
        return w.reshape(())
    if tuple(w.shape) != tuple(shape):
        raise ValueError(f'conn_weight has shape {tuple(w.shape)}, expected {tuple(shape)} or a scalar')
    return w


class FixedNumConn(Module):
    """Fixed number of postsynaptic targets per presynaptic neuron, float input.

    Parameters follow ``brainstate.nn.FixedNumConn`` (``_event_fixedprob.py:102-115``);
    ``device`` (extra) selects the CUDA device.  ``conn_num`` as a float is a
    connection probability and resolves to ``int(out_size[-1] * conn_num)``.
    """

    __module__ = 'brainstate_b200.nn'

    def __init__(
        self,
        in_size: Size,
        out_size: Size,
        conn_num: Union[int, float],
        conn_weight: Union[Callable, float, np.ndarray, torch.Tensor],
        efferent_target: str = 'post',
        afferent_ratio: Union[int, float] = 1.,
        allow_multi_conn: bool = True,
        seed: Optional[int] = None,
        name: Optional[str] = None,
        conn_init: str = 'vmap',
        param_type: type = ParamState,
        device=None,
    ):
        super().__init__(name=name)
        self.in_size = in_size
        self.out_size = out_size
        self.efferent_target = efferent_target
        assert efferent_target in ('pre', 'post'), 'The target of the connection must be either "pre" or "post".'
        if efferent_target == 'pre':
            # the reference rejects this layout up front (_event_fixedprob.py:123-140)
            raise NotImplementedError(
                "efferent_target='pre' is not currently supported by FixedNumConn: "
                "use efferent_target='post' instead.")
        assert 0. <= afferent_ratio <= 1., 'Afferent ratio must be in [0, 1].'
        if isinstance(conn_num, float):
            assert 0. <= conn_num <= 1., 'Connection probability must be in [0, 1].'
            conn_num = int(self.out_size[-1] * conn_num)
        assert isinstance(conn_num, int), 'Connection number must be an integer.'
        self.conn_num = conn_num
        self.seed = seed
        self.allow_multi_conn = allow_multi_conn
        self.method = 'scatter'        # 'gather' = deterministic post-centric forward; 'fixed' = order-free fixed-point scatter

        dev = _device(device)
        if self.conn_num >= 1:
            n_post = self.out_size[-1]
            n_pre = self.in_size[-1]
            # One seeded host stream drives the indices and then the row mask
            # (_event_fixedprob.py:161-171,184); seed=None uses NumPy's global generator.
            if allow_multi_conn and seed is None:
                indices = np.random.randint(0, n_post, size=(n_pre, self.conn_num)).astype(np.int32)
            elif allow_multi_conn:
                indices = fixed_num_indices(seed, n_pre, n_post, self.conn_num)
            else:
                indices = init_indices_without_replace(self.conn_num, n_pre, n_post, seed, conn_init)

            if afferent_ratio == 1.:
                idx_dev = torch.from_numpy(indices).to(dev)
                w = _init_weight(conn_weight, (n_pre, self.conn_num), dev)
                self.weight = param_type(w)
                self.conn = FixedPostNumConn((w, idx_dev), shape=(n_pre, n_post))
            else:
                # the row mask continues the stream after n_pre*conn_num bounded draws
                if seed is None:
                    rng = np.random
                else:
                    rng = np.random.RandomState(seed)
                    if allow_multi_conn:
                        fixed_num_indices_skip(rng, n_pre * self.conn_num, n_post)
                self.pre_selected = rng.random_sample(n_pre) < afferent_ratio
                flat = np.ascontiguousarray(indices[self.pre_selected].reshape(-1))
                w = _init_weight(conn_weight, (flat.size,), dev)
                self.weight = param_type(w)
                indptr = (np.arange(1, n_pre + 1) * self.conn_num
                          - np.cumsum(~self.pre_selected) * self.conn_num)
                indptr = np.insert(indptr, 0, 0).astype(np.int32)
                self.conn = CSR((w, torch.from_numpy(flat).to(dev), torch.from_numpy(indptr).to(dev)),
                                shape=(n_pre, n_post))
        else:
            w = _init_weight(conn_weight, (), dev)
            self.weight = FakeState(w)

    def _apply(self, x):
        return x @ self.conn.with_data(self.weight.value)

    def update(self, x):
        if self.conn_num >= 1:
            if isinstance(x, EventArray):
                return self.conn.with_data(self.weight.value)._vecmat(x.value, event=True, method=self.method)
            return self._apply(x)
        value = x.value if isinstance(x, EventArray) else x
        weight = self.weight.value
        return torch.zeros(tuple(value.shape[:-1]) + (self.out_size[-1],), dtype=weight.dtype,
                           device=weight.device)


class EventFixedNumConn(FixedNumConn):
    """Fixed number of targets per presynaptic neuron, spike input
    (``brainstate.nn.EventFixedNumConn``, ``_event_fixedprob.py:213-252``): every
    nonzero entry of ``spk`` is one event."""

    __module__ = 'brainstate_b200.nn'

    def update(self, spk):
        return super().update(EventArray(spk))


EventFixedProb = EventFixedNumConn
