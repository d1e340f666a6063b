"""Dense event layer with the reference's signature
(``brainstate/nn/_event_linear.py:53-102``).

``EventLinear.update(spk)``: with a scalar weight every output receives
``count(spk != 0) * w`` (``float_as_event``) or ``sum(spk) * w``; with a matrix
weight the output is ``[spk != 0] @ W`` or the plain ``spk @ W``.  The event-driven
forward, its weight cotangent ``[spk != 0]^T @ ct`` and the scalar-weight form are
kernels of ``libbsx.so``; the plain dense product and the input cotangent ``ct @ W^T``
are ordinary dense GEMMs and go to ``torch.matmul``.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Union

import numpy as np
import torch

from .. import _lib
from ..event import _flatten_batch, _require_cuda, spike_format_of
from ._event_fixedprob import _device, _init_weight
from ._module import Module, Size
from ._state import ParamState

__all__ = ['EventLinear', 'dense_event_matmul']


class _DenseEvent(torch.autograd.Function):
    """``y = [spk != 0] @ W``.  The cotangent w.r.t. a float ``spk`` is the dense
    ``ct @ W^T`` (the value-sum gradient, ``_event_linear.py:84-91``); w.r.t. ``W``
    it is ``[spk != 0]^T @ ct``."""

    @staticmethod
    def forward(spk, weight):
        _require_cuda(spk, 'spikes')
        n_pre, n_post = weight.shape
        sb, lead = _flatten_batch(spk, n_pre)
        w = weight.contiguous()
        out = torch.empty((sb.shape[0], n_post), dtype=torch.float32, device=spk.device)
        _lib.check(_lib.lib().bsx_dense_event_vecmat(_lib.ptr(sb), spike_format_of(sb), _lib.ptr(w),
                                                     sb.shape[0], n_pre, n_post, _lib.ptr(out),
                                                     _lib.current_stream()))
        return out.reshape(lead + (n_post,))

    @staticmethod
    def setup_context(ctx, inputs, output):
        spk, weight = inputs
        ctx.save_for_backward(spk, weight)
        ctx.save_for_forward(spk, weight)

    @staticmethod
    def backward(ctx, ct):
        spk, weight = ctx.saved_tensors
        d_spk = d_w = None
        if ctx.needs_input_grad[0] and spk.dtype.is_floating_point:
            d_spk = ct @ weight.t()
        if ctx.needs_input_grad[1]:
            n_pre, n_post = weight.shape
            sb, _ = _flatten_batch(spk, n_pre)
            ctb = ct.reshape(-1, n_post).to(torch.float32).contiguous()
            if n_pre <= 65535 and sb.dtype in (torch.bool, torch.uint8, torch.float32):
                d_w = torch.empty((n_pre, n_post), dtype=torch.float32, device=ct.device)
                _lib.check(_lib.lib().bsx_dense_event_dw(_lib.ptr(sb), spike_format_of(sb), _lib.ptr(ctb), sb.shape[0],
                                                         n_pre, n_post, _lib.ptr(d_w), _lib.current_stream()))
            else:
                d_w = (sb != 0).to(torch.float32).t() @ ctb
        return d_spk, d_w

    @staticmethod
    def jvp(ctx, spk_dot, w_dot):
        spk, weight = ctx.saved_tensors
        out = None
        if spk_dot is not None:
            out = spk_dot.to(torch.float32) @ weight
        if w_dot is not None:
            term = _DenseEvent.apply(spk, w_dot)
            out = term if out is None else out + term
        return out


class _DenseScalar(torch.autograd.Function):
    """``y[..., :] = r * w`` with ``r`` the event count or the value sum of the last axis of ``spk``
    (``_event_linear.py:77-97``).  The cotangent of a float ``spk`` is ``w * sum_j ct[..., j]`` for
    every input (the reference routes the gradient through the value sum, ``:84-91``)."""

    @staticmethod
    def forward(spk, weight, float_as_event, n_post):
        _require_cuda(spk, 'spikes')
        n_pre = spk.shape[-1]
        sb, lead = _flatten_batch(spk, n_pre)
        if sb.dtype not in (torch.bool, torch.uint8, torch.float32):
            sb = sb.to(torch.float32)
        out = torch.empty((sb.shape[0], n_post), dtype=torch.float32, device=spk.device)
        reduced = torch.empty(sb.shape[0], dtype=torch.float32, device=spk.device)
        w = weight.reshape(1).to(torch.float32).contiguous()
        _lib.check(_lib.lib().bsx_dense_event_scalar(_lib.ptr(sb), spike_format_of(sb), _lib.ptr(w), int(float_as_event),
                                                     sb.shape[0], n_pre, n_post, _lib.ptr(out), _lib.ptr(reduced),
                                                     _lib.current_stream()))
        return out.reshape(lead + (n_post,)), reduced.reshape(lead)

    @staticmethod
    def setup_context(ctx, inputs, output):
        spk, weight, _, _ = inputs
        ctx.save_for_backward(weight, output[1])
        ctx.spk_shape, ctx.spk_float = spk.shape, spk.dtype.is_floating_point
        ctx.mark_non_differentiable(output[1])

    @staticmethod
    def backward(ctx, ct, _):
        weight, reduced = ctx.saved_tensors
        row = ct.sum(dim=-1)                                     # (batch dims)
        d_spk = d_w = None
        if ctx.needs_input_grad[0] and ctx.spk_float:
            d_spk = (row * weight.reshape(())).unsqueeze(-1).expand(ctx.spk_shape)
        if ctx.needs_input_grad[1]:
            d_w = (row * reduced).sum().reshape(weight.shape)
        return d_spk, d_w, None, None


def dense_event_matmul(spk: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``brainevent.EventArray(spk) @ weight`` for a dense ``weight``."""
    return _DenseEvent.apply(spk, weight)


class EventLinear(Module):
    """``brainstate.nn.EventLinear`` (``_event_linear.py:33-102``).  ``block_size`` is
    kept for signature compatibility and unused, as in the reference (``:69``)."""

    __module__ = 'brainstate_b200.nn'

    def __init__(
        self,
        in_size: Size,
        out_size: Size,
        weight: Union[Callable, float, np.ndarray, torch.Tensor],
        float_as_event: bool = True,
        block_size: int = 64,
        name: Optional[str] = None,
        param_type: type = ParamState,
        device=None,
    ):
        super().__init__(name=name)
        self.in_size = in_size
        self.out_size = out_size
        self.float_as_event = float_as_event
        self.block_size = block_size
        w = _init_weight(weight, (self.in_size[-1], self.out_size[-1]), _device(device))
        self.weight = param_type(w)

    def update(self, spk: torch.Tensor) -> torch.Tensor:
        weight = self.weight.value
        if weight.numel() == 1:
            # homogeneous weight: reduce, then broadcast (_event_linear.py:77-97), one kernel
            return _DenseScalar.apply(spk, weight, self.float_as_event, self.out_size[-1])[0]
        if self.float_as_event:
            return dense_event_matmul(spk, weight)
        return spk.to(torch.float32) @ weight
