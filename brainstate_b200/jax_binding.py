"""JAX binding of the bsx library through XLA FFI custom calls.

This is the registration module a JAX-based ``brainstate`` would import in place of
``brainevent``: it registers the handlers of ``ffi/bsx_ffi.cc`` as XLA custom-call targets
and defines, for the product behind ``brainstate.nn.FixedNumConn.update``
(``brainstate/nn/_event_fixedprob.py:202-205,249-252``),

* a primitive-like callable with a reverse-mode rule (``jax.custom_vjp``: the transpose
  product and the weight cotangent pinned by ``_event_fixedprob_test.py:56-88``),
* a forward-mode variant (``jax.custom_jvp``: ``y_dot = x_dot @ W + a @ W_dot``,
  ``_event_fixedprob_test.py:90-126``),
* batching by folding leading dimensions into the batch the kernels take natively
  (``vmap_method='broadcast_all'``: a ``jax.vmap`` over spikes stays one launch).

The pattern follows how the reference registers its own primitives
(``brainstate/transform/_unvmap.py:90,135-141``).

JAX is not a dependency of this package: importing this module without ``jax`` raises
``ImportError`` with that message, nothing else in the package imports it, and it has not
been run in an environment that has jaxlib (none was available when it was written).
Build the handler library first (see the header of ``ffi/bsx_ffi.cc``) and pass its path
to :func:`register`.
"""
from __future__ import annotations

import ctypes
import os

try:
    import jax
    import jax.numpy as jnp
    import numpy as np
    from jax import ffi as jffi
except ImportError as e:                                      # pragma: no cover - needs jax
    raise ImportError('brainstate_b200.jax_binding needs jax and jaxlib (with jax.ffi); '
                      'the torch-based layers in brainstate_b200.nn do not') from e

from . import _lib

__all__ = ['register', 'event_vecmat', 'float_vecmat', 'event_vecmat_fwd_mode', 'event_matvec', 'dense_event_vecmat']

_TARGETS = ('bsx_ffi_vecmat', 'bsx_ffi_matvec', 'bsx_ffi_vecmat_vjp', 'bsx_ffi_dense_event_vecmat')
_registered = False


def register(ffi_library: str | None = None):
    """Loads ``libbsx_ffi.so`` (default: beside ``libbsx.so``) and registers its handlers for
    the CUDA platform.  Idempotent."""
    global _registered
    if _registered:
        return
    _lib.lib()                                               # libbsx.so first: the handlers link against it
    path = ffi_library or os.path.join(os.path.dirname(_lib.LIB_PATH), 'libbsx_ffi.so')
    handle = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    for name in _TARGETS:
        jffi.register_ffi_target(name, jffi.pycapsule(getattr(handle, name)), platform='CUDA')
    _registered = True


def _conn_operands(indices, indptr, weights):
    indices = jnp.asarray(indices, jnp.int32)
    indptr = jnp.zeros((0,), jnp.int32) if indptr is None else jnp.asarray(indptr)
    weights = jnp.asarray(weights, jnp.float32).reshape(-1) if jnp.ndim(weights) == 0 else jnp.asarray(weights, jnp.float32)
    return indices, indptr, weights


def _n_pre(indices, indptr):
    return indices.shape[0] if indptr is None else indptr.shape[0] - 1


def _scratch(nbytes: int):
    return jax.ShapeDtypeStruct((max(int(nbytes), 16),), jnp.uint8)


def _vecmat_call(x, indices, indptr, weights, n_post: int, event: bool):
    register()
    idx, ip, w = _conn_operands(indices, indptr, weights)
    lead = x.shape[:-1]
    batch = int(np.prod(lead)) if lead else 1
    ws = _lib.lib().bsx_event_vecmat_workspace_bytes(batch, x.shape[-1])
    out = jax.ShapeDtypeStruct(lead + (n_post,), jnp.float32)
    y, _ = jffi.ffi_call('bsx_ffi_vecmat', (out, _scratch(ws)), vmap_method='broadcast_all')(
        x, idx, ip, w, n_post=np.int64(n_post), event=bool(event))
    return y


def _vjp_call(x, ct, indices, indptr, weights, event: bool, need_dx: bool, need_dw: bool):
    register()
    idx, ip, w = _conn_operands(indices, indptr, weights)
    lead = x.shape[:-1]
    batch = int(np.prod(lead)) if lead else 1
    ws = _lib.lib().bsx_vecmat_vjp_batched_workspace_bytes(batch, ct.shape[-1])
    dx = jax.ShapeDtypeStruct(x.shape if need_dx else (0,), jnp.float32)
    dw = jax.ShapeDtypeStruct(w.shape if need_dw else (0,), jnp.float32)
    dx, dw, _ = jffi.ffi_call('bsx_ffi_vecmat_vjp', (dx, dw, _scratch(ws)), vmap_method='sequential')(
        x, ct.astype(jnp.float32), idx, ip, w, event=bool(event))
    return dx, dw


def _make_vecmat(event: bool):
    @jax.custom_vjp
    def vecmat(x, weights, indices, indptr, n_post):
        return _vecmat_call(x, indices, indptr, weights, n_post, event)

    def fwd(x, weights, indices, indptr, n_post):
        return _vecmat_call(x, indices, indptr, weights, n_post, event), (x, weights, indices, indptr)

    def bwd(res, ct):
        x, weights, indices, indptr = res
        float_x = jnp.issubdtype(x.dtype, jnp.floating)
        dx, dw = _vjp_call(x, ct, indices, indptr, weights, event, need_dx=float_x, need_dw=True)
        dx = dx.astype(x.dtype) if float_x else np.zeros(x.shape, jax.dtypes.float0)
        return dx, dw.reshape(jnp.shape(weights)), None, None, None

    vecmat.defvjp(fwd, bwd)
    return vecmat


_event_vecmat = _make_vecmat(True)
_float_vecmat = _make_vecmat(False)


def event_vecmat(spk, weights, indices, n_post: int, indptr=None):
    """``EventArray(spk) @ conn``: every nonzero entry of ``spk`` is a unit event.  Reverse-mode
    differentiable in ``weights`` and (for float ``spk``) in ``spk``: the input cotangent is the
    dense ``ct @ W^T`` (``brainstate/nn/_event_linear.py:84-91``)."""
    return _event_vecmat(spk, weights, jnp.asarray(indices, jnp.int32), indptr, n_post)


def float_vecmat(x, weights, indices, n_post: int, indptr=None):
    """``x @ conn`` for float ``x`` (``brainstate/nn/_event_fixedprob.py:202-205``)."""
    return _float_vecmat(x, weights, jnp.asarray(indices, jnp.int32), indptr, n_post)


def event_vecmat_fwd_mode(spk, weights, indices, n_post: int, indptr=None):
    """The same product with a forward-mode rule (``jax.jvp`` / ``jax.jacfwd``):
    ``y_dot = spk_dot @ W + [spk != 0] @ W_dot`` — two more launches of the same kernels."""
    idx = jnp.asarray(indices, jnp.int32)

    @jax.custom_jvp
    def f(spk, weights):
        return _vecmat_call(spk, idx, indptr, weights, n_post, True)

    @f.defjvp
    def f_jvp(primals, tangents):
        spk, weights = primals
        s_dot, w_dot = tangents
        y = f(spk, weights)
        y_dot = _vecmat_call(jnp.asarray(s_dot, jnp.float32), idx, indptr, weights, n_post, False)
        y_dot = y_dot + _vecmat_call(spk, idx, indptr, w_dot, n_post, True)
        return y, y_dot

    return f(spk, weights)


def event_matvec(spk_post, weights, indices, indptr=None):
    """``conn @ EventArray(spk_post)``: deterministic gather over the rows."""
    register()
    idx, ip, w = _conn_operands(indices, indptr, weights)
    n_pre = _n_pre(idx, indptr)
    lead = spk_post.shape[:-1]
    batch = int(np.prod(lead)) if lead else 1
    ws = _lib.lib().bsx_event_matvec_workspace_bytes(batch, spk_post.shape[-1])
    out = jax.ShapeDtypeStruct(lead + (n_pre,), jnp.float32)
    y, _ = jffi.ffi_call('bsx_ffi_matvec', (out, _scratch(ws)), vmap_method='broadcast_all')(
        spk_post, idx, ip, w, n_pre=np.int64(n_pre), event=True)
    return y


def dense_event_vecmat(spk, weight):
    """``EventArray(spk) @ W`` for a dense ``W`` (``brainstate/nn/_event_linear.py:99-100``)."""
    register()
    out = jax.ShapeDtypeStruct(spk.shape[:-1] + (weight.shape[1],), jnp.float32)
    return jffi.ffi_call('bsx_ffi_dense_event_vecmat', out, vmap_method='broadcast_all')(spk, jnp.asarray(weight, jnp.float32))
