"""Event products for batches that live in host memory.

A caller that keeps its spike vectors and results in (pinned) host memory pays
for two PCIe crossings per batch.  ``HostEventProducts`` hides them behind the
kernels: the batch is cut into chunks, and three CUDA streams run the upload of
chunk ``c+1``, the products of chunk ``c`` and the download of chunk ``c-1`` at
the same time.  The arithmetic is the same library calls as the device-resident
path (``bsx_event_vecmat``, ``bsx_event_matvec``); nothing is computed on the host.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import check, lib

__all__ = ['HostEventProducts']


class HostEventProducts:
    """``y_fwd = EventArray(spk) @ conn`` and/or ``y_rev = conn @ EventArray(spk)`` for
    ``spk`` of shape ``(T, n)`` in pinned host memory, results written to pinned
    host memory.  Requires a square connectivity when both products are asked for.

    chunk : vectors per pipeline stage (16 = one pass of the batched gather).
    reverse_method : ``'gather'`` (deterministic, rate-independent cost) or ``'scatter'``
        (event-driven over the transposed copy; the faster one below about 3 % firing).
    """

    def __init__(self, conn, chunk: int = 16, forward: bool = True, reverse: bool = True, slots: int = 3,
                 reverse_method: str = 'gather'):
        if reverse_method not in ('gather', 'scatter'):
            raise ValueError(f"reverse_method must be 'gather' or 'scatter', got {reverse_method!r}")
        self.reverse_method = reverse_method
        self.conn = conn
        self.chunk = int(chunk)
        self.forward, self.reverse = forward, reverse
        n_pre, n_post = conn.shape
        if forward and reverse and n_pre != n_post:
            raise ValueError('both products of one spike batch need a square connectivity')
        self.n_in = n_pre if forward else n_post
        dev = conn.indices.device
        self.dev = dev
        self.slots = slots
        l = lib()
        self.s_in, self.s_comp, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.spk = [torch.empty((self.chunk, self.n_in), dtype=torch.bool, device=dev) for _ in range(slots)]
        self.y_fwd = [torch.empty((self.chunk, n_post), dtype=torch.float32, device=dev) for _ in range(slots)] if forward else None
        self.y_rev = [torch.empty((self.chunk, n_pre), dtype=torch.float32, device=dev) for _ in range(slots)] if reverse else None
        self.ws_f_bytes = l.bsx_event_vecmat_workspace_bytes(self.chunk, n_pre)
        if reverse and reverse_method == 'scatter':
            self.st_t = conn._transposed_struct(conn.data)
            self.ws_r_bytes = l.bsx_event_vecmat_workspace_bytes(self.chunk, n_post)
        else:
            self.ws_r_bytes = l.bsx_event_matvec_workspace_bytes(self.chunk, n_post)
        self.ws_f = torch.empty(max(self.ws_f_bytes, 1), dtype=torch.uint8, device=dev)   # compute is serial: one set
        self.ws_r = torch.empty(max(self.ws_r_bytes, 1), dtype=torch.uint8, device=dev)
        self.st = conn._struct()
        # chunks that fill the GPU run the scatter over the copies grouped by output slice
        self.sliced = l.bsx_event_vecmat_variant(C.byref(self.st), _lib.SPK_BOOL8, self.chunk) == _lib.VECMAT_SHARED_SLICES
        self.scale_f = self.scale_t = None
        if self.sliced:
            self.st_f = conn._sliced_struct(conn.data) if forward else None
            if reverse and reverse_method == 'scatter':
                self.st_t = conn._transposed_sliced_struct(conn.data)
            if conn.hetero:     # heterogeneous weights: fixed-point sums (order-free, faster than float atomics)
                self.scale_f = conn._fixed_scale('s', self.st_f, conn.data) if forward else None
                self.scale_t = (conn._fixed_scale('ts', self.st_t, conn.data)
                                if reverse and reverse_method == 'scatter' else None)
            from . import event as _event
            if _event.PACKED_SLICES:       # the compressed copies are built here, not inside the first call
                if forward:
                    conn._packed('s', self.st_f, conn.data, self.scale_f or 0)
                if reverse and reverse_method == 'scatter':
                    conn._packed('ts', self.st_t, conn.data, self.scale_t or 0)

    def __call__(self, spk_host: torch.Tensor, y_fwd_host: Optional[torch.Tensor] = None,
                 y_rev_host: Optional[torch.Tensor] = None):
        if not spk_host.is_pinned():
            raise ValueError('spk_host must be pinned host memory (tensor.pin_memory())')
        if spk_host.dtype != torch.bool or spk_host.dim() != 2 or spk_host.shape[1] != self.n_in:
            raise ValueError(f'spk_host must be bool of shape (T, {self.n_in})')
        if self.forward and (y_fwd_host is None or not y_fwd_host.is_pinned()):
            raise ValueError('y_fwd_host must be a pinned float32 host tensor')
        if self.reverse and (y_rev_host is None or not y_rev_host.is_pinned()):
            raise ValueError('y_rev_host must be a pinned float32 host tensor')
        l = lib()
        T = spk_host.shape[0]
        n_chunks = (T + self.chunk - 1) // self.chunk
        cur = torch.cuda.current_stream(self.dev)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        ev_in = [torch.cuda.Event() for _ in range(n_chunks)]
        ev_comp = [torch.cuda.Event() for _ in range(n_chunks)]
        ev_out = [torch.cuda.Event() for _ in range(n_chunks)]
        for c in range(n_chunks):
            lo, hi = c * self.chunk, min(T, (c + 1) * self.chunk)
            nb, slot = hi - lo, c % self.slots
            with torch.cuda.stream(self.s_in):
                if c >= self.slots:
                    self.s_in.wait_event(ev_comp[c - self.slots])      # the slot's spikes were consumed
                self.spk[slot][:nb].copy_(spk_host[lo:hi], non_blocking=True)
                ev_in[c].record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(ev_in[c])
                if c >= self.slots:
                    self.s_comp.wait_event(ev_out[c - self.slots])     # the slot's results were downloaded
                stream = self.s_comp.cuda_stream
                if self.forward and self.sliced:
                    self.conn._sliced_call('s', self.st_f, self.conn.data, self.scale_f, self.spk[slot], _lib.SPK_BOOL8,
                                           nb, self.y_fwd[slot], False)
                elif self.forward:
                    check(l.bsx_event_vecmat(C.byref(self.st), self.spk[slot].data_ptr(), _lib.SPK_BOOL8, nb,
                                             self.y_fwd[slot].data_ptr(), 0, self.ws_f.data_ptr(), self.ws_f_bytes,
                                             stream))
                if self.reverse and self.reverse_method == 'scatter' and self.sliced:
                    self.conn._sliced_call('ts', self.st_t, self.conn.data, self.scale_t, self.spk[slot],
                                           _lib.SPK_BOOL8, nb, self.y_rev[slot], False)
                elif self.reverse and self.reverse_method == 'scatter':
                    check(l.bsx_event_vecmat(C.byref(self.st_t), self.spk[slot].data_ptr(), _lib.SPK_BOOL8, nb,
                                             self.y_rev[slot].data_ptr(), 0, self.ws_r.data_ptr(), self.ws_r_bytes,
                                             stream))
                elif self.reverse:
                    check(l.bsx_event_matvec(C.byref(self.st), self.spk[slot].data_ptr(), _lib.SPK_BOOL8, nb,
                                             self.y_rev[slot].data_ptr(), self.ws_r.data_ptr(), self.ws_r_bytes,
                                             stream))
                ev_comp[c].record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_comp[c])
                if self.forward:
                    y_fwd_host[lo:hi].copy_(self.y_fwd[slot][:nb], non_blocking=True)
                if self.reverse:
                    y_rev_host[lo:hi].copy_(self.y_rev[slot][:nb], non_blocking=True)
                ev_out[c].record(self.s_out)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_comp)
        cur.wait_stream(self.s_in)
        return y_fwd_host, y_rev_host
