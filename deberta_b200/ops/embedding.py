"""Embedding lookup with an optional second (delta) table, and its gradient scatter.

Covers the plain word-embedding gather and the gradient-disentangled form ``base[ids] + delta[ids]`` of the
reference (``modeling/rtd.py:157-226``) in one kernel; the backward adds the output gradient rows straight into the
fp32 ``main_grad`` buffers of the trainable tables (no dense ``[vocab, hidden]`` gradient tensor, no sort). Without a
GPU, without ``main_grad`` buffers, or for other dtypes it is ``F.embedding``.
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

__all__ = ["embedding_lookup"]


def _usable(table: torch.Tensor | None) -> bool:
    return table is None or (table.is_cuda and table.dtype == torch.bfloat16 and table.is_contiguous()
                             and table.shape[1] % 8 == 0)


def _grad_ready(table: torch.Tensor | None) -> bool:
    """Frozen tables need nothing; trainable ones need the engine's fp32 gradient buffer."""
    if table is None or not table.requires_grad:
        return True
    g = getattr(table, "main_grad", None)
    return g is not None and g.dtype == torch.float32 and g.is_contiguous()


class _Embed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, delta, padding_idx):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        vocab, hidden = table.shape
        out = torch.empty((flat.numel(), hidden), dtype=table.dtype, device=table.device)
        _lib.call("db200_embed_fwd", _lib.ptr(flat), _lib.ptr(table), _lib.ptr(delta), _lib.ptr(out),
                  ctypes.c_longlong(flat.numel()), ctypes.c_int(hidden), ctypes.c_longlong(vocab), _lib.stream_ptr())
        ctx.ids, ctx.tables, ctx.padding_idx = flat, (table, delta), padding_idx
        return out.view(*ids.shape, hidden)

    @staticmethod
    def backward(ctx, dout):
        d2 = dout.reshape(-1, dout.shape[-1])
        if d2.stride(-1) != 1 or d2.stride(0) % 8 or d2.data_ptr() % 16:
            d2 = d2.contiguous()
        pad = -1 if ctx.padding_idx is None else int(ctx.padding_idx)
        for table in ctx.tables:
            if table is None or not table.requires_grad:
                continue
            vocab, hidden = table.shape
            _lib.call("db200_embed_bwd", _lib.ptr(ctx.ids), _lib.ptr(d2), ctypes.c_longlong(d2.stride(0)),
                      _lib.ptr(table.main_grad), ctypes.c_longlong(ctx.ids.numel()), ctypes.c_int(hidden),
                      ctypes.c_longlong(vocab), ctypes.c_longlong(pad), _lib.stream_ptr())
        return None, None, None, None


def embedding_lookup(ids: torch.Tensor, table: torch.Tensor, delta: torch.Tensor | None = None,
                     padding_idx: int | None = None) -> torch.Tensor:
    """``table[ids] (+ delta[ids])``; gradients of trainable tables go to their ``main_grad`` on the kernel path."""
    if _usable(table) and _usable(delta) and table.is_cuda and _grad_ready(table) and _grad_ready(delta) and \
            (delta is None or delta.shape == table.shape):
        if torch.is_grad_enabled() and (table.requires_grad or (delta is not None and delta.requires_grad)):
            return _Embed.apply(ids, table, delta, padding_idx)
        return _Embed.forward(_NoCtx(), ids, table, delta, padding_idx)
    out = F.embedding(ids, table, padding_idx=padding_idx)
    if delta is not None:
        out = out + F.embedding(ids, delta, padding_idx=padding_idx)
    return out


class _NoCtx:
    """Stand-in context for calling the forward outside autograd."""
