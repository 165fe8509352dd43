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


def embed_forward(ids, table, delta):
    """``table[ids] (+ delta[ids])``: one kernel on bf16 CUDA tables, ``F.embedding`` otherwise."""
    if table.is_cuda and table.dtype == torch.bfloat16:
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        vocab, hidden = table.shape
        out = torch.empty((flat.numel(), hidden), dtype=table.dtype, device=table.device)
        _lib.call("db200_embed_fwd", _lib.ptr(flat), _lib.ptr(table), _lib.ptr(delta), _lib.ptr(out),
                  ctypes.c_longlong(flat.numel()), ctypes.c_int(hidden), ctypes.c_longlong(vocab), _lib.stream_ptr())
        return out.view(*ids.shape, hidden)
    out = F.embedding(ids, table)
    return out if delta is None else out + F.embedding(ids, delta)


def embed_backward(dout, ids, vocab: int, padding_idx: int, grads) -> None:
    """Add the rows of ``dout`` to row ``ids[t]`` of every fp32 buffer in ``grads`` (``None`` entries skipped)."""
    d2 = dout.reshape(-1, dout.shape[-1])
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    if d2.is_cuda and d2.dtype == torch.bfloat16:
        if d2.stride(-1) != 1 or d2.stride(0) % 8 or d2.data_ptr() % 16:
            d2 = d2.contiguous()
        for g in grads:
            if g is not None:
                _lib.call("db200_embed_bwd", _lib.ptr(flat), _lib.ptr(d2), ctypes.c_longlong(d2.stride(0)), _lib.ptr(g),
                          ctypes.c_longlong(flat.numel()), ctypes.c_int(d2.shape[1]), ctypes.c_longlong(vocab),
                          ctypes.c_longlong(int(padding_idx)), _lib.stream_ptr())
        return
    rows = d2.float()
    if padding_idx >= 0:
        rows = rows * flat.ne(padding_idx).unsqueeze(-1).to(rows.dtype)
    for g in grads:
        if g is not None:
            g.index_add_(0, flat, rows.to(g.dtype))


class _Embed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, delta, padding_idx):
        ctx.ids, ctx.tables, ctx.padding_idx = ids, (table, delta), padding_idx
        return embed_forward(ids, table, delta)

    @staticmethod
    def backward(ctx, dout):
        pad = -1 if ctx.padding_idx is None else int(ctx.padding_idx)
        grads = [t.main_grad if (t is not None and t.requires_grad) else None for t in ctx.tables]
        embed_backward(dout, ctx.ids, ctx.tables[0].shape[0], pad, grads)
        return None, None, None, None


def embedding_lookup(ids: torch.Tensor, table: torch.Tensor, delta: torch.Tensor | None = None,
                     padding_idx: int | None = None) -> torch.Tensor:
    """``table[ids] (+ delta[ids])``; gradients of trainable tables go to their ``main_grad`` on the kernel path."""
    # Under a compiler the lookup is F.embedding (the kernel path scatters into the engine's gradient buffers, and ops that
    # mutate views of the flat gradient storage do not go into a compiled graph: see ops/linear.py:linear).
    if _usable(table) and _usable(delta) and table.is_cuda and _grad_ready(table) and _grad_ready(delta) and \
            (delta is None or delta.shape == table.shape) and not torch.compiler.is_compiling():
        if torch.is_grad_enabled() and (table.requires_grad or (delta is not None and delta.requires_grad)):
            return _Embed.apply(ids, table, delta, padding_idx)
        return embed_forward(ids, table, delta)
    out = F.embedding(ids, table, padding_idx=padding_idx)
    if delta is not None:
        out = out + F.embedding(ids, delta, padding_idx=padding_idx)
    return out
