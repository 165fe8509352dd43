"""Masked-row gather ``x[idx]`` over token rows and its gradient (``csrc/elementwise.cu``).

The generator's head only sees the masked positions (``modeling/rtd.py:1061-1065`` of the reference gathers them with
``index_select``). On bf16 CUDA tensors the forward is one copy kernel that also records the inverse map, and the
backward writes every row of the gradient exactly once (selected rows get their gradient, the others zeros), so no
zero-filled ``[tokens, hidden]`` tensor and no ``index_add`` pass exist. Elsewhere it is ``index_select``.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

__all__ = ["gather_rows"]


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx):
        M, H = x.shape
        idx = idx.to(torch.int64).contiguous()
        out = torch.empty((idx.numel(), H), dtype=x.dtype, device=x.device)
        inv = torch.empty(M, dtype=torch.int32, device=x.device)
        _lib.call("db200_rows_gather", _lib.ptr(x), ctypes.c_longlong(x.stride(0)), _lib.ptr(idx), _lib.ptr(out),
                  _lib.ptr(inv), ctypes.c_longlong(M), ctypes.c_longlong(idx.numel()), ctypes.c_int(H), _lib.stream_ptr())
        ctx.save_for_backward(inv)
        ctx.shape = (M, H)
        return out

    @staticmethod
    def backward(ctx, dout):
        (inv,) = ctx.saved_tensors
        M, H = ctx.shape
        if dout.stride(-1) != 1 or dout.stride(0) % 8 or dout.data_ptr() % 16:
            dout = dout.contiguous()
        dx = torch.empty((M, H), dtype=dout.dtype, device=dout.device)
        _lib.call("db200_rows_scatter", _lib.ptr(dout), ctypes.c_longlong(dout.stride(0)), _lib.ptr(inv), _lib.ptr(dx),
                  ctypes.c_longlong(M), ctypes.c_int(H), _lib.stream_ptr())
        return dx, None


def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``x[idx]`` for a 2-D ``x`` and distinct row indices ``idx`` (the masked positions of a batch)."""
    ok = (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 8 == 0 and x.stride(1) == 1
          and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and not torch.compiler.is_compiling())
    if not ok:
        return x.index_select(0, idx)
    return _GatherRows.apply(x, idx)
