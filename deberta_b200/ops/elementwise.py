"""Fused elementwise operators of the RoPE backbone: rotary embedding and the SwiGLU gate.

On bf16 CUDA tensors they run on ``csrc/elementwise.cu`` (one pass each, forward and backward); everywhere else
they are the PyTorch compositions the reference uses (``modeling/rope.py:145-174``, ``modeling/rope_encoder.py:290-343``),
which are also the oracles of the GPU tests.
"""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

__all__ = ["rotary_tokens", "swiglu"]


def _kernel_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _rows_view(x: torch.Tensor) -> torch.Tensor:
    """[..., H] → [rows, H] with unit inner stride and a row stride that is a multiple of 8 (else a copy)."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    return x2


class _Rotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, heads, rotary_dim):
        B, S, H = x.shape
        x2 = _rows_view(x)
        y = torch.empty((B * S, H), dtype=x.dtype, device=x.device)
        _lib.call("db200_rotary_bf16", _lib.ptr(x2), _lib.ptr(y), ctypes.c_longlong(x2.stride(0)), ctypes.c_longlong(H),
                  _lib.ptr(cos), _lib.ptr(sin), ctypes.c_longlong(B * S), ctypes.c_int(S), ctypes.c_int(heads),
                  ctypes.c_int(H // heads), ctypes.c_int(rotary_dim), ctypes.c_int(0), _lib.stream_ptr())
        ctx.save_for_backward(cos, sin)
        ctx.meta = (B, S, H, heads, rotary_dim)
        return y.view(B, S, H)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        B, S, H, heads, rotary_dim = ctx.meta
        d2 = _rows_view(dy)
        dx = torch.empty((B * S, H), dtype=dy.dtype, device=dy.device)
        _lib.call("db200_rotary_bf16", _lib.ptr(d2), _lib.ptr(dx), ctypes.c_longlong(d2.stride(0)), ctypes.c_longlong(H),
                  _lib.ptr(cos), _lib.ptr(sin), ctypes.c_longlong(B * S), ctypes.c_int(S), ctypes.c_int(heads),
                  ctypes.c_int(H // heads), ctypes.c_int(rotary_dim), ctypes.c_int(1), _lib.stream_ptr())
        return dx.view(B, S, H), None, None, None, None


def rotary_tokens(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, heads: int, rotary_dim: int) -> torch.Tensor:
    """Interleaved-pair rotary embedding of a token-major ``[B, S, heads*d]`` tensor.

    ``cos`` / ``sin``: ``[S, rotary_dim]`` with every frequency repeated twice (the model's rotary cache).
    """
    if rotary_dim <= 0:
        return x
    B, S, H = x.shape
    d = H // heads
    if _kernel_ok(x) and d % 8 == 0 and rotary_dim % 2 == 0:
        c = cos.detach().to(torch.float32).contiguous()
        s = sin.detach().to(torch.float32).contiguous()
        return _Rotary.apply(x, c, s, heads, rotary_dim)
    from .attention import rotate_interleaved

    c, s = cos.to(x.dtype)[None, :, None, :], sin.to(x.dtype)[None, :, None, :]
    return rotate_interleaved(x.reshape(B, S, heads, d), c, s, rotary_dim).reshape(B, S, H)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        rows, two_f = gu.shape
        f = two_f // 2
        out = torch.empty((rows, f), dtype=gu.dtype, device=gu.device)
        _lib.call("db200_swiglu_fwd", _lib.ptr(gu), ctypes.c_longlong(gu.stride(0)), _lib.ptr(out), ctypes.c_longlong(f),
                  ctypes.c_longlong(rows), ctypes.c_int(f), _lib.stream_ptr())
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        rows, two_f = gu.shape
        f = two_f // 2
        d2 = _rows_view(dout)
        dgu = torch.empty((rows, two_f), dtype=gu.dtype, device=gu.device)
        _lib.call("db200_swiglu_bwd", _lib.ptr(gu), ctypes.c_longlong(gu.stride(0)), _lib.ptr(d2),
                  ctypes.c_longlong(d2.stride(0)), _lib.ptr(dgu), ctypes.c_longlong(two_f), ctypes.c_longlong(rows),
                  ctypes.c_int(f), _lib.stream_ptr())
        return dgu


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    f = gate_up.shape[-1] // 2
    if _kernel_ok(gate_up) and f % 8 == 0 and gate_up.shape[-1] == 2 * f:
        lead = gate_up.shape[:-1]
        return _SwiGLU.apply(_rows_view(gate_up)).view(*lead, f)
    gate, up = gate_up.chunk(2, dim=-1)
    return F.silu(gate) * up
