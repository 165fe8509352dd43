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


def rotary_apply(x, cos, sin, heads: int, rotary_dim: int, inverse: bool):
    """Rotate (``inverse``: rotate back, i.e. the gradient of the rotation) a token-major ``[B, S, H]`` tensor."""
    B, S, H = x.shape
    if _kernel_ok(x):
        x2 = _rows_view(x)
        y = torch.empty((B * S, H), dtype=x.dtype, device=x.device)
        _lib.call("db200_rotary_bf16", _lib.ptr(x2), _lib.ptr(y), ctypes.c_longlong(x2.stride(0)), ctypes.c_longlong(H),
                  _lib.ptr(cos), _lib.ptr(sin), ctypes.c_longlong(B * S), ctypes.c_int(S), ctypes.c_int(heads),
                  ctypes.c_int(H // heads), ctypes.c_int(rotary_dim), ctypes.c_int(int(inverse)), _lib.stream_ptr())
        return y.view(B, S, H)
    from .attention import rotate_interleaved

    d = H // heads
    c = cos.to(x.dtype)[None, :, None, :]
    s = (-sin if inverse else sin).to(x.dtype)[None, :, None, :]
    return rotate_interleaved(x.reshape(B, S, heads, d), c, s, rotary_dim).reshape(B, S, H)


class _Rotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, heads, rotary_dim):
        ctx.save_for_backward(cos, sin)
        ctx.meta = (heads, rotary_dim)
        return rotary_apply(x, cos, sin, heads, rotary_dim, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        heads, rotary_dim = ctx.meta
        return rotary_apply(dy, cos, sin, heads, rotary_dim, True), None, None, None, None


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
        if torch.compiler.is_compiling():
            from . import library

            return library.rotary(x, c, s, heads, rotary_dim, False)
        return _Rotary.apply(x, c, s, heads, rotary_dim)
    from .attention import rotate_interleaved

    c, s = cos.to(x.dtype)[None, :, None, :], sin.to(x.dtype)[None, :, None, :]
    return rotate_interleaved(x.reshape(B, S, heads, d), c, s, rotary_dim).reshape(B, S, H)


def swiglu_forward(gu):
    rows, two_f = gu.shape
    f = two_f // 2
    if _kernel_ok(gu):
        out = torch.empty((rows, f), dtype=gu.dtype, device=gu.device)
        _lib.call("db200_swiglu_fwd", _lib.ptr(gu), ctypes.c_longlong(gu.stride(0)), _lib.ptr(out), ctypes.c_longlong(f),
                  ctypes.c_longlong(rows), ctypes.c_int(f), _lib.stream_ptr())
        return out
    return F.silu(gu[:, :f]) * gu[:, f:]


def swiglu_backward(gu, dout):
    rows, two_f = gu.shape
    f = two_f // 2
    if _kernel_ok(gu):
        d2 = _rows_view(dout)
        dgu = torch.empty((rows, two_f), dtype=gu.dtype, device=gu.device)
        _lib.call("db200_swiglu_bwd", _lib.ptr(gu), ctypes.c_longlong(gu.stride(0)), _lib.ptr(d2),
                  ctypes.c_longlong(d2.stride(0)), _lib.ptr(dgu), ctypes.c_longlong(two_f), ctypes.c_longlong(rows),
                  ctypes.c_int(f), _lib.stream_ptr())
        return dgu
    gate, up = gu[:, :f].float(), gu[:, f:].float()
    sig = torch.sigmoid(gate)
    d = dout.float()
    return torch.cat([d * up * sig * (1 + gate * (1 - sig)), d * gate * sig], dim=-1).to(gu.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return swiglu_forward(gu)

    @staticmethod
    def backward(ctx, dout):
        return swiglu_backward(ctx.saved_tensors[0], dout)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    f = gate_up.shape[-1] // 2
    if _kernel_ok(gate_up) and f % 8 == 0 and gate_up.shape[-1] == 2 * f:
        lead = gate_up.shape[:-1]
        if torch.compiler.is_compiling():
            from . import library

            return library.swiglu(_rows_view(gate_up)).view(*lead, f)
        return _SwiGLU.apply(_rows_view(gate_up)).view(*lead, f)
    gate, up = gate_up.chunk(2, dim=-1)
    return F.silu(gate) * up
