"""Linear layers and the fused GELU feed-forward block on the tcgen05 GEMM.

On bf16 CUDA tensors every product (forward, data gradient, weight gradient) runs on
``csrc/gemm.cu`` with the bias / residual / GELU / GELU-derivative work folded into the
GEMM epilogues. Weight and bias gradients are accumulated in fp32 directly into
``param.main_grad`` when the engine attached one (so micro-batch accumulation costs no
extra pass); otherwise they are returned to autograd. Everything else (CPU, fp32)
takes the plain PyTorch path, which is also the oracle for the GPU tests.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .gemm import EPI_DGELU, EPI_GELU, gemm

__all__ = ["linear", "ffn_gelu", "use_kernels"]


def use_kernels(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _weight_grad(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor | None:
    """dW[out,in] = dyᵀ·x, accumulated into ``w.main_grad`` when present."""
    main = getattr(w, "main_grad", None)
    if main is not None:
        gemm(dy, x, a_mn=True, b_mn=True, out=main, accumulate=True)
        return None
    return gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)


def colsum_into(dy: torch.Tensor, out: torch.Tensor) -> None:
    """``out[n] += Σ_m dy[m, n]`` (bf16 in, fp32 accumulate) on the column-sum kernel."""
    import ctypes

    from . import _lib

    _lib.call("db200_colsum_bf16", _lib.ptr(dy), ctypes.c_longlong(dy.stride(0)), ctypes.c_int(dy.shape[0]),
              ctypes.c_int(dy.shape[1]), _lib.ptr(out), _lib.stream_ptr())


def _bias_grad(dy: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor | None:
    if b is None:
        return None
    main = getattr(b, "main_grad", None)
    kernel_ok = dy.is_cuda and dy.dtype == torch.bfloat16 and dy.stride(1) == 1 and dy.stride(0) % 8 == 0 and dy.data_ptr() % 16 == 0
    if main is not None and kernel_ok:
        colsum_into(dy, main)
        return None
    if kernel_ok:
        g = torch.zeros(dy.shape[1], dtype=torch.float32, device=dy.device)
        colsum_into(dy, g)
    else:
        g = dy.sum(dim=0, dtype=torch.float32)
    if main is not None:
        main.add_(g)
        return None
    return g.to(b.dtype)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual):
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None
        ctx.bias_ref = b
        ctx.has_res = residual is not None
        return gemm(x, w, bias=b, residual=residual)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _weight_grad(dy, x, w) if w.requires_grad else None
        db = _bias_grad(dy, ctx.bias_ref) if (ctx.has_bias and ctx.bias_ref.requires_grad) else None
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


def linear(
    x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None, residual: torch.Tensor | None = None
) -> torch.Tensor:
    """``x @ wᵀ + b (+ residual)`` over the last dim of ``x`` (any leading shape)."""
    if not (use_kernels(x) and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0):
        out = F.linear(x, w.to(x.dtype) if w.dtype != x.dtype else w, None if b is None else b.to(x.dtype))
        return out if residual is None else out + residual
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    r2 = None if residual is None else residual.reshape(-1, w.shape[0]).contiguous()
    out = _Linear.apply(x2, w, b, r2)
    return out.view(*lead, w.shape[0])


class _FFNGelu(torch.autograd.Function):
    """y = W2·gelu(W1·x + b1) + b2 + residual, with dGELU fused into the W2 data-gradient GEMM."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        z, a = gemm(x, w1, bias=b1, epi=EPI_GELU)
        y = gemm(a, w2, bias=b2, residual=residual)
        ctx.save_for_backward(x, w1, w2, z, a)
        ctx.params = (b1, b2)
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w1, w2, z, a = ctx.saved_tensors
        b1, b2 = ctx.params
        dy = dy.contiguous()
        dz = gemm(dy, w2, b_mn=True, epi=EPI_DGELU, aux=z)
        dw2 = _weight_grad(dy, a, w2) if w2.requires_grad else None
        db2 = _bias_grad(dy, b2) if (b2 is not None and b2.requires_grad) else None
        dx = gemm(dz, w1, b_mn=True) if ctx.needs_input_grad[0] else None
        dw1 = _weight_grad(dz, x, w1) if w1.requires_grad else None
        db1 = _bias_grad(dz, b1) if (b1 is not None and b1.requires_grad) else None
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None)


def ffn_gelu(x, w1, b1, w2, b2, residual=None):
    """Feed-forward block with exact-erf GELU: ``W2·gelu(W1·x+b1)+b2 (+residual)``."""
    if not (use_kernels(x) and w1.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w1.shape[0] % 8 == 0):
        h = F.gelu(F.linear(x, w1.to(x.dtype), None if b1 is None else b1.to(x.dtype)))
        out = F.linear(h, w2.to(x.dtype), None if b2 is None else b2.to(x.dtype))
        return out if residual is None else out + residual
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    r2 = None if residual is None else residual.reshape(-1, w2.shape[0]).contiguous()
    out = _FFNGelu.apply(x2, w1, b1, w2, b2, r2)
    return out.view(*lead, w2.shape[0])
