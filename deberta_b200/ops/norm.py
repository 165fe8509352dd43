"""LayerNorm and RMSNorm with fp32 statistics (``csrc/norm.cu`` on bf16 CUDA tensors)."""

from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

__all__ = ["layer_norm", "rms_norm", "layer_norm_reference", "rms_norm_reference"]


def layer_norm_reference(x, weight, bias, eps, row_keep=None):
    y = F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)
    if row_keep is not None:
        y = y * row_keep.unsqueeze(-1).to(y.dtype)
    return y.to(x.dtype)


def rms_norm_reference(x, weight, eps, row_keep=None):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.float()
    if row_keep is not None:
        y = y * row_keep.unsqueeze(-1).to(y.dtype)
    return y.to(x.dtype)


def _kernel_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (
        x.is_cuda
        and x.dtype == torch.bfloat16
        and weight.dtype == torch.bfloat16
        and x.shape[-1] % 8 == 0
        and x.shape[-1] <= 2048
    )


def norm_forward(x, weight, bias, row_keep, eps: float, rms: bool):
    """(y, mean, rstd) of ``x`` [rows, H]; ``mean`` is empty for RMSNorm. Kernel on bf16 CUDA, PyTorch otherwise."""
    rows, H = x.shape
    if _kernel_ok(x, weight):
        y = torch.empty_like(x)
        mean = torch.empty(0 if rms else rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        keep = None if row_keep is None else row_keep.to(torch.uint8).contiguous()
        _lib.call(
            "db200_norm_fwd", _lib.ptr(x), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(keep), _lib.ptr(y),
            _lib.ptr(None if rms else mean), _lib.ptr(rstd), ctypes.c_int(rows), ctypes.c_int(H), ctypes.c_float(eps),
            ctypes.c_int(int(rms)), _lib.stream_ptr(),
        )
        return y, mean, rstd
    xf = x.float()
    if rms:
        mean = torch.empty(0, dtype=torch.float32, device=x.device)
        rstd = torch.rsqrt(xf.pow(2).mean(dim=-1) + eps)
        y = xf * rstd[:, None] * weight.float()
    else:
        mean = xf.mean(dim=-1)
        rstd = torch.rsqrt(xf.var(dim=-1, unbiased=False) + eps)
        y = (xf - mean[:, None]) * rstd[:, None] * weight.float()
        if bias is not None:
            y = y + bias.float()
    if row_keep is not None:
        y = y * row_keep.reshape(-1, 1).to(y.dtype)
    return y.to(x.dtype), mean, rstd


def norm_backward(dy, x, weight, mean, rstd, row_keep, rms: bool, has_bias: bool, w_grad, b_grad):
    """(dx, dgamma, dbeta): a parameter gradient that was added to its fp32 buffer (``w_grad`` / ``b_grad``) is ``None``."""
    rows, H = x.shape
    dy = dy.contiguous()
    if _kernel_ok(x, weight):
        dx = torch.empty_like(x)
        dg = w_grad if w_grad is not None else torch.zeros(H, dtype=torch.float32, device=x.device)
        db = None
        if has_bias:
            db = b_grad if b_grad is not None else torch.zeros(H, dtype=torch.float32, device=x.device)
        keep = None if row_keep is None else row_keep.to(torch.uint8).contiguous()
        _lib.call(
            "db200_norm_bwd", _lib.ptr(dy), _lib.ptr(x), _lib.ptr(weight), _lib.ptr(None if rms else mean), _lib.ptr(rstd),
            _lib.ptr(keep), _lib.ptr(dx), _lib.ptr(dg), _lib.ptr(db), ctypes.c_int(rows), ctypes.c_int(H),
            ctypes.c_int(int(rms)), _lib.stream_ptr(),
        )
        return (dx, None if w_grad is not None else dg.to(weight.dtype),
                None if (db is None or b_grad is not None) else db.to(weight.dtype))
    dyf, xf, g = dy.float(), x.float(), weight.float()
    if row_keep is not None:
        dyf = dyf * row_keep.reshape(-1, 1).to(dyf.dtype)
    xhat = xf * rstd[:, None] if rms else (xf - mean[:, None]) * rstd[:, None]
    dgamma = (dyf * xhat).sum(0)
    dbeta = dyf.sum(0) if has_bias else None
    dxhat = dyf * g
    if rms:
        dx = rstd[:, None] * (dxhat - xhat * (dxhat * xhat).mean(dim=-1, keepdim=True))
    else:
        dx = rstd[:, None] * (dxhat - dxhat.mean(dim=-1, keepdim=True) - xhat * (dxhat * xhat).mean(dim=-1, keepdim=True))
    if w_grad is not None:
        w_grad.add_(dgamma)
        dgamma = None
    if dbeta is not None and b_grad is not None:
        b_grad.add_(dbeta)
        dbeta = None
    return (dx.to(x.dtype), None if dgamma is None else dgamma.to(weight.dtype),
            None if dbeta is None else dbeta.to(weight.dtype))


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms, row_keep):
        keep = None if row_keep is None else row_keep.to(torch.uint8).contiguous()
        y, mean, rstd = norm_forward(x, weight, bias, keep, eps, rms)
        ctx.save_for_backward(x, mean, rstd, keep)
        ctx.refs = (weight, bias)
        ctx.rms = rms
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd, keep = ctx.saved_tensors
        weight, bias = ctx.refs
        has_bias = bias is not None and bias.requires_grad
        w_grad = getattr(weight, "main_grad", None) if weight.requires_grad else None
        b_grad = getattr(bias, "main_grad", None) if has_bias else None
        dx, gw, gb = norm_backward(dy, x, weight, mean, rstd, keep, ctx.rms, has_bias, w_grad, b_grad)
        return dx, (gw if weight.requires_grad else None), gb, None, None, None


def _norm_apply(x2, weight, bias, eps: float, rms: bool, rk):
    if torch.compiler.is_compiling():
        from . import library

        # (no gradient buffers under a compiler: see ops/linear.py:linear)
        return library.norm(x2, weight, bias, rk, float(eps), rms, None, None)[0]
    return _Norm.apply(x2, weight, bias, float(eps), rms, rk)


def layer_norm(x, weight, bias, eps: float, row_keep: torch.Tensor | None = None):
    """LayerNorm over the last dim; ``row_keep`` (bool per row) zeroes whole output rows."""
    if not _kernel_ok(x, weight):
        return layer_norm_reference(x, weight, bias, eps, row_keep)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    rk = None if row_keep is None else row_keep.reshape(-1)
    return _norm_apply(x2, weight, bias, eps, False, rk).view(*lead, x.shape[-1])


def rms_norm(x, weight, eps: float, row_keep: torch.Tensor | None = None):
    """RMSNorm ``x * rsqrt(mean(x^2) + eps) * weight`` with fp32 reduction."""
    if not _kernel_ok(x, weight):
        return rms_norm_reference(x, weight, eps, row_keep)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    rk = None if row_keep is None else row_keep.reshape(-1)
    return _norm_apply(x2, weight, None, eps, True, rk).view(*lead, x.shape[-1])
