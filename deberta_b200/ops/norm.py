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


def _grad_target(p: torch.Tensor | None):
    """(buffer to accumulate into, whether it is the engine's main_grad)."""
    if p is None:
        return None, False
    main = getattr(p, "main_grad", None)
    if main is not None:
        return main, True
    return torch.zeros(p.shape, dtype=torch.float32, device=p.device), False


class _Norm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms, row_keep):
        rows, H = x.shape
        y = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if not rms else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        keep = None if row_keep is None else row_keep.to(torch.uint8).contiguous()
        _lib.call(
            "db200_norm_fwd", _lib.ptr(x), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(keep), _lib.ptr(y),
            _lib.ptr(mean), _lib.ptr(rstd), ctypes.c_int(rows), ctypes.c_int(H), ctypes.c_float(eps),
            ctypes.c_int(int(rms)), _lib.stream_ptr(),
        )
        ctx.save_for_backward(x, mean, rstd, keep)
        ctx.refs = (weight, bias)
        ctx.rms = rms
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd, keep = ctx.saved_tensors
        weight, bias = ctx.refs
        rows, H = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dg, g_main = _grad_target(weight if weight.requires_grad else None)
        db, b_main = _grad_target(bias if (bias is not None and bias.requires_grad) else None)
        if dg is None:  # kernel always needs somewhere to put the weight gradient
            dg = torch.zeros(H, dtype=torch.float32, device=x.device)
        _lib.call(
            "db200_norm_bwd", _lib.ptr(dy), _lib.ptr(x), _lib.ptr(weight), _lib.ptr(mean), _lib.ptr(rstd),
            _lib.ptr(keep), _lib.ptr(dx), _lib.ptr(dg), _lib.ptr(db), ctypes.c_int(rows), ctypes.c_int(H),
            ctypes.c_int(int(ctx.rms)), _lib.stream_ptr(),
        )
        gw = None if (g_main or not weight.requires_grad) else dg.to(weight.dtype)
        gb = None if (b_main or db is None) else db.to(bias.dtype)
        return dx, gw, gb, None, None, None


def layer_norm(x, weight, bias, eps: float, row_keep: torch.Tensor | None = None):
    """LayerNorm over the last dim; ``row_keep`` (bool per row) zeroes whole output rows."""
    if not _kernel_ok(x, weight):
        return layer_norm_reference(x, weight, bias, eps, row_keep)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    rk = None if row_keep is None else row_keep.reshape(-1)
    return _Norm.apply(x2, weight, bias, float(eps), False, rk).view(*lead, x.shape[-1])


def rms_norm(x, weight, eps: float, row_keep: torch.Tensor | None = None):
    """RMSNorm ``x * rsqrt(mean(x^2) + eps) * weight`` with fp32 reduction."""
    if not _kernel_ok(x, weight):
        return rms_norm_reference(x, weight, eps, row_keep)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    rk = None if row_keep is None else row_keep.reshape(-1)
    return _Norm.apply(x2, weight, None, float(eps), True, rk).view(*lead, x.shape[-1])
