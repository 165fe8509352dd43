"""Fused vocabulary projection + cross-entropy + Gumbel-max sampling on the tcgen05 GEMM.

Forward: one sweep over vocabulary tiles of the tied embedding table; each tile's epilogue
reduces its logits to (max, sum-exp, label logit, best noisy logit) per row, a small kernel
combines the tiles. The ``[N, V]`` logits are never written. Backward recomputes the logits
tile by tile and writes ``softmax − onehot`` once in bf16, which feeds the two gradient GEMMs.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .gemm import GemmArgsCache, gemm
from .linear import _weight_grad

_SEED_STATE = {"counter": 0}


def vocab_ce_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 2
            and x.shape[1] % 8 == 0 and weight.is_contiguous() and x.shape[0] > 0)


def _next_seed() -> int:
    """A fresh 64-bit seed per call, derived from torch's CPU generator so runs are reproducible under manual_seed."""
    _SEED_STATE["counter"] += 1
    base = int(torch.initial_seed()) & 0xFFFFFFFFFFFF
    return (base * 0x9E3779B97F4A7C15 + _SEED_STATE["counter"] * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF


def _ce_gemm(x, weight, bias, labels, *, epi, **extra) -> None:
    a = GemmArgsCache.get()
    ctypes.memset(ctypes.byref(a), 0, ctypes.sizeof(a))
    N, E = x.shape
    a.A, a.B = x.data_ptr(), weight.data_ptr()
    a.bias = None if bias is None else bias.data_ptr()
    a.M, a.N, a.K, a.batch = N, weight.shape[0], E, 1
    a.lda, a.ldb = x.stride(0), weight.stride(0)
    a.alpha, a.epi = 1.0, epi
    a.labels = labels.data_ptr()
    for k, v in extra.items():
        setattr(a, k, v)
    _lib.call("db200_gemm_bf16", ctypes.byref(a), _lib.stream_ptr())


class _VocabCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, labels, forbidden, temperature):
        x = x.contiguous()
        N, V = x.shape[0], weight.shape[0]
        dev = x.device
        bias_c = None if bias is None else bias.to(torch.bfloat16).contiguous()
        labels = labels.to(torch.int64).contiguous()
        tile_n = int(_lib.lib().db200_gemm_tile_n(ctypes.c_int(V)))
        tiles_n = (V + tile_n - 1) // tile_n
        part = torch.empty((4, tiles_n, N), dtype=torch.float32, device=dev)
        label_logit = torch.zeros(N, dtype=torch.float32, device=dev)
        forb = None if (forbidden is None or forbidden.numel() == 0) else forbidden.to(torch.uint8).contiguous()
        _ce_gemm(x, weight, bias_c, labels, epi=_lib.EPI_CE_FWD, forbidden=None if forb is None else forb.data_ptr(),
                 inv_temp=1.0 / float(temperature), seed=_next_seed(), ce_part=part.data_ptr(),
                 label_logit=label_logit.data_ptr())
        lse = torch.empty(N, dtype=torch.float32, device=dev)
        loss_rows = torch.empty(N, dtype=torch.float32, device=dev)
        sampled = torch.empty(N, dtype=torch.int64, device=dev)
        _lib.call("db200_ce_combine", _lib.ptr(part), _lib.ptr(label_logit), ctypes.c_int(tiles_n), ctypes.c_int(N),
                  _lib.ptr(lse), _lib.ptr(loss_rows), _lib.ptr(sampled), _lib.stream_ptr())
        ctx.save_for_backward(x, weight, bias_c, labels, lse)
        ctx.bias_ref = bias
        ctx.mark_non_differentiable(sampled)
        return loss_rows.mean(), sampled

    @staticmethod
    def backward(ctx, grad_loss, _grad_sampled):
        x, weight, bias_c, labels, lse = ctx.saved_tensors
        bias = ctx.bias_ref
        N, V = x.shape[0], weight.shape[0]
        Vp = (V + 63) // 64 * 64
        dlogits = torch.empty((N, Vp), dtype=torch.bfloat16, device=x.device)[:, :V]
        g = grad_loss.detach().float().reshape(1).contiguous()
        _ce_gemm(x, weight, bias_c, labels, epi=_lib.EPI_CE_BWD, out=dlogits.data_ptr(), ldo=Vp, row_lse=lse.data_ptr(),
                 gscale=1.0 / N, gscale_ptr=g.data_ptr())
        dx = gemm(dlogits, weight, b_mn=True)
        dw = _weight_grad(dlogits, x, weight) if weight.requires_grad else None
        db = None
        if bias is not None and bias.requires_grad:
            from .linear import colsum_into

            main = getattr(bias, "main_grad", None)
            gb = main if main is not None else torch.zeros(V, dtype=torch.float32, device=x.device)
            colsum_into(dlogits, gb)
            if main is None:
                db = gb.to(bias.dtype)
        return dx, dw, db, None, None, None


def mlm_loss_and_sample_cuda(x, weight, bias, labels, forbidden_mask, temperature: float):
    if float(temperature) <= 0:
        raise ValueError("sampling_temperature must be > 0")
    loss, sampled = _VocabCE.apply(x, weight, bias, labels, forbidden_mask, float(temperature))
    return loss, sampled
