"""Fused vocabulary projection + cross-entropy + sampling from ``softmax(logits / T)`` on the tcgen05 GEMM.

Forward: one sweep over vocabulary tiles of the tied embedding table; each tile's epilogue
reduces its logits to (max, sum-exp, label logit, sampling candidate) per row, a small kernel
combines the tiles. The candidate is exact two-level sampling: inside every 32-column group an id is drawn by
inverting the running sum of ``exp(logit / T)`` over the allowed ids, and the groups compete through Gumbel-max keys
``ln(group mass) + Gumbel noise``, so a row costs two uniforms per 32 logits instead of a Gumbel draw per logit. The ``[N, V]`` logits are never written. Backward recomputes the logits
tile by tile and writes ``softmax − onehot`` once in bf16, which feeds the two gradient GEMMs.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .gemm import GemmArgsCache, gemm
from .linear import _param_grads, weight_grad_into

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
        ctx.weight_ref = weight  # the parameter itself: a saved tensor may come back without its gradient buffer
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
        want_b = bias is not None and bias.requires_grad
        w_main = getattr(ctx.weight_ref, "main_grad", None)
        b_main = getattr(bias, "main_grad", None) if want_b else None
        if weight.requires_grad and want_b and w_main is not None and b_main is not None:
            # the table's gradient GEMM sums dlogits over the rows on the tensor cores as well: no column-sum pass
            # over the [N, V] tensor
            dw, db = _param_grads(dlogits, x, ctx.weight_ref, bias)
        else:
            dw = weight_grad_into(dlogits, x, weight, w_main) if weight.requires_grad else None
            db = None
            if want_b:
                from .linear import colsum_into

                gb = b_main if b_main is not None else torch.zeros(V, dtype=torch.float32, device=x.device)
                colsum_into(dlogits, gb)
                if b_main is None:
                    db = gb.to(bias.dtype)
        return dx, dw, db, None, None, None


def mlm_loss_and_sample_cuda(x, weight, bias, labels, forbidden_mask, temperature: float):
    if float(temperature) <= 0:
        raise ValueError("sampling_temperature must be > 0")
    loss, sampled = _VocabCE.apply(x, weight, bias, labels, forbidden_mask, float(temperature))
    return loss, sampled


# ---- replaced-token-detection head ---------------------------------------------------------------------------------

class _RTDHead(torch.autograd.Function):
    """dense + GELU (GEMM epilogue) → classifier dot + masked BCE + counts (one kernel); see ``csrc/elementwise.cu``."""

    @staticmethod
    def forward(ctx, x, dense_w, dense_b, cls_w, cls_b, labels, active):
        from .gemm import EPI_GELU

        pre, act = gemm(x, dense_w, bias=dense_b, epi=EPI_GELU)
        T, H = act.shape
        logits = torch.empty(T, dtype=torch.float32, device=x.device)
        stats = torch.zeros(4, dtype=torch.float32, device=x.device)
        _lib.call("db200_rtd_tail_fwd", _lib.ptr(act), ctypes.c_longlong(act.stride(0)), _lib.ptr(cls_w), _lib.ptr(cls_b),
                  _lib.ptr(labels), _lib.ptr(active), _lib.ptr(logits), _lib.ptr(stats), ctypes.c_longlong(T),
                  ctypes.c_int(H), _lib.stream_ptr())
        denom = stats[2].clamp(min=1.0)
        ctx.save_for_backward(x, dense_w, pre, act, logits, labels, active, stats)
        ctx.refs = (dense_b, cls_w, cls_b)
        out = (stats[0] / denom, stats[1] / denom, stats[2].clone(), stats[3].clone())
        ctx.mark_non_differentiable(*out[1:])
        return out

    @staticmethod
    def backward(ctx, grad_loss, *_unused):
        from .linear import _param_grads

        x, dense_w, pre, act, logits, labels, active, stats = ctx.saved_tensors
        dense_b, cls_w, cls_b = ctx.refs
        T, H = act.shape
        dev = x.device
        g = grad_loss.detach().float().reshape(1).contiguous()
        d_pre = torch.empty_like(pre)
        dw_main, db_main = getattr(cls_w, "main_grad", None), getattr(cls_b, "main_grad", None) if cls_b is not None else None
        dw = dw_main if dw_main is not None else torch.zeros(H, dtype=torch.float32, device=dev)
        db = db_main if db_main is not None else torch.zeros(1, dtype=torch.float32, device=dev)
        _lib.call("db200_rtd_tail_bwd", _lib.ptr(act), ctypes.c_longlong(act.stride(0)), _lib.ptr(pre),
                  ctypes.c_longlong(pre.stride(0)), _lib.ptr(cls_w), _lib.ptr(logits), _lib.ptr(labels), _lib.ptr(active),
                  _lib.ptr(g), _lib.ptr(stats), _lib.ptr(d_pre), ctypes.c_longlong(d_pre.stride(0)), _lib.ptr(dw), _lib.ptr(db),
                  ctypes.c_longlong(T), ctypes.c_int(H), _lib.stream_ptr())
        dx = gemm(d_pre, dense_w, b_mn=True) if ctx.needs_input_grad[0] else None
        d_dense_w, d_dense_b = _param_grads(d_pre, x, dense_w, dense_b)
        d_cls_w = None if dw_main is not None else dw.view(1, H).to(cls_w.dtype)
        d_cls_b = None if (cls_b is None or db_main is not None) else db.to(cls_b.dtype)
        return dx, d_dense_w, d_dense_b, d_cls_w, d_cls_b, None, None


def rtd_head_supported(x: torch.Tensor, dense_w: torch.Tensor, cls_w: torch.Tensor, act_name: str) -> bool:
    h = x.shape[-1]
    return (x.is_cuda and x.dtype == torch.bfloat16 and dense_w.dtype == torch.bfloat16 and cls_w.dtype == torch.bfloat16
            and act_name == "gelu" and h % 8 == 0 and h <= 1024 and tuple(dense_w.shape) == (h, h)
            and tuple(cls_w.shape) == (1, h) and cls_w.is_contiguous())


def rtd_head_loss_cuda(x, dense_w, dense_b, cls_w, cls_b, labels, active):
    """(loss, accuracy, active-token count, positive count) of the RTD head on normalised hidden states ``x`` [..., H]."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    lab = labels.reshape(-1).gt(0.5).to(torch.int64).contiguous() if labels.is_floating_point() else \
        labels.reshape(-1).to(torch.int64).contiguous()
    act = active.reshape(-1).to(torch.uint8).contiguous()
    return _RTDHead.apply(x2, dense_w, dense_b, cls_w, cls_b, lab, act)
