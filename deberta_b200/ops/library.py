"""The kernel-backed operators as ``torch.library`` custom ops (namespace ``db200``).

Every hot operator of the backbones exists twice over the same launchers: as a ``torch.autograd.Function`` (the
eager path: lowest call overhead) and, here, as a pair of opaque custom ops — forward and backward — with fake
(meta) kernels and ``register_autograd`` formulas. ``torch.compile`` cannot look into ``ctypes`` launches, but it can
carry these ops through Dynamo, AOTAutograd and Inductor as single graph nodes, so compiling the Python glue
around them (``train.compile.enabled``) neither breaks the graph nor re-implements a kernel; the reference compiles
its eager modules the same way (``training/compile.py:154-265``). The public functions of ``ops/linear.py``,
``ops/norm.py``, ``ops/embedding.py``, ``ops/elementwise.py`` and ``ops/attention_cuda.py`` switch to these ops while
a compiler is tracing (``torch.compiler.is_compiling()``).

Conventions
* Gradients of parameters that the engine owns go straight into their fp32 ``main_grad`` buffers; those buffers are
  explicit, mutated arguments of the backward ops (``mutates_args``), and the autograd formula then returns ``None``
  for the parameter. Without a buffer the gradient tensor is returned instead. The public operator functions pass NO
  buffers while a compiler traces: the engine's buffers are views at offsets inside one flat storage, and Inductor
  handles a mutated graph input that is such a view by copying ``offset + size`` elements starting at the view's own
  address, which runs past the end of the storage (seen as an illegal address in a generated copy kernel). Gradients then
  flow back as tensors and the engine's post-accumulate hook adds them to the buffers. Buffers that own their storage
  (as in the tests of this module) are fine.
* On bf16 CUDA tensors the ops launch the sm_100a kernels; on anything else they evaluate the PyTorch statement of the
  same operator, which is what ``torch.library.opcheck`` exercises on a machine without a GPU.
"""

from __future__ import annotations

import torch
from torch import Tensor
from torch.library import custom_op

from .gemm import EPI_GELU_GRAD, EPI_MUL, gemm

__all__ = ["OPS"]

_EMPTY = (0,)


def _kernels(x: Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def _none_or_empty(flag: bool, like: Tensor, shape) -> Tensor:
    return like.new_empty(_EMPTY) if flag else like.new_empty(shape)


# ---------------------------------------------------------------------------------------------------------------
# linear
# ---------------------------------------------------------------------------------------------------------------
@custom_op("db200::linear", mutates_args=())
def linear(x: Tensor, w: Tensor, b: Tensor | None, residual: Tensor | None, w_grad: Tensor | None,
           b_grad: Tensor | None) -> Tensor:
    """``x[M,K] @ w[N,K]ᵀ + b + residual``; ``w_grad`` / ``b_grad`` are the fp32 buffers the backward accumulates into."""
    if _kernels(x):
        return gemm(x, w, bias=b, residual=residual)
    out = torch.nn.functional.linear(x, w.to(x.dtype), None if b is None else b.to(x.dtype))
    return out if residual is None else out + residual


@linear.register_fake
def _(x, w, b, residual, w_grad, b_grad):
    return x.new_empty((x.shape[0], w.shape[0]))


@custom_op("db200::linear_bwd", mutates_args=("w_grad", "b_grad"))
def linear_bwd(dy: Tensor, x: Tensor, w: Tensor, w_grad: Tensor | None, b_grad: Tensor | None, has_bias: bool,
               need_dx: bool) -> tuple[Tensor, Tensor, Tensor]:
    """(dx, dw, db); a gradient that went into its buffer comes back as an empty tensor."""
    from .linear import param_grads_into

    dy = dy.contiguous()
    if _kernels(dy):
        dx = gemm(dy, w, b_mn=True) if need_dx else dy.new_empty(_EMPTY)
    else:
        dx = (dy @ w.to(dy.dtype)) if need_dx else dy.new_empty(_EMPTY)
    dw, db = param_grads_into(dy, x, w, w_grad, b_grad, True, has_bias)
    return dx, (dw if dw is not None else w.new_empty(_EMPTY)), (db if db is not None else w.new_empty(_EMPTY))


@linear_bwd.register_fake
def _(dy, x, w, w_grad, b_grad, has_bias, need_dx):
    return (dy.new_empty((dy.shape[0], w.shape[1])) if need_dx else dy.new_empty(_EMPTY),
            _none_or_empty(w_grad is not None, w, w.shape),
            _none_or_empty(b_grad is not None or not has_bias, w, (w.shape[0],)))


def _linear_setup(ctx, inputs, output):
    x, w, b, residual, w_grad, b_grad = inputs
    ctx.save_for_backward(x, w)
    ctx.bufs = (w_grad, b_grad)
    ctx.has_bias, ctx.has_res = b is not None, residual is not None


def _linear_backward(ctx, dy):
    x, w = ctx.saved_tensors
    w_grad, b_grad = ctx.bufs
    dx, dw, db = linear_bwd(dy, x, w, w_grad, b_grad, ctx.has_bias, ctx.needs_input_grad[0])
    return (dx if ctx.needs_input_grad[0] else None, None if w_grad is not None else dw,
            None if (not ctx.has_bias or b_grad is not None) else db, dy if ctx.has_res else None, None, None)


linear.register_autograd(_linear_backward, setup_context=_linear_setup)


# ---------------------------------------------------------------------------------------------------------------
# fused query/key/value projection (three adjacent weights read as one [3N, K] matrix)
# ---------------------------------------------------------------------------------------------------------------
@custom_op("db200::linear_qkv", mutates_args=())
def linear_qkv(x: Tensor, wq: Tensor, bq: Tensor | None, w_grad: Tensor, b_grad: Tensor | None) -> Tensor:
    from .linear import _span3

    n, k = wq.shape
    return gemm(x, _span3(wq, (3 * n, k)), bias=None if bq is None else _span3(bq, (3 * n,)))


@linear_qkv.register_fake
def _(x, wq, bq, w_grad, b_grad):
    return x.new_empty((x.shape[0], 3 * wq.shape[0]))


@custom_op("db200::linear_qkv_bwd", mutates_args=("w_grad", "b_grad"))
def linear_qkv_bwd(dqkv: Tensor, x: Tensor, wq: Tensor, w_grad: Tensor, b_grad: Tensor | None, need_dx: bool) -> Tensor:
    from .linear import _span3

    n, k = wq.shape
    if dqkv.stride(1) != 1 or dqkv.stride(0) % 8 or dqkv.data_ptr() % 16:
        dqkv = dqkv.contiguous()
    dx = gemm(dqkv, _span3(wq, (3 * n, k)), b_mn=True) if need_dx else dqkv.new_empty(_EMPTY)
    gemm(dqkv, x, a_mn=True, b_mn=True, out=_span3(w_grad, (3 * n, k)), accumulate=True,
         a_sum=None if b_grad is None else _span3(b_grad, (3 * n,)))
    return dx


@linear_qkv_bwd.register_fake
def _(dqkv, x, wq, w_grad, b_grad, need_dx):
    return dqkv.new_empty((dqkv.shape[0], wq.shape[1])) if need_dx else dqkv.new_empty(_EMPTY)


def _qkv_setup(ctx, inputs, output):
    x, wq, bq, w_grad, b_grad = inputs
    ctx.save_for_backward(x, wq)
    ctx.bufs = (w_grad, b_grad)


def _qkv_backward(ctx, dqkv):
    x, wq = ctx.saved_tensors
    dx = linear_qkv_bwd(dqkv, x, wq, ctx.bufs[0], ctx.bufs[1], ctx.needs_input_grad[0])
    return (dx if ctx.needs_input_grad[0] else None, None, None, None, None)


linear_qkv.register_autograd(_qkv_backward, setup_context=_qkv_setup)


# ---------------------------------------------------------------------------------------------------------------
# feed-forward block with exact-erf GELU
# ---------------------------------------------------------------------------------------------------------------
@custom_op("db200::ffn_gelu", mutates_args=())
def ffn_gelu(x: Tensor, w1: Tensor, b1: Tensor | None, w2: Tensor, b2: Tensor | None, residual: Tensor | None,
             w1_grad: Tensor | None, b1_grad: Tensor | None, w2_grad: Tensor | None,
             b2_grad: Tensor | None) -> tuple[Tensor, Tensor, Tensor]:
    """(y, gelu'(z), gelu(z)) with ``z = W1·x + b1`` and ``y = W2·gelu(z) + b2 + residual``."""
    if _kernels(x):
        g, a = gemm(x, w1, bias=b1, epi=EPI_GELU_GRAD)
        return gemm(a, w2, bias=b2, residual=residual), g, a
    from .gemm import gemm_reference

    g, a = gemm_reference(x, w1, bias=b1, epi=EPI_GELU_GRAD)
    return gemm_reference(a, w2, bias=b2, residual=residual), g, a


@ffn_gelu.register_fake
def _(x, w1, b1, w2, b2, residual, w1_grad, b1_grad, w2_grad, b2_grad):
    mid = x.new_empty((x.shape[0], w1.shape[0]))
    return x.new_empty((x.shape[0], w2.shape[0])), mid, torch.empty_like(mid)


@custom_op("db200::ffn_gelu_bwd", mutates_args=("w1_grad", "b1_grad", "w2_grad", "b2_grad"))
def ffn_gelu_bwd(dy: Tensor, x: Tensor, w1: Tensor, w2: Tensor, g: Tensor, a: Tensor, w1_grad: Tensor | None,
                 b1_grad: Tensor | None, w2_grad: Tensor | None, b2_grad: Tensor | None, has_b1: bool, has_b2: bool,
                 need_dx: bool) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    from .gemm import gemm_reference
    from .linear import param_grads_into

    dy = dy.contiguous()
    mm = gemm if _kernels(dy) else gemm_reference
    dz = mm(dy, w2, b_mn=True, epi=EPI_MUL, aux=g)
    dw2, db2 = param_grads_into(dy, a, w2, w2_grad, b2_grad, True, has_b2)
    dx = mm(dz, w1, b_mn=True) if need_dx else dy.new_empty(_EMPTY)
    dw1, db1 = param_grads_into(dz, x, w1, w1_grad, b1_grad, True, has_b1)
    e = lambda t, like: t if t is not None else like.new_empty(_EMPTY)  # noqa: E731
    return dx, e(dw1, w1), e(db1, w1), e(dw2, w2), e(db2, w2)


@ffn_gelu_bwd.register_fake
def _(dy, x, w1, w2, g, a, w1_grad, b1_grad, w2_grad, b2_grad, has_b1, has_b2, need_dx):
    return (dy.new_empty((dy.shape[0], w1.shape[1])) if need_dx else dy.new_empty(_EMPTY),
            _none_or_empty(w1_grad is not None, w1, w1.shape), _none_or_empty(b1_grad is not None or not has_b1, w1, (w1.shape[0],)),
            _none_or_empty(w2_grad is not None, w2, w2.shape), _none_or_empty(b2_grad is not None or not has_b2, w2, (w2.shape[0],)))


def _ffn_setup(ctx, inputs, output):
    x, w1, b1, w2, b2, residual, w1g, b1g, w2g, b2g = inputs
    _, g, a = output
    ctx.save_for_backward(x, w1, w2, g, a)
    ctx.bufs = (w1g, b1g, w2g, b2g)
    ctx.flags = (b1 is not None, b2 is not None, residual is not None)


def _ffn_backward(ctx, dy, _dg, _da):
    x, w1, w2, g, a = ctx.saved_tensors
    w1g, b1g, w2g, b2g = ctx.bufs
    has_b1, has_b2, has_res = ctx.flags
    dx, dw1, db1, dw2, db2 = ffn_gelu_bwd(dy, x, w1, w2, g, a, w1g, b1g, w2g, b2g, has_b1, has_b2, ctx.needs_input_grad[0])
    return (dx if ctx.needs_input_grad[0] else None, None if w1g is not None else dw1,
            None if (not has_b1 or b1g is not None) else db1, None if w2g is not None else dw2,
            None if (not has_b2 or b2g is not None) else db2, dy if has_res else None, None, None, None, None)


ffn_gelu.register_autograd(_ffn_backward, setup_context=_ffn_setup)


# ---------------------------------------------------------------------------------------------------------------
# LayerNorm / RMSNorm
# ---------------------------------------------------------------------------------------------------------------
@custom_op("db200::norm", mutates_args=())
def norm(x: Tensor, weight: Tensor, bias: Tensor | None, row_keep: Tensor | None, eps: float, rms: bool,
         w_grad: Tensor | None, b_grad: Tensor | None) -> tuple[Tensor, Tensor, Tensor]:
    """(y, mean, rstd) of a ``[rows, H]`` tensor; ``mean`` is empty for RMSNorm."""
    from .norm import norm_forward

    return norm_forward(x, weight, bias, row_keep, eps, rms)


@norm.register_fake
def _(x, weight, bias, row_keep, eps, rms, w_grad, b_grad):
    stat = x.new_empty((x.shape[0],), dtype=torch.float32)
    return torch.empty_like(x), (x.new_empty(_EMPTY, dtype=torch.float32) if rms else stat), torch.empty_like(stat)


@custom_op("db200::norm_bwd", mutates_args=("w_grad", "b_grad"))
def norm_bwd(dy: Tensor, x: Tensor, weight: Tensor, mean: Tensor, rstd: Tensor, row_keep: Tensor | None, rms: bool,
             has_bias: bool, w_grad: Tensor | None, b_grad: Tensor | None) -> tuple[Tensor, Tensor, Tensor]:
    from .norm import norm_backward

    dx, dg, db = norm_backward(dy, x, weight, mean, rstd, row_keep, rms, has_bias, w_grad, b_grad)
    e = lambda t: t if t is not None else weight.new_empty(_EMPTY)  # noqa: E731
    return dx, e(dg), e(db)


@norm_bwd.register_fake
def _(dy, x, weight, mean, rstd, row_keep, rms, has_bias, w_grad, b_grad):
    return (torch.empty_like(x), _none_or_empty(w_grad is not None, weight, weight.shape),
            _none_or_empty(b_grad is not None or not has_bias, weight, weight.shape))


def _norm_setup(ctx, inputs, output):
    x, weight, bias, row_keep, eps, rms, w_grad, b_grad = inputs
    _, mean, rstd = output
    ctx.save_for_backward(x, weight, mean, rstd, row_keep)
    ctx.bufs = (w_grad, b_grad)
    ctx.flags = (bool(rms), bias is not None)


def _norm_backward(ctx, dy, _dm, _dr):
    x, weight, mean, rstd, row_keep = ctx.saved_tensors
    w_grad, b_grad = ctx.bufs
    rms, has_bias = ctx.flags
    dx, dg, db = norm_bwd(dy, x, weight, mean, rstd, row_keep, rms, has_bias, w_grad, b_grad)
    return (dx, None if w_grad is not None else dg, None if (not has_bias or b_grad is not None) else db,
            None, None, None, None, None)


norm.register_autograd(_norm_backward, setup_context=_norm_setup)


# ---------------------------------------------------------------------------------------------------------------
# embedding lookup with an optional delta table
# ---------------------------------------------------------------------------------------------------------------
@custom_op("db200::embed", mutates_args=())
def embed(ids: Tensor, table: Tensor, delta: Tensor | None, padding_idx: int, table_grad: Tensor | None,
          delta_grad: Tensor | None) -> Tensor:
    from .embedding import embed_forward

    return embed_forward(ids, table, delta)


@embed.register_fake
def _(ids, table, delta, padding_idx, table_grad, delta_grad):
    return table.new_empty((*ids.shape, table.shape[1]))


@custom_op("db200::embed_bwd", mutates_args=("table_grad", "delta_grad"))
def embed_bwd(dout: Tensor, ids: Tensor, vocab: int, padding_idx: int, table_grad: Tensor | None,
              delta_grad: Tensor | None) -> None:
    from .embedding import embed_backward

    embed_backward(dout, ids, vocab, padding_idx, (table_grad, delta_grad))


@embed_bwd.register_fake
def _(dout, ids, vocab, padding_idx, table_grad, delta_grad):
    return None


def _embed_setup(ctx, inputs, output):
    ids, table, delta, padding_idx, table_grad, delta_grad = inputs
    ctx.save_for_backward(ids)
    ctx.meta = (int(table.shape[0]), int(padding_idx), table_grad, delta_grad)


def _embed_backward(ctx, dout):
    (ids,) = ctx.saved_tensors
    vocab, pad, tg, dg = ctx.meta
    embed_bwd(dout, ids, vocab, pad, tg, dg)
    return None, None, None, None, None, None


embed.register_autograd(_embed_backward, setup_context=_embed_setup)


# ---------------------------------------------------------------------------------------------------------------
# rotary embedding and SwiGLU gate
# ---------------------------------------------------------------------------------------------------------------
@custom_op("db200::rotary", mutates_args=())
def rotary(x: Tensor, cos: Tensor, sin: Tensor, heads: int, rotary_dim: int, inverse: bool) -> Tensor:
    from .elementwise import rotary_apply

    return rotary_apply(x, cos, sin, heads, rotary_dim, inverse)


@rotary.register_fake
def _(x, cos, sin, heads, rotary_dim, inverse):
    return x.new_empty(x.shape)


def _rotary_setup(ctx, inputs, output):
    _, cos, sin, heads, rotary_dim, inverse = inputs
    ctx.save_for_backward(cos, sin)
    ctx.meta = (heads, rotary_dim, inverse)


def _rotary_backward(ctx, dy):
    cos, sin = ctx.saved_tensors
    heads, rotary_dim, inverse = ctx.meta
    return rotary(dy, cos, sin, heads, rotary_dim, not inverse), None, None, None, None, None


rotary.register_autograd(_rotary_backward, setup_context=_rotary_setup)


@custom_op("db200::swiglu", mutates_args=())
def swiglu(gate_up: Tensor) -> Tensor:
    from .elementwise import swiglu_forward

    return swiglu_forward(gate_up)


@swiglu.register_fake
def _(gate_up):
    return gate_up.new_empty((gate_up.shape[0], gate_up.shape[1] // 2))


@custom_op("db200::swiglu_bwd", mutates_args=())
def swiglu_bwd(gate_up: Tensor, dout: Tensor) -> Tensor:
    from .elementwise import swiglu_backward

    return swiglu_backward(gate_up, dout)


@swiglu_bwd.register_fake
def _(gate_up, dout):
    return torch.empty_like(gate_up)


swiglu.register_autograd(lambda ctx, dout: swiglu_bwd(ctx.saved_tensors[0], dout),
                         setup_context=lambda ctx, inputs, output: ctx.save_for_backward(inputs[0]))


# ---------------------------------------------------------------------------------------------------------------
# flash attention (content scores, optional disentangled position terms, padding / document masks)
# ---------------------------------------------------------------------------------------------------------------
@custom_op("db200::flash_attn", mutates_args=())
def flash_attn(q: Tensor, k: Tensor, v: Tensor, pos_k: Tensor | None, pos_q: Tensor | None, key_keep: Tensor | None,
               doc_ids: Tensor | None, heads: int, scale: float, bucket_size: int, max_position: int,
               att_span: int) -> tuple[Tensor, Tensor, Tensor]:
    """(context ``[B,S,H]``, log-sum-exp ``[B,heads,S]``, position bias ``[B,heads,S,ldb]`` or empty)."""
    if not _kernels(q):
        out = _attn_reference(q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position, att_span)
        return out, q.new_zeros((q.shape[0], heads, q.shape[1]), dtype=torch.float32), q.new_empty(_EMPTY)
    from .attention_cuda import attention_forward

    return attention_forward(q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position, att_span)


def _attn_reference(q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position, att_span):
    """The fp32 PyTorch statement of the operator (CPU and non-bf16 tensors)."""
    from .attention import disentangled_attention_reference, relative_positions

    d = q.shape[-1] // heads
    rel = None
    if pos_k is not None or pos_q is not None:
        rel = relative_positions(q.shape[1], k.shape[1], bucket_size, max_position, device=q.device)
    return disentangled_attention_reference(q, k, v, pos_k, pos_q, heads=heads, scale_factor=scale * scale / d, rel_pos=rel,
                                            att_span=att_span, key_keep=key_keep, doc_ids=doc_ids)


def _attn_reference_backward(dout, q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position,
                             att_span):
    """Gradients of ``_attn_reference`` written out by hand (a custom-op body runs below autograd)."""
    from .attention import dense_keep_mask, relative_positions

    B, S, H = q.shape
    d = H // heads
    split = lambda t: t.float().view(B, -1, heads, d).permute(0, 2, 1, 3)  # noqa: E731
    merge = lambda t: t.permute(0, 2, 1, 3).reshape(B, -1, H)  # noqa: E731
    qh, kh, vh, do = split(q), split(k), split(v), split(dout)
    scores = qh @ kh.transpose(-1, -2)
    ic = ip = pk = pq = None
    if pos_k is not None or pos_q is not None:
        rel = relative_positions(S, S, bucket_size, max_position, device=q.device).clamp(-att_span, att_span)
        if pos_k is not None:
            pk = pos_k.float().view(-1, heads, d).permute(1, 0, 2)
            ic = (rel + att_span).clamp(0, 2 * att_span - 1)[None, None].expand(B, heads, S, S)
            scores = scores + (qh @ pk.transpose(-1, -2)).gather(-1, ic)
        if pos_q is not None:
            pq = pos_q.float().view(-1, heads, d).permute(1, 0, 2)
            ip = (att_span - rel.transpose(0, 1)).clamp(0, 2 * att_span - 1)[None, None].expand(B, heads, S, S)  # [k, q]
            scores = scores + (kh @ pq.transpose(-1, -2)).gather(-1, ip).transpose(-1, -2)
    scores = scores / scale
    keep, live = dense_keep_mask(key_keep, doc_ids, None)
    if keep is not None:
        scores = torch.where(live, scores.masked_fill(~keep, torch.finfo(scores.dtype).min), torch.zeros_like(scores))
    p = torch.softmax(scores, dim=-1)
    if keep is not None:
        p = p * live.to(p.dtype)
    dv = p.transpose(-1, -2) @ do
    dp = do @ vh.transpose(-1, -2)
    ds = p * (dp - (dp * p).sum(-1, keepdim=True)) / scale
    dq = ds @ kh
    dk = ds.transpose(-1, -2) @ qh
    dpk, dpq = q.new_empty(_EMPTY), q.new_empty(_EMPTY)
    if pk is not None:
        g = torch.zeros(B, heads, S, pk.shape[1]).scatter_add_(-1, ic, ds)       # [q, bucket]
        dq = dq + g @ pk
        dpk = (g.transpose(-1, -2) @ qh).sum(0).permute(1, 0, 2).reshape(-1, H).to(pos_k.dtype)
    if pq is not None:
        g = torch.zeros(B, heads, S, pq.shape[1]).scatter_add_(-1, ip, ds.transpose(-1, -2))  # [k, bucket]
        dk = dk + g @ pq
        dpq = (g.transpose(-1, -2) @ kh).sum(0).permute(1, 0, 2).reshape(-1, H).to(pos_q.dtype)
    return merge(dq).to(q.dtype), merge(dk).to(k.dtype), merge(dv).to(v.dtype), dpk, dpq


@flash_attn.register_fake
def _(q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position, att_span):
    from .attention_cuda import BIAS_MODE_MAX_SEQ

    B, S, H = q.shape
    has_pos = pos_k is not None or pos_q is not None
    bias = (q.new_empty((B, heads, S, (S + 127) // 128 * 128)) if (has_pos and S <= BIAS_MODE_MAX_SEQ and q.is_cuda)
            else q.new_empty(_EMPTY))
    return q.new_empty((B, S, H)), q.new_empty((B, heads, S), dtype=torch.float32), bias


@custom_op("db200::flash_attn_bwd", mutates_args=())
def flash_attn_bwd(dout: Tensor, q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, bias: Tensor,
                   pos_k: Tensor | None, pos_q: Tensor | None, key_keep: Tensor | None, doc_ids: Tensor | None,
                   heads: int, scale: float, bucket_size: int, max_position: int,
                   att_span: int) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    """(dq, dk, dv, dpos_k, dpos_q); absent position tables give empty gradients."""
    if not _kernels(q):
        return _attn_reference_backward(dout, q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size,
                                        max_position, att_span)
    from .attention_cuda import attention_backward

    return attention_backward(dout, q, k, v, out, lse, bias, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size,
                              max_position, att_span)


@flash_attn_bwd.register_fake
def _(dout, q, k, v, out, lse, bias, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position, att_span):
    e = lambda t: q.new_empty(_EMPTY) if t is None else torch.empty_like(t)  # noqa: E731
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), e(pos_k), e(pos_q)


def _attn_setup(ctx, inputs, output):
    q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position, att_span = inputs
    out, lse, bias = output
    ctx.save_for_backward(q, k, v, out, lse, bias, pos_k, pos_q, key_keep, doc_ids)
    ctx.meta = (heads, scale, bucket_size, max_position, att_span)


def _attn_backward(ctx, dout, _dlse, _dbias):
    q, k, v, out, lse, bias, pos_k, pos_q, key_keep, doc_ids = ctx.saved_tensors
    dq, dk, dv, dpk, dpq = flash_attn_bwd(dout, q, k, v, out, lse, bias, pos_k, pos_q, key_keep, doc_ids, *ctx.meta)
    return (dq, dk, dv, None if pos_k is None else dpk, None if pos_q is None else dpq, None, None, None, None, None,
            None, None)


flash_attn.register_autograd(_attn_backward, setup_context=_attn_setup)


OPS = {"linear": linear, "linear_bwd": linear_bwd, "linear_qkv": linear_qkv, "linear_qkv_bwd": linear_qkv_bwd,
       "ffn_gelu": ffn_gelu, "ffn_gelu_bwd": ffn_gelu_bwd, "norm": norm, "norm_bwd": norm_bwd, "embed": embed,
       "embed_bwd": embed_bwd, "rotary": rotary, "swiglu": swiglu, "swiglu_bwd": swiglu_bwd, "flash_attn": flash_attn,
       "flash_attn_bwd": flash_attn_bwd}
