"""Attention operators.

``disentangled_attention`` — DeBERTa-v2/v3 content + position attention
(content→content, content→position, position→content with log-bucketed relative
positions); ``rope_attention`` — rotary attention for the rope backbone. Both take
token-major ``[B, S, H]`` projections (heads are column slices, no transposes) and a
compact mask description instead of a dense ``S×S`` tensor:

* ``key_keep``  ``[B, S]`` bool: padding mask; a masked position is also a dead query
  (its output row is zero), which is what the reference's broadcast and outer-product
  masks both mean (``deberta_v2_native.py:617-639``).
* ``doc_ids``   ``[B, S]`` int: packed-document ids (0 = padding); attention stays inside
  a document, inactive queries produce zeros (``training/compile.py:310-349``).
* ``pair_keep`` ``[B, S, S]`` bool: arbitrary pairwise mask, reference path only.

The PyTorch implementations in this file are the fp32 oracle and the CPU path. On
bf16 CUDA tensors the flash-style sm_100a kernels take over (``csrc/attention.cu``).
"""

from __future__ import annotations

import math

import torch

__all__ = [
    "log_bucket_positions",
    "relative_position_luts",
    "disentangled_attention",
    "disentangled_attention_reference",
    "rope_attention",
    "rope_attention_reference",
    "dense_keep_mask",
]


def log_bucket_positions(rel: torch.Tensor, bucket_size: int, max_position: int) -> torch.Tensor:
    """Signed log-bucket id of relative offsets ``rel = q - k`` (``deberta_v2_native.py:51-84``).

    Offsets are first clamped to ``±(max_position-1)``; ``|rel| < bucket_size/2`` keeps its
    value, larger distances map logarithmically onto the remaining buckets.
    """
    rel = rel.to(torch.long)
    if max_position > 0:
        rel = rel.clamp(-max_position + 1, max_position - 1)
    mid = bucket_size // 2
    if mid <= 1:
        return rel
    denom = math.log(max(float(max_position - 1), float(mid + 1)) / float(mid))
    if denom <= 0.0:
        return rel
    mag = rel.abs().clamp_min(1)
    far = torch.ceil(torch.log(mag.float() / float(mid)) / denom * float(mid - 1)) + float(mid)
    bucket = torch.where(mag < mid, mag.to(far.dtype), far) * torch.sign(rel).to(far.dtype)
    return bucket.to(torch.long)


def relative_positions(q_len: int, k_len: int, bucket_size: int, max_position: int, device=None) -> torch.Tensor:
    """``[q_len, k_len]`` matrix of (bucketed) relative positions ``q - k``."""
    rel = torch.arange(q_len, device=device)[:, None] - torch.arange(k_len, device=device)[None, :]
    if bucket_size > 0 and max_position > 0:
        rel = log_bucket_positions(rel, bucket_size, max_position)
    return rel.to(torch.long)


def relative_position_luts(
    q_len: int, k_len: int, bucket_size: int, max_position: int, att_span: int, device=None
) -> tuple[torch.Tensor, torch.Tensor]:
    """Lookup tables over ``delta = q - k`` (index ``delta + k_len - 1``).

    Returns ``(c2p_idx, p2c_idx)``: rows of the projected relative-embedding tables that
    the content→position and position→content terms read for each offset.
    """
    delta = torch.arange(-(k_len - 1), q_len, device=device)
    rel = log_bucket_positions(delta, bucket_size, max_position) if (bucket_size > 0 and max_position > 0) else delta
    rel = rel.clamp(-att_span, att_span)
    c2p = (rel + att_span).clamp(0, 2 * att_span - 1)
    p2c = (att_span - rel).clamp(0, 2 * att_span - 1)
    return c2p.to(torch.int32), p2c.to(torch.int32)


def dense_keep_mask(
    key_keep: torch.Tensor | None, doc_ids: torch.Tensor | None, pair_keep: torch.Tensor | None
) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """(keep ``[B,1,Sq|1,Sk]`` bool, live_queries ``[B,1,Sq,1]`` bool) for the reference path."""
    if pair_keep is not None:
        keep = pair_keep.bool()[:, None]
        live = torch.diagonal(keep, dim1=-2, dim2=-1).unsqueeze(-1)
        return keep, live
    if doc_ids is not None:
        active = doc_ids.ne(0)
        same = doc_ids[:, :, None].eq(doc_ids[:, None, :])
        keep = same & active[:, :, None] & active[:, None, :]
        # inactive queries keep a single edge to position 0 so no row is empty; their output is zeroed
        keep[:, :, 0] = keep[:, :, 0] | ~active
        idx = torch.arange(doc_ids.shape[1], device=doc_ids.device)
        keep[:, idx, idx] = active
        keep = keep[:, None]
        return keep, active[:, None, :, None]
    if key_keep is not None:
        kk = key_keep.bool()
        return kk[:, None, None, :], kk[:, None, :, None]
    return None, None


def _split_heads(x: torch.Tensor, heads: int) -> torch.Tensor:
    b, s, h = x.shape
    return x.view(b, s, heads, h // heads).permute(0, 2, 1, 3)


def disentangled_attention_reference(
    q, k, v, pos_k, pos_q, *, heads: int, scale_factor: int, rel_pos: torch.Tensor | None,
    att_span: int, key_keep=None, doc_ids=None, pair_keep=None, dropout_p: float = 0.0, training: bool = False,
):
    """fp32-score statement of DeBERTa disentangled attention (``deberta_v2_native.py:564-652``).

    ``q``: [B,Sq,H]; ``k``,``v``: [B,Sk,H]; ``pos_k``/``pos_q``: [2·att_span, H] projected relative
    embeddings or ``None`` to drop that term; ``rel_pos``: [Sq,Sk] signed bucket ids.
    """
    d = q.shape[-1] // heads
    scale = math.sqrt(float(d * scale_factor))
    qh, kh, vh = _split_heads(q, heads), _split_heads(k, heads), _split_heads(v, heads)
    qf, kf = qh.float(), kh.float()
    scores = torch.matmul(qf, kf.transpose(-1, -2)) / scale
    if rel_pos is not None and (pos_k is not None or pos_q is not None):
        rel = rel_pos.clamp(-att_span, att_span)
        B, _, Sq, _ = qf.shape
        Sk = kf.shape[2]
        if pos_k is not None:
            pk = pos_k.view(2 * att_span, heads, d).permute(1, 0, 2).float()
            c2p = torch.einsum("bhqd,hpd->bhqp", qf, pk)
            idx = (rel + att_span).clamp(0, 2 * att_span - 1)
            scores = scores + c2p.gather(-1, idx[None, None].expand(B, heads, Sq, Sk)) / scale
        if pos_q is not None:
            pq = pos_q.view(2 * att_span, heads, d).permute(1, 0, 2).float()
            p2c = torch.einsum("bhkd,hpd->bhkp", kf, pq)
            idx = (att_span - rel.transpose(0, 1)).clamp(0, 2 * att_span - 1)
            scores = scores + p2c.gather(-1, idx[None, None].expand(B, heads, Sk, Sq)).transpose(-1, -2) / scale
    keep, live = dense_keep_mask(key_keep, doc_ids, pair_keep)
    if keep is not None:
        scores = scores.masked_fill(~keep, torch.finfo(scores.dtype).min)
        scores = torch.where(live, scores, torch.zeros_like(scores))
    probs = torch.softmax(scores, dim=-1)
    if dropout_p > 0.0 and training:
        probs = torch.nn.functional.dropout(probs, dropout_p, True)
    if keep is not None:
        probs = probs * live.to(probs.dtype)
    ctx = torch.matmul(probs.to(vh.dtype), vh)
    b, h, s, dd = ctx.shape
    return ctx.permute(0, 2, 1, 3).reshape(b, s, h * dd).to(q.dtype)


def disentangled_attention(
    q, k, v, pos_k, pos_q, *, heads: int, scale_factor: int, bucket_size: int, max_position: int, att_span: int,
    key_keep=None, doc_ids=None, pair_keep=None, dropout_p: float = 0.0, training: bool = False,
    rel_pos: torch.Tensor | None = None,
):
    """Disentangled attention context ``[B,Sq,H]``; dispatches to the sm_100a kernel when possible."""
    from . import attention_cuda

    if attention_cuda.disentangled_supported(q, k, v, pos_k, pos_q, heads, pair_keep, dropout_p, training, rel_pos):
        return attention_cuda.disentangled_attention_cuda(
            q, k, v, pos_k, pos_q, heads=heads, scale_factor=scale_factor, bucket_size=bucket_size,
            max_position=max_position, att_span=att_span, key_keep=key_keep, doc_ids=doc_ids,
        )
    if rel_pos is None and (pos_k is not None or pos_q is not None):
        rel_pos = relative_positions(q.shape[1], k.shape[1], bucket_size, max_position, device=q.device)
    return disentangled_attention_reference(
        q, k, v, pos_k, pos_q, heads=heads, scale_factor=scale_factor, rel_pos=rel_pos, att_span=att_span,
        key_keep=key_keep, doc_ids=doc_ids, pair_keep=pair_keep, dropout_p=dropout_p, training=training,
    )


# ---------------------------------------------------------------------------------------
# rotary attention
# ---------------------------------------------------------------------------------------
def rotate_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Rotate even/odd pairs of the first ``rotary_dim`` features (``rope.py:24-34,145-174``).

    ``x``: [B,h,S,d]; ``cos``/``sin``: [S, rotary_dim] with each frequency repeated twice.
    """
    xr, xp = x[..., :rotary_dim], x[..., rotary_dim:]
    x_even, x_odd = xr[..., 0::2], xr[..., 1::2]
    rot = torch.stack((-x_odd, x_even), dim=-1).flatten(-2)
    out = xr * cos + rot * sin
    return torch.cat((out, xp), dim=-1) if xp.shape[-1] else out


def rope_attention_reference(
    q, k, v, cos, sin, *, heads: int, rotary_dim: int, key_keep=None, doc_ids=None, pair_keep=None,
    dropout_p: float = 0.0, training: bool = False,
):
    """Rotary attention with fp32 scores and dead-row guards (``rope_encoder.py:204-287``).

    Returns the context ``[B,S,H]``; rows of inactive queries are zero.
    """
    d = q.shape[-1] // heads
    qh, kh, vh = _split_heads(q, heads), _split_heads(k, heads), _split_heads(v, heads)
    if rotary_dim > 0:
        c, s = cos.to(qh.dtype)[None, None], sin.to(qh.dtype)[None, None]
        qh = rotate_interleaved(qh, c, s, rotary_dim)
        kh = rotate_interleaved(kh, c, s, rotary_dim)
    scores = torch.matmul(qh.float(), kh.float().transpose(-1, -2)) / math.sqrt(float(d))
    keep, live = dense_keep_mask(key_keep, doc_ids, pair_keep)
    if keep is not None:
        scores = scores.masked_fill(~keep, torch.finfo(scores.dtype).min)
    probs = torch.softmax(scores, dim=-1)
    if dropout_p > 0.0 and training:
        probs = torch.nn.functional.dropout(probs, dropout_p, True)
    ctx = torch.matmul(probs.to(vh.dtype), vh)
    if live is not None:
        ctx = ctx * live.to(ctx.dtype)
    b, h, s_, dd = ctx.shape
    return ctx.permute(0, 2, 1, 3).reshape(b, s_, h * dd).to(q.dtype)


def rope_attention(
    q, k, v, cos, sin, *, heads: int, rotary_dim: int, key_keep=None, doc_ids=None, pair_keep=None,
    dropout_p: float = 0.0, training: bool = False,
):
    """Rotary attention context ``[B,S,H]``; dispatches to the sm_100a kernel when possible."""
    from . import attention_cuda

    if attention_cuda.rope_supported(q, k, v, heads, rotary_dim, pair_keep, dropout_p, training):
        return attention_cuda.rope_attention_cuda(
            q, k, v, cos, sin, heads=heads, rotary_dim=rotary_dim, key_keep=key_keep, doc_ids=doc_ids
        )
    return rope_attention_reference(
        q, k, v, cos, sin, heads=heads, rotary_dim=rotary_dim, key_keep=key_keep, doc_ids=doc_ids,
        pair_keep=pair_keep, dropout_p=dropout_p, training=training,
    )
