"""Launchers and autograd glue for the sm_100a attention kernels (``csrc/attention.cu``, ``csrc/posbias_tc.cu``).

Position terms of disentangled attention (``deberta_v2_native.py:349-432``), up to ``BIAS_MODE_MAX_SEQ`` tokens:
``csrc/posbias_tc.cu`` computes the ``[B, heads, S, S]`` bias ``Q·PosK[δ] + K·PosQ[δ]`` tile by tile on the
tensor cores (window products in TMEM, bucket lookup in shared memory) and, in the backward pass, folds the bias
gradient onto the bucket axis inside the kernel and multiplies it into dQ, dK and the table gradients; no
``[tokens, heads, 2·span]`` score table is ever written. Longer sequences, and bucket maps whose tiles span more
than 256 table rows, use the table path: two per-head score tables from the batched GEMM, gathered inside the
attention kernels (or pre-gathered by ``csrc/posbias.cu``), and their gradients reduced by prefix-sum scans.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from .gemm import gemm

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


class AttnArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p),
        ("ldq", c_ll), ("ldk", c_ll), ("ldv", c_ll),
        ("out", c_void_p), ("ldo", c_ll), ("lse", c_void_p),
        ("B", c_int), ("S", c_int), ("heads", c_int), ("span2", c_int),
        ("scale", c_float),
        ("c2p", c_void_p), ("p2c", c_void_p), ("lut_c2p", c_void_p), ("lut_p2c", c_void_p),
        ("key_keep", c_void_p), ("doc_ids", c_void_p),
        ("dout", c_void_p), ("ld_do", c_ll), ("delta", c_void_p), ("dq_acc", c_void_p),
        ("dk", c_void_p), ("dv", c_void_p), ("ld_dk", c_ll), ("ld_dv", c_ll),
        ("d_c2p", c_void_p), ("d_p2c", c_void_p),
        ("bias", c_void_p), ("dbias", c_void_p), ("ldb", c_ll),
        ("doc_tiles", c_void_p),
    ]


class PosBiasArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("ldq", c_ll), ("ldk", c_ll),
        ("pos_k", c_void_p), ("pos_q", c_void_p), ("ld_pos", c_ll),
        ("lut_c2p", c_void_p), ("lut_p2c", c_void_p), ("lut_c2p_host", c_void_p), ("lut_p2c_host", c_void_p),
        ("B", c_int), ("S", c_int), ("heads", c_int), ("span2", c_int),
        ("bias", c_void_p), ("ldb", c_ll), ("dbias", c_void_p),
        ("dq_acc", c_void_p), ("dk", c_void_p), ("ld_dk", c_ll),
        ("d_pos_k", c_void_p), ("d_pos_q", c_void_p),
    ]


# Up to this sequence length the position terms are pre-gathered into a key-indexed
# [B, heads, S, S] bf16 bias (contiguous vector loads in the attention kernels); beyond it the
# kernels gather from the bucket-indexed tables directly, which needs no S x S storage.
BIAS_MODE_MAX_SEQ = 1024
# Build the bias with the tensor-core tile kernel of posbias_tc.cu (False: score tables from the batched GEMM + gather).
POSBIAS_TENSOR_CORE = True
# Reduce the bias gradient with the tile kernel too (fold in shared memory + MMAs) instead of the prefix-sum scans and
# four batched GEMMs. Measured at B=32, S=512, 12 heads: 595 us against 440 us for the scan path, so it is off by default.
POSBIAS_TENSOR_CORE_BWD = False
_TC_REJECTED = -13  # launcher: this bucket map / table size needs the table path


def set_forward_key_tile(keys: int) -> int:
    """Keys per tile of the forward kernel: 64 (two CTAs per SM; warp-specialised where the mask / position mode allows
    it: the default), 65 (64-key tiles without warp specialisation) or 128 (one 512-thread CTA per SM). Returns the
    previous setting. The results agree to rounding; the choice is about latency hiding."""
    return int(_lib.lib().db200_attn_set_fwd_key_tile(c_int(int(keys))))


def set_backward_persistent(on: bool | int) -> int:
    """Backward kernel scheduling: ``True`` (default) starts one CTA per SM that walks the (batch, head, key tile) work
    items, so barriers and tensor memory are set up once and the next item's operands travel while the current item's
    gradients leave the tensor memory; ``False`` starts one CTA per item; an integer above 1 caps the number of CTAs
    (tests use it to give every CTA several items on small inputs). Inputs with document ids always get a CTA per
    item (their items differ in length). Returns the previous setting; results are identical up to the order of the
    fp32 additions into the query gradient."""
    return int(_lib.lib().db200_attn_set_bwd_persistent(c_int(int(on))))


_LUT_CACHE: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _luts(S: int, bucket_size: int, max_position: int, att_span: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    key = (S, bucket_size, max_position, att_span, str(device))
    hit = _LUT_CACHE.get(key)
    if hit is None:
        from .attention import relative_position_luts

        c2p, p2c = relative_position_luts(S, S, bucket_size, max_position, att_span)
        c2p, p2c = c2p.to(torch.int16).contiguous(), p2c.to(torch.int16).contiguous()
        hit = (c2p.to(device), p2c.to(device))
        _LUT_CACHE[key] = hit
        _LUT_HOST[(hit[0].data_ptr(), hit[1].data_ptr())] = (c2p, p2c)
    return hit


_LUT_HOST: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _posbias_args(q, k, pos_k, pos_q, luts, heads: int, span2: int) -> PosBiasArgs:
    B, S, _ = q.shape
    host = _LUT_HOST[(luts[0].data_ptr(), luts[1].data_ptr())]
    a = PosBiasArgs()
    a.q, a.k, a.ldq, a.ldk = q.data_ptr(), k.data_ptr(), q.stride(1), k.stride(1)
    a.pos_k = None if pos_k is None else pos_k.data_ptr()
    a.pos_q = None if pos_q is None else pos_q.data_ptr()
    a.ld_pos = (pos_k if pos_k is not None else pos_q).stride(0)
    a.lut_c2p, a.lut_p2c = luts[0].data_ptr(), luts[1].data_ptr()
    a.lut_c2p_host, a.lut_p2c_host = host[0].data_ptr(), host[1].data_ptr()
    a.B, a.S, a.heads, a.span2 = B, S, heads, span2
    return a


_RANGE_CACHE: dict[tuple, tuple] = {}


def _bucket_ranges(lut: torch.Tensor, S: int, span2: int) -> torch.Tensor | None:
    """Bucket edges for the prefix-sum scatter: int32 ``[sign, E_0 .. E_span2]`` on the LUT's device.

    With ``sign = +1`` bucket ``j`` collects the offsets ``E_j <= q-k < E_{j+1}``; with ``sign = -1`` (the bucket index
    falls as ``q-k`` grows) it collects ``E_{j+1} <= q-k < E_j``; unused buckets have ``E_j = E_{j+1}``.
    ``None`` when the map is not monotone in ``q-k`` (the kernels then fall back to the atomic scatter).
    """
    idx = lut.to(torch.int64).cpu()
    delta = torch.arange(-(S - 1), S, dtype=torch.int64)
    big = 1 << 20
    lo = torch.full((span2,), big, dtype=torch.int64).scatter_reduce_(0, idx, delta, "amin").tolist()
    hi = torch.full((span2,), -big, dtype=torch.int64).scatter_reduce_(0, idx, delta, "amax").tolist()
    cnt = torch.bincount(idx, minlength=span2).tolist()
    used = [j for j in range(span2) if cnt[j] > 0]
    if not used or span2 % 8 or any(hi[j] - lo[j] + 1 != cnt[j] for j in used):
        return None
    sign = 1 if (len(used) < 2 or lo[used[1]] > lo[used[0]]) else -1
    start = (lambda j: lo[j]) if sign > 0 else (lambda j: hi[j] + 1)
    end = (lambda j: hi[j] + 1) if sign > 0 else (lambda j: lo[j])
    edges = [0] * (span2 + 1)
    last = used[-1]
    for j in range(last + 1, span2 + 1):
        edges[j] = end(last)
    live = set(used)
    for j in range(last, -1, -1):
        if j in live:
            if end(j) != edges[j + 1]:
                return None  # a gap or an overlap between neighbouring buckets
            edges[j] = start(j)
        else:
            edges[j] = edges[j + 1]
    return torch.tensor([sign, *edges], dtype=torch.int32).to(lut.device)


def _ranges(luts: tuple[torch.Tensor, torch.Tensor], S: int, span2: int) -> tuple:
    key = (luts[0].data_ptr(), luts[1].data_ptr(), S, span2)
    hit = _RANGE_CACHE.get(key)
    if hit is None:
        hit = (_bucket_ranges(luts[0], S, span2), _bucket_ranges(luts[1], S, span2))
        _RANGE_CACHE[key] = hit
    return hit


def _token_major(x: torch.Tensor) -> torch.Tensor:
    """[B,S,H] with unit inner stride, 16-byte aligned rows and batch stride = S · row stride (else a copy)."""
    B, S, H = x.shape
    if x.stride(2) != 1 or x.stride(0) != S * x.stride(1) or x.stride(1) % 8 or x.data_ptr() % 16:
        return x.contiguous()
    return x


# Both products of one side of the position-term gradient from ONE pass over the folded gradient table
# (csrc/posgrad.cu) instead of two batched GEMMs that each read it. Off: the two GEMMs (A/B comparisons, tests).
POSGRAD_DUAL = True


def _posgrad_dual(g, tab, x, out_f32, out_bf16, d_tab, heads: int, acc_in=None) -> bool:
    """``rows += g·tab`` (fp32 ``out_f32`` or bf16 ``out_bf16``) and ``d_tab += gᵀ·x`` per head in one kernel. ``g``:
    ``[T, heads, W]`` bf16, ``tab``: ``[W, heads*64]``, ``x``: ``[T, heads*64]`` rows (any row stride), ``d_tab``:
    ``[W, heads*64]`` fp32. With ``acc_in`` (fp32 ``[T, heads*64]``) the bf16 rows become ``acc_in + g·tab``, rounded
    once. Returns False when the shape is not covered (W other than 256 / 512) or the path is off."""
    T, _, W = g.shape
    if not POSGRAD_DUAL or W not in (256, 512) or not g.is_contiguous() or tab.shape[0] != W or tab.stride(1) != 1:
        return False
    out = out_f32 if out_f32 is not None else out_bf16
    rc = _lib.call_rc(
        "db200_posgrad_dual", _lib.ptr(g), c_ll(heads * W), _lib.ptr(tab), c_ll(tab.stride(0)), _lib.ptr(x),
        c_ll(x.stride(0)), _lib.ptr(out_f32), c_ll(out.stride(0) if out_f32 is not None else 0), _lib.ptr(out_bf16),
        c_ll(out.stride(0) if out_bf16 is not None else 0), _lib.ptr(acc_in),
        c_ll(acc_in.stride(0) if acc_in is not None else 0), _lib.ptr(d_tab), c_ll(d_tab.stride(0)), c_int(T),
        c_int(heads), c_int(W), _lib.stream_ptr(), accept=(_TC_REJECTED,))
    return rc == 0


def _heads_view(x2: torch.Tensor, heads: int) -> torch.Tensor:
    """[rows, H] (row stride ld) → [heads, rows, 64] view for the batched GEMM."""
    rows, H = x2.shape
    return x2.as_strided((heads, rows, H // heads), (H // heads, x2.stride(0), 1), x2.storage_offset())


def _common_ok(q, k, v, heads, pair_keep, dropout_p, training) -> bool:
    return (
        q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
        and pair_keep is None and not (training and dropout_p > 0.0)
        and q.dim() == 3 and q.shape == k.shape == v.shape and q.shape[-1] == heads * 64
    )


def disentangled_supported(q, k, v, pos_k, pos_q, heads, pair_keep, dropout_p, training, rel_pos) -> bool:
    if not _common_ok(q, k, v, heads, pair_keep, dropout_p, training) or rel_pos is not None:
        return False
    has_pos = pos_k is not None or pos_q is not None
    return not has_pos or (q.shape[1] <= 4096 and all(t is None or t.shape[0] <= 32767 for t in (pos_k, pos_q)))


def rope_supported(q, k, v, heads, rotary_dim, pair_keep, dropout_p, training) -> bool:
    return _common_ok(q, k, v, heads, pair_keep, dropout_p, training)


def _score_tables(q, k, pos_k, pos_q, heads: int):
    """``C2P = Q·PosKᵀ`` and ``P2C = K·PosQᵀ`` as ``[tokens, heads, 2·span]`` bf16 tables (batched GEMM per head)."""
    B, S, H = q.shape
    T = B * S
    q2 = q.as_strided((T, H), (q.stride(1), 1), q.storage_offset())
    k2 = k.as_strided((T, H), (k.stride(1), 1), k.storage_offset())
    c2p = p2c = None
    if pos_k is not None:
        c2p = torch.empty((T, heads, pos_k.shape[0]), dtype=torch.bfloat16, device=q.device)
        gemm(_heads_view(q2, heads), _heads_view(pos_k, heads), out=c2p.permute(1, 0, 2))
    if pos_q is not None:
        p2c = torch.empty((T, heads, pos_q.shape[0]), dtype=torch.bfloat16, device=q.device)
        gemm(_heads_view(k2, heads), _heads_view(pos_q, heads), out=p2c.permute(1, 0, 2))
    return c2p, p2c


def position_bias(q, k, pos_k, pos_q, luts, heads: int, tensor_core: bool | None = None):
    """Key-indexed position bias ``[B, heads, S, ldb]`` (unscaled, bf16) and whether the tensor-core kernel built it.

    ``q``/``k``: token-major ``[B, S, heads·64]`` bf16; ``pos_k``/``pos_q``: ``[2·span, heads·64]`` or ``None``.
    """
    B, S, _ = q.shape
    span2 = (pos_k if pos_k is not None else pos_q).shape[0]
    ldb = (S + 127) // 128 * 128
    bias = torch.empty((B, heads, S, ldb), dtype=torch.bfloat16, device=q.device)
    if POSBIAS_TENSOR_CORE if tensor_core is None else tensor_core:
        pa = _posbias_args(q, k, pos_k, pos_q, luts, heads, span2)
        pa.bias, pa.ldb = bias.data_ptr(), ldb
        if _lib.call_rc("db200_posbias_tc_fwd", ctypes.byref(pa), _lib.stream_ptr(), accept=(_TC_REJECTED,)) == 0:
            return bias, True
    c2p, p2c = _score_tables(q, k, pos_k, pos_q, heads)
    _lib.call("db200_posbias_build", _lib.ptr(c2p), _lib.ptr(p2c), _lib.ptr(luts[0]), _lib.ptr(luts[1]),
              _lib.ptr(bias), c_int(B), c_int(S), c_int(ldb), c_int(heads), c_int(span2), _lib.stream_ptr())
    return bias, False


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, pos_k, pos_q, heads, scale, luts, key_keep, doc_ids):
        q, k, v = _token_major(q), _token_major(k), _token_major(v)
        B, S, H = q.shape
        T = B * S
        out = torch.empty((B, S, H), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((B, heads, S), dtype=torch.float32, device=q.device)
        c2p = p2c = None
        span2 = 0 if pos_k is None and pos_q is None else (pos_k if pos_k is not None else pos_q).shape[0]
        ldb = (S + 127) // 128 * 128
        bias = None
        tc_bias = False
        if span2 and S <= BIAS_MODE_MAX_SEQ:
            bias, tc_bias = position_bias(q, k, pos_k, pos_q, luts, heads)
        elif span2:
            c2p, p2c = _score_tables(q, k, pos_k, pos_q, heads)
        kk = None if key_keep is None else key_keep.to(torch.uint8).contiguous()
        dd = None if doc_ids is None else doc_ids.to(torch.int32).contiguous()
        tiles = None
        if dd is not None:  # id range of every 128-token tile: the kernels visit only tiles that share a document
            tiles = torch.empty((B, (S + 127) // 128, 2), dtype=torch.int32, device=q.device)
            _lib.call("db200_attn_doc_tiles", _lib.ptr(dd), _lib.ptr(tiles), c_int(B), c_int(S), _lib.stream_ptr())
        a = AttnArgs()
        a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
        a.ldq, a.ldk, a.ldv = q.stride(1), k.stride(1), v.stride(1)
        a.out, a.ldo, a.lse = out.data_ptr(), H, lse.data_ptr()
        a.B, a.S, a.heads, a.span2, a.scale = B, S, heads, (0 if bias is not None else span2), scale
        a.c2p = None if c2p is None else c2p.data_ptr()
        a.p2c = None if p2c is None else p2c.data_ptr()
        if bias is not None:
            a.bias, a.ldb = bias.data_ptr(), ldb
        elif span2:
            a.lut_c2p, a.lut_p2c = luts[0].data_ptr(), luts[1].data_ptr()
        a.key_keep = None if kk is None else kk.data_ptr()
        a.doc_ids = None if dd is None else dd.data_ptr()
        a.doc_tiles = None if tiles is None else tiles.data_ptr()
        _lib.call("db200_attn_fwd", ctypes.byref(a), _lib.stream_ptr())
        ctx.save_for_backward(q, k, v, out, lse, c2p, p2c, pos_k, pos_q, kk, dd, bias, tiles)
        ctx.meta = (heads, scale, luts, span2, tc_bias)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, c2p, p2c, pos_k, pos_q, kk, dd, bias, tiles = ctx.saved_tensors
        heads, scale, luts, span2, tc_bias = ctx.meta
        B, S, H = q.shape
        T = B * S
        dev = q.device
        dout = dout.contiguous()
        delta = torch.empty((B, heads, S), dtype=torch.float32, device=dev)
        dq_acc = torch.empty((T, H), dtype=torch.float32, device=dev)  # cleared by the delta kernel
        _lib.call("db200_attn_delta", _lib.ptr(dout), ctypes.c_longlong(H), _lib.ptr(out), ctypes.c_longlong(H),
                  _lib.ptr(delta), _lib.ptr(dq_acc), c_int(B), c_int(S), c_int(heads), _lib.stream_ptr())
        # dQ | dK | dV side by side in one [T, 3H] buffer: a fused QKV projection takes it as is
        dqkv = torch.empty((T, 3 * H), dtype=torch.bfloat16, device=dev)
        dk, dv = dqkv[:, H : 2 * H], dqkv[:, 2 * H :]
        d_c2p = torch.zeros((T, heads, span2), dtype=torch.float32, device=dev) if c2p is not None else None
        d_p2c = torch.zeros((T, heads, span2), dtype=torch.float32, device=dev) if p2c is not None else None
        # skipped tiles are never written: with document ids the bias gradient starts from zero
        dbias = (torch.zeros_like(bias) if tiles is not None else torch.empty_like(bias)) if bias is not None else None
        a = AttnArgs()
        a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
        a.ldq, a.ldk, a.ldv = q.stride(1), k.stride(1), v.stride(1)
        a.lse = lse.data_ptr()
        a.B, a.S, a.heads, a.span2, a.scale = B, S, heads, (0 if bias is not None else span2), scale
        a.c2p = None if c2p is None else c2p.data_ptr()
        a.p2c = None if p2c is None else p2c.data_ptr()
        if bias is not None:
            a.bias, a.dbias, a.ldb = bias.data_ptr(), dbias.data_ptr(), bias.shape[-1]
        elif span2:
            a.lut_c2p, a.lut_p2c = luts[0].data_ptr(), luts[1].data_ptr()
        a.key_keep = None if kk is None else kk.data_ptr()
        a.doc_ids = None if dd is None else dd.data_ptr()
        a.doc_tiles = None if tiles is None else tiles.data_ptr()
        a.dout, a.ld_do, a.delta = dout.data_ptr(), H, delta.data_ptr()
        a.dq_acc, a.dk, a.dv, a.ld_dk, a.ld_dv = dq_acc.data_ptr(), dk.data_ptr(), dv.data_ptr(), 3 * H, 3 * H
        a.d_c2p = None if d_c2p is None else d_c2p.data_ptr()
        a.d_p2c = None if d_p2c is None else d_p2c.data_ptr()
        _lib.call("db200_attn_bwd", ctypes.byref(a), _lib.stream_ptr())
        d_pos_k = d_pos_q = None
        g_c2p = None if d_c2p is None else d_c2p.to(torch.bfloat16)
        g_p2c = None if d_p2c is None else d_p2c.to(torch.bfloat16)
        tc_done = False
        if bias is not None and POSBIAS_TENSOR_CORE_BWD:
            # fold the bias gradient onto the bucket axis and multiply it into dQ, dK and the table gradients in one kernel
            pa = _posbias_args(q, k, pos_k, pos_q, luts, heads, span2)
            pa.dbias, pa.ldb = dbias.data_ptr(), bias.shape[-1]
            pa.dq_acc, pa.dk, pa.ld_dk = dq_acc.data_ptr(), dk.data_ptr(), 3 * H
            gk = None if pos_k is None else torch.zeros(pos_k.shape, dtype=torch.float32, device=dev)
            gq = None if pos_q is None else torch.zeros(pos_q.shape, dtype=torch.float32, device=dev)
            pa.d_pos_k = None if gk is None else gk.data_ptr()
            pa.d_pos_q = None if gq is None else gq.data_ptr()
            if _lib.call_rc("db200_posbias_tc_bwd", ctypes.byref(pa), _lib.stream_ptr(), accept=(_TC_REJECTED,)) == 0:
                tc_done = True
                d_pos_k = None if gk is None else gk.to(pos_k.dtype)
                d_pos_q = None if gq is None else gq.to(pos_q.dtype)
        if bias is not None and not tc_done:  # reduce the key-indexed bias gradient back onto the bucket-indexed tables
            for which, tab in ((0, pos_k), (1, pos_q)):
                if tab is None:
                    continue
                gt = torch.empty((T, heads, span2), dtype=torch.bfloat16, device=dev)
                rng = _ranges(luts, S, span2)[which]
                if rng is not None:  # monotone bucket map: differences of prefix sums
                    _lib.call("db200_posbias_scatter_ranges", _lib.ptr(dbias), _lib.ptr(rng), _lib.ptr(gt), c_int(which),
                              c_int(B), c_int(S), c_int(bias.shape[-1]), c_int(heads), c_int(span2), _lib.stream_ptr())
                else:
                    _lib.call("db200_posbias_scatter", _lib.ptr(dbias), _lib.ptr(luts[which]), _lib.ptr(gt), c_int(which),
                              c_int(B), c_int(S), c_int(bias.shape[-1]), c_int(heads), c_int(span2), _lib.stream_ptr())
                if which == 0:
                    g_c2p = gt
                else:
                    g_p2c = gt
        q2 = q.as_strided((T, H), (q.stride(1), 1), q.storage_offset())
        k2 = k.as_strided((T, H), (k.stride(1), 1), k.storage_offset())
        # the two table gradients accumulate in fp32 (split-K over the tokens: measured faster than one bf16 pass that can
        # only use 48 CTAs); side by side in one buffer when both exist, so that one fill serves both
        both = g_c2p is not None and g_p2c is not None and pos_k.shape == pos_q.shape and pos_k.dtype == pos_q.dtype
        acc = torch.zeros((2, *pos_k.shape), dtype=torch.float32, device=dev) if both else None
        dq_done = False
        if g_c2p is not None:
            # dQ += dC2P · PosK ; dPosK = dC2Pᵀ · Q   (per head)
            d_pos_k = acc[0] if both else torch.zeros(pos_k.shape, dtype=torch.float32, device=dev)
            # (the query rows leave as bf16 = fp32 accumulator of the attention kernel + this product: no cast pass)
            dq_done = _posgrad_dual(g_c2p, pos_k, q2, None, dqkv[:, :H], d_pos_k, heads, acc_in=dq_acc)
            if not dq_done:
                g = g_c2p.permute(1, 0, 2)  # [heads, T, span2]
                gemm(g, _heads_view(pos_k, heads), b_mn=True, out=_heads_view(dq_acc, heads), accumulate=True)
                gemm(g, _heads_view(q2, heads), a_mn=True, b_mn=True, out=_heads_view(d_pos_k, heads), accumulate=True)
            if not both:
                d_pos_k = d_pos_k.to(pos_k.dtype)
        if g_p2c is not None:
            # dK += dP2C · PosQ ; dPosQ = dP2Cᵀ · K   (per head)
            d_pos_q = acc[1] if both else torch.zeros(pos_q.shape, dtype=torch.float32, device=dev)
            if not _posgrad_dual(g_p2c, pos_q, k2, None, dk, d_pos_q, heads):
                g = g_p2c.permute(1, 0, 2)
                dkh = _heads_view(dk, heads)
                gemm(g, _heads_view(pos_q, heads), b_mn=True, residual=dkh, out=dkh)  # added in the GEMM epilogue
                gemm(g, _heads_view(k2, heads), a_mn=True, b_mn=True, out=_heads_view(d_pos_q, heads), accumulate=True)
            if not both:
                d_pos_q = d_pos_q.to(pos_q.dtype)
        if both:  # (two casts: the outputs of a custom op must not alias each other)
            d_pos_k, d_pos_q = acc[0].to(pos_k.dtype), acc[1].to(pos_q.dtype)
        dq = dqkv[:, :H]
        if not dq_done:
            _lib.call("db200_cast_f32_bf16", _lib.ptr(dq_acc), _lib.ptr(dq), ctypes.c_longlong(3 * H), ctypes.c_longlong(T),
                      c_int(H), _lib.stream_ptr())
        return dq.view(B, S, H), dk.view(B, S, H), dv.view(B, S, H), d_pos_k, d_pos_q, None, None, None, None, None


class _Ctx:
    """What ``_FlashAttention.forward`` / ``backward`` need from an autograd context, for calls outside autograd."""

    saved_tensors: tuple = ()
    meta: tuple = ()

    def save_for_backward(self, *tensors) -> None:
        self.saved_tensors = tensors


def attention_forward(q, k, v, pos_k, pos_q, key_keep, doc_ids, heads: int, scale: float, bucket_size: int,
                      max_position: int, att_span: int):
    """Body of the ``db200::flash_attn`` op: (context, log-sum-exp, position bias or an empty tensor)."""
    luts = _luts(q.shape[1], bucket_size, max_position, att_span, q.device) if (pos_k is not None or pos_q is not None) else None
    ctx = _Ctx()
    out = _FlashAttention.forward(ctx, q, k, v, pos_k, pos_q, heads, scale, luts, key_keep, doc_ids)
    lse, bias = ctx.saved_tensors[4], ctx.saved_tensors[11]
    return out, lse, (bias if bias is not None else q.new_empty((0,)))


def attention_backward(dout, q, k, v, out, lse, bias, pos_k, pos_q, key_keep, doc_ids, heads: int, scale: float,
                       bucket_size: int, max_position: int, att_span: int):
    """Body of ``db200::flash_attn_bwd``: (dq, dk, dv, dpos_k, dpos_q); what the forward kept beside its outputs (score
    tables of the gather mode, the document-tile table) is rebuilt here."""
    has_pos = pos_k is not None or pos_q is not None
    luts = _luts(q.shape[1], bucket_size, max_position, att_span, q.device) if has_pos else None
    q, k, v = _token_major(q), _token_major(k), _token_major(v)
    B, S, _ = q.shape
    bias = bias if bias.numel() else None
    span2 = (pos_k if pos_k is not None else pos_q).shape[0] if has_pos else 0
    c2p = p2c = None
    if has_pos and bias is None:
        c2p, p2c = _score_tables(q, k, pos_k, pos_q, heads)
    kk = None if key_keep is None else key_keep.to(torch.uint8).contiguous()
    dd = None if doc_ids is None else doc_ids.to(torch.int32).contiguous()
    tiles = None
    if dd is not None:
        tiles = torch.empty((B, (S + 127) // 128, 2), dtype=torch.int32, device=q.device)
        _lib.call("db200_attn_doc_tiles", _lib.ptr(dd), _lib.ptr(tiles), c_int(B), c_int(S), _lib.stream_ptr())
    ctx = _Ctx()
    ctx.saved_tensors = (q, k, v, out, lse, c2p, p2c, pos_k, pos_q, kk, dd, bias, tiles)
    ctx.meta = (heads, scale, luts, span2, bias is not None)
    dq, dk, dv, dpk, dpq = _FlashAttention.backward(ctx, dout)[:5]
    e = lambda t: t if t is not None else q.new_empty((0,))  # noqa: E731
    return dq.contiguous(), dk.contiguous(), dv.contiguous(), e(dpk), e(dpq)


def disentangled_attention_cuda(q, k, v, pos_k, pos_q, *, heads, scale_factor, bucket_size, max_position, att_span,
                                key_keep=None, doc_ids=None) -> torch.Tensor:
    d = q.shape[-1] // heads
    scale = math.sqrt(float(d * scale_factor))
    luts = None
    if pos_k is not None or pos_q is not None:
        # (no slice when the table already has 2·span rows: the slice's backward would zero-fill and copy it)
        trim = lambda t: t if t is None or (t.shape[0] == 2 * att_span and t.is_contiguous()) else t[: 2 * att_span].contiguous()  # noqa: E731
        pos_k, pos_q = trim(pos_k), trim(pos_q)
    if torch.compiler.is_compiling():
        from . import library

        return library.flash_attn(q, k, v, pos_k, pos_q, key_keep, doc_ids, heads, scale, bucket_size, max_position,
                                  att_span)[0]
    if pos_k is not None or pos_q is not None:
        luts = _luts(q.shape[1], bucket_size, max_position, att_span, q.device)
    return _FlashAttention.apply(q, k, v, pos_k, pos_q, heads, scale, luts, key_keep, doc_ids)


def _rotate_rows(x2, out, cos, sin, S: int, heads: int, head_dim: int, rotary_dim: int, inverse: bool) -> None:
    """Rotary kernel over ``[rows, heads·head_dim]`` row views (``out`` may be ``x2``: in place)."""
    _lib.call("db200_rotary_bf16", _lib.ptr(x2), _lib.ptr(out), ctypes.c_longlong(x2.stride(0)),
              ctypes.c_longlong(out.stride(0)), _lib.ptr(cos), _lib.ptr(sin), ctypes.c_longlong(x2.shape[0]), c_int(S),
              c_int(heads), c_int(head_dim), c_int(rotary_dim), c_int(int(inverse)), _lib.stream_ptr())


class _RopeAttention(torch.autograd.Function):
    """Rotation of q and k + flash attention as one autograd node. Forward: q and k, which a fused QKV projection
    leaves side by side, are rotated by ONE launch into a ``[tokens, 2H]`` buffer. Backward: the attention kernel writes
    dQ | dK | dV side by side and the inverse rotation runs in place on the first two thirds of that buffer, so the QKV
    projection's backward receives one ``[tokens, 3H]`` tensor without a concatenation."""

    @staticmethod
    def forward(ctx, q, k, v, cos, sin, heads, rotary_dim, key_keep, doc_ids):
        q, k, v = _token_major(q), _token_major(k), _token_major(v)
        B, S, H = q.shape
        T, d = B * S, H // heads
        rows = lambda t: t.as_strided((T, H), (t.stride(1), 1), t.storage_offset())  # noqa: E731
        qk = torch.empty((T, 2 * H), dtype=q.dtype, device=q.device)
        if q.stride(1) == k.stride(1) and k.data_ptr() == q.data_ptr() + H * q.element_size():
            both = q.as_strided((T, 2 * H), (q.stride(1), 1), q.storage_offset())
            _rotate_rows(both, qk, cos, sin, S, 2 * heads, d, rotary_dim, False)
        else:
            _rotate_rows(rows(q), qk[:, :H], cos, sin, S, heads, d, rotary_dim, False)
            _rotate_rows(rows(k), qk[:, H:], cos, sin, S, heads, d, rotary_dim, False)
        qr = qk.as_strided((B, S, H), (S * 2 * H, 2 * H, 1), 0)
        kr = qk.as_strided((B, S, H), (S * 2 * H, 2 * H, 1), H)
        inner = _Ctx()
        out = _FlashAttention.forward(inner, qr, kr, v, None, None, heads, math.sqrt(float(d)), None, key_keep, doc_ids)
        # through save_for_backward, not as attributes: the saved set contains this node's own output, and an attribute
        # would close a reference cycle (node -> output -> node) that only the garbage collector could free
        ctx.save_for_backward(cos, sin, *inner.saved_tensors)
        ctx.inner_meta = inner.meta
        ctx.rot = (heads, rotary_dim)
        return out

    @staticmethod
    def backward(ctx, dout):
        heads, rotary_dim = ctx.rot
        cos, sin, *saved = ctx.saved_tensors
        inner = _Ctx()
        inner.saved_tensors = tuple(saved)
        inner.meta = ctx.inner_meta
        dq, dk, dv = _FlashAttention.backward(inner, dout)[:3]
        B, S, H = dq.shape
        # dq and dk are the first two column blocks of one [tokens, 3H] buffer: rotate both back where they are
        both = dq.as_strided((B * S, 2 * H), (dq.stride(1), 1), dq.storage_offset())
        _rotate_rows(both, both, cos, sin, S, 2 * heads, H // heads, rotary_dim, True)
        return dq, dk, dv, None, None, None, None, None, None


def rope_attention_cuda(q, k, v, cos, sin, *, heads, rotary_dim, key_keep=None, doc_ids=None) -> torch.Tensor:
    """Rotary attention: interleaved-pair rotation of q and k, then the same flash kernel without position tables."""
    B, S, H = q.shape
    d = H // heads
    if torch.compiler.is_compiling():
        from . import library
        from .elementwise import rotary_tokens

        if rotary_dim > 0:
            q = rotary_tokens(q, cos, sin, heads=heads, rotary_dim=rotary_dim)
            k = rotary_tokens(k, cos, sin, heads=heads, rotary_dim=rotary_dim)
        return library.flash_attn(q, k, v, None, None, key_keep, doc_ids, heads, math.sqrt(float(d)), 0, 0, 0)[0]
    if rotary_dim > 0 and d % 8 == 0 and rotary_dim % 2 == 0:
        c = cos.detach().to(torch.float32).contiguous()
        s = sin.detach().to(torch.float32).contiguous()
        return _RopeAttention.apply(q, k, v, c, s, heads, rotary_dim, key_keep, doc_ids)
    if rotary_dim > 0:
        from .elementwise import rotary_tokens

        q = rotary_tokens(q, cos, sin, heads=heads, rotary_dim=rotary_dim)
        k = rotary_tokens(k, cos, sin, heads=heads, rotary_dim=rotary_dim)
    return _FlashAttention.apply(q, k, v, None, None, heads, math.sqrt(float(d)), None, key_keep, doc_ids)
