"""sm_100a attention kernels vs. the fp32 PyTorch statements of the same operators (forward and gradients)."""

from __future__ import annotations

import pytest
import torch

from deberta_b200.ops import _lib
from deberta_b200.ops.attention import (disentangled_attention, disentangled_attention_reference, relative_positions,
                                        rope_attention, rope_attention_reference)

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=[64, 65, 128], ids=["kt64ws", "kt64", "kt128"])
def forward_key_tile(request):
    """Every case runs on the three forward kernels: 64 keys per tile with a dedicated TMA/MMA warp (the default where
    it applies), 64 keys per tile with block-wide barriers (65), and 128 keys per tile (one CTA per SM). The backward
    kernel runs with one CTA per SM walking the work items (the default), with one CTA per item, and with at most three
    CTAs, so that on these small inputs every CTA goes through several items."""
    from deberta_b200.ops.attention_cuda import set_backward_persistent, set_forward_key_tile

    old = set_forward_key_tile(request.param)
    old_bwd = set_backward_persistent({64: 1, 65: 0, 128: 3}[request.param])
    yield request.param
    set_forward_key_tile(old)
    set_backward_persistent(old_bwd)


def _rel_err(got, ref):
    return (got.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-6)


def _inputs(B, S, heads, span, seed=0, scale=0.5):
    g = torch.Generator(device="cuda").manual_seed(seed)
    H = heads * 64
    mk = lambda *s: (torch.randn(*s, device="cuda", generator=g) * scale).to(torch.bfloat16).requires_grad_(True)  # noqa: E731
    return mk(B, S, H), mk(B, S, H), mk(B, S, H), mk(2 * span, H), mk(2 * span, H)


def _set_position_mode(monkeypatch, mode):
    """"tc": bias and its gradient by the tensor-core tile kernels; "tc_fwd": bias by the tile kernel, gradient by
    prefix-sum scans (the default); "bias": bias pre-gathered from score tables, gradient by scans; "gather": bucket
    tables read inside the attention kernels."""
    from deberta_b200.ops import attention_cuda

    monkeypatch.setattr(attention_cuda, "BIAS_MODE_MAX_SEQ", 0 if mode == "gather" else 1024)
    monkeypatch.setattr(attention_cuda, "POSBIAS_TENSOR_CORE", mode in ("tc", "tc_fwd"))
    monkeypatch.setattr(attention_cuda, "POSBIAS_TENSOR_CORE_BWD", mode == "tc")


@pytest.mark.parametrize("mode", ["tc", "tc_fwd", "bias", "gather"])
@pytest.mark.parametrize("B,S,heads,mask", [(2, 512, 2, "none"), (2, 200, 3, "pad"), (1, 384, 2, "doc"), (2, 128, 1, "none")])
def test_disentangled_forward_backward(B, S, heads, mask, mode, monkeypatch):
    _set_position_mode(monkeypatch, mode)
    span, buckets, maxpos = 256, 256, 512
    q, k, v, pk, pq = _inputs(B, S, heads, span)
    kw = {}
    if mask == "pad":
        keep = torch.ones(B, S, dtype=torch.bool, device="cuda")
        keep[0, S - 37:] = False
        kw["key_keep"] = keep
    elif mask == "doc":
        doc = torch.ones(B, S, dtype=torch.long, device="cuda")
        doc[:, 100:] = 2
        doc[:, 300:] = 3
        doc[:, S - 20:] = 0
        kw["doc_ids"] = doc
    out = disentangled_attention(q, k, v, pk, pq, heads=heads, scale_factor=3, bucket_size=buckets, max_position=maxpos,
                                 att_span=span, **kw)
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, k, v, pk, pq)]
    ref = disentangled_attention_reference(*ref_in, heads=heads, scale_factor=3,
                                           rel_pos=relative_positions(S, S, buckets, maxpos, device="cuda"),
                                           att_span=span, **kw)
    _lib.check_status()
    assert _rel_err(out, ref) < 2e-2
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    _lib.check_status()
    for name, a, b in zip("q k v pos_k pos_q".split(), (q, k, v, pk, pq), ref_in):
        assert _rel_err(a.grad, b.grad) < 4e-2, name


@pytest.mark.parametrize("S,mask", [(256, "none"), (1000, "doc"), (320, "pad")])
def test_rope_forward_backward(S, mask):
    B, heads = 2, 2
    q, k, v, _, _ = _inputs(B, S, heads, 8, seed=3)
    inv = 1.0 / (10000 ** (torch.arange(0, 64, 2, device="cuda").float() / 64))
    ang = torch.repeat_interleave(torch.outer(torch.arange(S, device="cuda").float(), inv), 2, dim=-1)
    cos, sin = ang.cos(), ang.sin()
    kw = {}
    if mask == "doc":
        doc = torch.ones(B, S, dtype=torch.long, device="cuda")
        doc[:, 333:] = 2
        doc[1, 700:] = 3
        doc[0, 990:] = 0
        kw["doc_ids"] = doc
    elif mask == "pad":
        keep = torch.ones(B, S, dtype=torch.bool, device="cuda")
        keep[1, 250:] = False
        kw["key_keep"] = keep
    out = rope_attention(q, k, v, cos, sin, heads=heads, rotary_dim=64, **kw)
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = rope_attention_reference(*ref_in, cos, sin, heads=heads, rotary_dim=64, **kw)
    _lib.check_status()
    assert _rel_err(out, ref) < 2e-2
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    _lib.check_status()
    for name, a, b in zip("qkv", (q, k, v), ref_in):
        assert _rel_err(a.grad, b.grad) < 4e-2, name


@pytest.mark.parametrize("rotary_dim", [64, 32])
def test_rope_attention_on_side_by_side_qkv_rotates_in_one_launch_and_in_place(rotary_dim):
    """q, k, v as the three column blocks of one [B, S, 3H] projection (what the fused QKV GEMM produces): the rotation
    of q and k is one launch, the gradients come back as views of one [tokens, 3H] buffer (rotated back in place), and
    both match the fp32 statement, also with a partial rotary dimension."""
    B, S, heads = 2, 384, 3
    H = heads * 64
    g = torch.Generator(device="cuda").manual_seed(9)
    qkv = (torch.randn(B, S, 3 * H, device="cuda", generator=g) * 0.5).to(torch.bfloat16).requires_grad_(True)
    q, k, v = qkv[..., :H], qkv[..., H:2 * H], qkv[..., 2 * H:]
    inv = 1.0 / (10000 ** (torch.arange(0, rotary_dim, 2, device="cuda").float() / rotary_dim))
    ang = torch.repeat_interleave(torch.outer(torch.arange(S, device="cuda").float(), inv), 2, dim=-1)
    cos, sin = ang.cos(), ang.sin()
    out = rope_attention(q, k, v, cos, sin, heads=heads, rotary_dim=rotary_dim)
    ref_qkv = qkv.detach().float().requires_grad_(True)
    ref = rope_attention_reference(ref_qkv[..., :H], ref_qkv[..., H:2 * H], ref_qkv[..., 2 * H:], cos, sin, heads=heads,
                                   rotary_dim=rotary_dim)
    assert _rel_err(out, ref) < 2e-2
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    _lib.check_status()
    for lo, name in ((0, "q"), (H, "k"), (2 * H, "v")):
        assert _rel_err(qkv.grad[..., lo:lo + H], ref_qkv.grad[..., lo:lo + H]) < 4e-2, name


def _packed_doc_ids(B, S, mean_len, seed, tail_pad=0, shuffle_ids=False):
    g = torch.Generator().manual_seed(seed)
    doc = torch.zeros(B, S, dtype=torch.long)
    for b in range(B):
        pos, d = 0, 1
        while pos < S - tail_pad:
            n = int(torch.randint(max(1, mean_len // 2), mean_len * 2, (1,), generator=g))
            doc[b, pos:min(S - tail_pad, pos + n)] = d
            pos, d = pos + n, d + 1
        if shuffle_ids:  # ids need not grow along the row: relabel the documents at random
            perm = torch.randperm(d, generator=g) + 1
            live = doc[b] > 0
            doc[b, live] = perm[doc[b, live] - 1]
    return doc.cuda()


@pytest.mark.parametrize("S,mean_len,tail_pad,shuffle", [(1024, 60, 0, False), (1024, 200, 300, False), (768, 90, 140, True),
                                                         (2048, 150, 0, False), (4300, 500, 200, False)])  # 34 tiles: two ballots
def test_rope_packed_documents_skip_tiles(S, mean_len, tail_pad, shuffle):
    """Many short documents per row: most tile pairs share no document and are skipped; results must not change."""
    B, heads = 2, 2
    q, k, v, _, _ = _inputs(B, S, heads, 8, seed=5)
    inv = 1.0 / (10000 ** (torch.arange(0, 64, 2, device="cuda").float() / 64))
    ang = torch.repeat_interleave(torch.outer(torch.arange(S, device="cuda").float(), inv), 2, dim=-1)
    cos, sin = ang.cos(), ang.sin()
    doc = _packed_doc_ids(B, S, mean_len, seed=S + mean_len, tail_pad=tail_pad, shuffle_ids=shuffle)
    out = rope_attention(q, k, v, cos, sin, heads=heads, rotary_dim=64, doc_ids=doc)
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    ref = rope_attention_reference(*ref_in, cos, sin, heads=heads, rotary_dim=64, doc_ids=doc)
    _lib.check_status()
    assert _rel_err(out, ref) < 2e-2
    if tail_pad:
        assert float(out[:, S - tail_pad:].abs().max()) == 0.0  # padding queries give zero rows
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    _lib.check_status()
    for name, a, b in zip("qkv", (q, k, v), ref_in):
        assert _rel_err(a.grad, b.grad) < 4e-2, name


@pytest.mark.parametrize("mode,S", [("tc", 640), ("bias", 640), ("gather", 640)])
def test_disentangled_packed_documents_skip_tiles(mode, S, monkeypatch):
    _set_position_mode(monkeypatch, mode)
    B, heads, span, buckets, maxpos = 2, 2, 256, 256, 512
    q, k, v, pk, pq = _inputs(B, S, heads, span, seed=7)
    doc = _packed_doc_ids(B, S, 70, seed=11, tail_pad=150)
    out = disentangled_attention(q, k, v, pk, pq, heads=heads, scale_factor=3, bucket_size=buckets, max_position=maxpos,
                                 att_span=span, doc_ids=doc)
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, k, v, pk, pq)]
    ref = disentangled_attention_reference(*ref_in, heads=heads, scale_factor=3,
                                           rel_pos=relative_positions(S, S, buckets, maxpos, device="cuda"),
                                           att_span=span, doc_ids=doc)
    _lib.check_status()
    assert _rel_err(out, ref) < 2e-2
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    _lib.check_status()
    for name, a, b in zip("q k v pos_k pos_q".split(), (q, k, v, pk, pq), ref_in):
        assert _rel_err(a.grad, b.grad) < 4e-2, name


def test_document_tile_table_matches_pytorch():
    import ctypes

    B, S = 3, 1000
    doc = _packed_doc_ids(B, S, 50, seed=2, tail_pad=260, shuffle_ids=True).to(torch.int32)
    nt = (S + 127) // 128
    tiles = torch.empty(B, nt, 2, dtype=torch.int32, device="cuda")
    _lib.call("db200_attn_doc_tiles", _lib.ptr(doc), _lib.ptr(tiles), ctypes.c_int(B), ctypes.c_int(S), _lib.stream_ptr())
    padded = torch.zeros(B, nt * 128, dtype=torch.int32, device="cuda")
    padded[:, :S] = doc
    padded = padded.view(B, nt, 128)
    lo = torch.where(padded > 0, padded, torch.full_like(padded, 2**31 - 1)).amin(-1)
    hi = torch.where(padded > 0, padded, torch.full_like(padded, -1)).amax(-1)
    assert torch.equal(tiles[..., 0], lo) and torch.equal(tiles[..., 1], hi)
    assert int(tiles[0, -1, 1]) == -1  # the last tile of every row is padding only


def test_rope_packed_documents_speed_report():
    B, S, heads = 4, 4096, 12
    q, k, v, _, _ = _inputs(B, S, heads, 8, seed=9, scale=0.3)
    inv = 1.0 / (10000 ** (torch.arange(0, 64, 2, device="cuda").float() / 64))
    ang = torch.repeat_interleave(torch.outer(torch.arange(S, device="cuda").float(), inv), 2, dim=-1)
    cos, sin = ang.cos(), ang.sin()
    one = torch.ones(B, S, dtype=torch.long, device="cuda")
    packed = _packed_doc_ids(B, S, 300, seed=4)
    for label, doc in (("one document per row", one), ("packed, ~300-token documents", packed)):
        fn = lambda: rope_attention(q, k, v, cos, sin, heads=heads, rotary_dim=64, doc_ids=doc)  # noqa: E731,B023
        g = torch.randn_like(fn())
        for name, f in (("fwd", fn), ("fwd+bwd", lambda: fn().backward(g))):  # noqa: B023
            for _ in range(2):
                f()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(5):
                f()
            e.record()
            torch.cuda.synchronize()
            print(f"\n[rope attention B={B} S={S} h={heads}, {label}] {name}: {s.elapsed_time(e) / 5 * 1e3:.0f} us")
    _lib.check_status()


def test_attention_speed_report():
    B, S, heads, span = 32, 512, 12, 256
    q, k, v, pk, pq = _inputs(B, S, heads, span, scale=0.3)
    fn = lambda: disentangled_attention(q, k, v, pk, pq, heads=heads, scale_factor=3, bucket_size=256,  # noqa: E731
                                        max_position=512, att_span=span)
    out = fn()
    g = torch.randn_like(out)
    for label, f in (("fwd", fn), ("fwd+bwd", lambda: fn().backward(g))):
        for _ in range(2):
            f()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(5):
            f()
        e.record()
        torch.cuda.synchronize()
        print(f"\n[disentangled attention B={B} S={S} h={heads}] {label}: {s.elapsed_time(e) / 5 * 1e3:.0f} us")
    _lib.check_status()


def test_rotary_and_swiglu_kernels_match_pytorch():
    from deberta_b200.ops.attention import rotate_interleaved
    from deberta_b200.ops.elementwise import rotary_tokens, swiglu

    dev = torch.device("cuda")
    torch.manual_seed(0)
    B, S, heads, d, rot = 2, 100, 4, 64, 32
    x = (torch.randn(B, S, heads * d, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2, device=dev).float() / d))
    ang = torch.arange(S, device=dev).float()[:, None] * inv[None]
    emb = torch.repeat_interleave(ang, 2, dim=-1)
    cos, sin = emb.cos(), emb.sin()
    y = rotary_tokens(x, cos, sin, heads=heads, rotary_dim=rot)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    yr = rotate_interleaved(xr.reshape(B, S, heads, d), cos[None, :, None, :], sin[None, :, None, :], rot).reshape(B, S, -1)
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 2e-2
    assert (x.grad.float() - xr.grad).abs().max() < 3e-2
    # SwiGLU
    gu = (torch.randn(300, 2 * 256, device=dev)).to(torch.bfloat16).requires_grad_(True)
    out = swiglu(gu)
    go = torch.randn_like(out)
    out.backward(go)
    gr = gu.detach().float().requires_grad_(True)
    a, b = gr.chunk(2, dim=-1)
    ref = torch.nn.functional.silu(a) * b
    ref.backward(go.float())
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max()
    assert (gu.grad.float() - gr.grad).abs().max() <= 2e-2 * gr.grad.abs().max()


def _bias_reference(q, k, pos_k, pos_q, heads, S, buckets, maxpos, span):
    """fp32 statement of the position bias: Q·PosK[δ(q-k)+span] + K·PosQ[span-δ(q-k)] (unscaled)."""
    B = q.shape[0]
    rel = relative_positions(S, S, buckets, maxpos, device=q.device).clamp(-span, span)
    qh = q.float().view(B, S, heads, 64).permute(0, 2, 1, 3)
    kh = k.float().view(B, S, heads, 64).permute(0, 2, 1, 3)
    out = torch.zeros(B, heads, S, S, device=q.device)
    if pos_k is not None:
        pk = pos_k.float().view(2 * span, heads, 64).permute(1, 0, 2)
        c2p = torch.einsum("bhqd,hpd->bhqp", qh, pk)
        out = out + c2p.gather(-1, (rel + span).clamp(0, 2 * span - 1)[None, None].expand(B, heads, S, S))
    if pos_q is not None:
        pq = pos_q.float().view(2 * span, heads, 64).permute(1, 0, 2)
        p2c = torch.einsum("bhkd,hpd->bhkp", kh, pq)
        idx = (span - rel.transpose(0, 1)).clamp(0, 2 * span - 1)
        out = out + p2c.gather(-1, idx[None, None].expand(B, heads, S, S)).transpose(-1, -2)
    return out


@pytest.mark.parametrize("B,S,heads,span,buckets,maxpos,which", [
    (2, 512, 2, 256, 256, 512, "both"), (1, 200, 3, 256, 256, 512, "both"), (2, 128, 1, 256, 256, 512, "c2p"),
    (1, 384, 2, 256, 256, 512, "p2c"), (1, 1024, 1, 256, 256, 512, "both"), (2, 300, 2, 32, 32, 64, "both")])
def test_position_bias_on_tensor_cores_matches_fp32(B, S, heads, span, buckets, maxpos, which):
    from deberta_b200.ops import attention_cuda

    q, k, _, pk, pq = _inputs(B, S, heads, span, seed=13)
    q, k, pk, pq = (t.detach() for t in (q, k, pk, pq))
    if which == "c2p":
        pq = None
    if which == "p2c":
        pk = None
    luts = attention_cuda._luts(S, buckets, maxpos, span, q.device)
    bias, used = attention_cuda.position_bias(q, k, pk, pq, luts, heads, tensor_core=True)
    _lib.check_status()
    assert used, "the tensor-core kernel rejected a bucket map it is meant to cover"
    ref = _bias_reference(q, k, pk, pq, heads, S, buckets, maxpos, span)
    assert _rel_err(bias[..., :S], ref) < 1.5e-2
    table, used2 = attention_cuda.position_bias(q, k, pk, pq, luts, heads, tensor_core=False)
    assert not used2 and _rel_err(table[..., :S], ref) < 1.5e-2


@pytest.mark.parametrize("which,S,span,buckets,maxpos", [("c2p", 256, 256, 256, 512), ("p2c", 330, 256, 256, 512),
                                                         ("both", 1000, 256, 256, 512), ("both", 300, 32, 32, 64)])
def test_position_terms_single_sided_and_long_rows(which, S, span, buckets, maxpos, monkeypatch):
    """One position term at a time, a 1000-token row (runs of offsets that share a log bucket cross the 32-entry
    parts of the fold and the tiles), and a 64-row table (one window block)."""
    _set_position_mode(monkeypatch, "tc")
    B, heads = 1, 2
    q, k, v, pk, pq = _inputs(B, S, heads, span, seed=21)
    pos = {"c2p": (pk, None), "p2c": (None, pq), "both": (pk, pq)}[which]
    out = disentangled_attention(q, k, v, *pos, heads=heads, scale_factor=1 + sum(t is not None for t in pos),
                                 bucket_size=buckets, max_position=maxpos, att_span=span)
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, k, v, pk, pq)]
    ref_pos = [None if t is None else r for t, r in zip(pos, ref_in[3:])]
    ref = disentangled_attention_reference(*ref_in[:3], *ref_pos, heads=heads, scale_factor=1 + sum(t is not None for t in pos),
                                           rel_pos=relative_positions(S, S, buckets, maxpos, device="cuda"), att_span=span)
    _lib.check_status()
    assert _rel_err(out, ref) < 2e-2
    w = torch.randn_like(ref)
    (out.float() * w).sum().backward()
    (ref * w).sum().backward()
    _lib.check_status()
    for name, a, b in zip("q k v pos_k pos_q".split(), (q, k, v, pk, pq), ref_in):
        if b.grad is None:
            assert a.grad is None or float(a.grad.abs().max()) == 0.0, name
            continue
        assert _rel_err(a.grad, b.grad) < 4e-2, name


@pytest.mark.parametrize("T,heads,W", [(1000, 3, 512), (256, 2, 256), (130, 1, 512)])
def test_position_gradient_dual_kernel_matches_fp32(T, heads, W):
    """One pass over the folded gradient table gives both products of a side: rows += g·tab (fp32 accumulator for the
    query side, bf16 read-modify-write for the key side) and d_tab += gᵀ·x, per head; x and the bf16 rows are column
    slices of wider buffers, T is not a multiple of the 128-token tile, and what the outputs held before is kept."""
    from deberta_b200.ops import attention_cuda

    torch.manual_seed(11)
    H = heads * 64
    g = (torch.randn(T, heads, W, device="cuda") * 0.3).to(torch.bfloat16)
    tab = (torch.randn(W, H, device="cuda") * 0.3).to(torch.bfloat16)
    wide = (torch.randn(T, 3 * H, device="cuda") * 0.5).to(torch.bfloat16)
    x = wide[:, H : 2 * H]
    gf, tf, xf = g.float(), tab.float().view(W, heads, 64), x.float().reshape(T, heads, 64)
    want_rows = torch.einsum("thw,whd->thd", gf, tf).reshape(T, H)
    want_tab = torch.einsum("thw,thd->whd", gf, xf).reshape(W, H)
    # query side: fp32 accumulator
    acc = torch.full((T, H), 0.5, device="cuda")
    d_tab = torch.full((W, H), -1.0, device="cuda")
    assert attention_cuda._posgrad_dual(g, tab, x, acc, None, d_tab, heads)
    _lib.check_status()
    assert (acc - 0.5 - want_rows).abs().max() <= 2e-2 * want_rows.abs().max()
    assert (d_tab + 1.0 - want_tab).abs().max() <= 2e-2 * want_tab.abs().max()
    # query side as the training step runs it: bf16 rows = fp32 accumulator + product, rounded once
    acc_in = torch.randn(T, H, device="cuda")
    rows = torch.zeros(T, 3 * H, device="cuda", dtype=torch.bfloat16)
    d_tab3 = torch.zeros(W, H, device="cuda")
    assert attention_cuda._posgrad_dual(g, tab, x, None, rows[:, :H], d_tab3, heads, acc_in=acc_in)
    _lib.check_status()
    assert (rows[:, :H].float() - (acc_in + want_rows)).abs().max() <= 2e-2 * (acc_in + want_rows).abs().max()
    assert float(rows[:, H:].abs().max()) == 0.0
    # key side: bf16 rows inside a wider buffer, everything around them untouched
    out_wide = (torch.randn(T, 3 * H, device="cuda") * 0.5).to(torch.bfloat16)
    before = out_wide.clone()
    d_tab2 = torch.zeros(W, H, device="cuda")
    assert attention_cuda._posgrad_dual(g, tab, x, None, out_wide[:, H : 2 * H], d_tab2, heads)
    _lib.check_status()
    assert torch.equal(out_wide[:, :H], before[:, :H]) and torch.equal(out_wide[:, 2 * H :], before[:, 2 * H :])
    got = out_wide[:, H : 2 * H].float() - before[:, H : 2 * H].float()
    assert (got - want_rows).abs().max() <= 3e-2 * want_rows.abs().max()
    assert (d_tab2 - want_tab).abs().max() <= 2e-2 * want_tab.abs().max()
