"""Out-of-bounds and race checks that need no sanitizer: canary-padded outputs and run-twice bit comparison.

Every kernel under test writes into a window of a larger, sentinel-filled allocation; the sentinels before, after and
between the rows of the window must survive. Kernels whose results do not depend on the order of atomic additions
must give bit-identical outputs on a second run; the ones that reduce with fp32 atomics are compared within rounding.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

from deberta_b200.ops import _lib
from deberta_b200.ops.gemm import EPI_GELU_GRAD, EPI_MUL, gemm, gemm_reference

pytestmark = pytest.mark.gpu

SENTINEL = -7.75  # exactly representable in bf16


def _rand(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _window(rows, cols, dtype, pad_rows=3, pad_cols=24):
    """(window view [rows, cols] with a padded row stride, whole buffer, mask of the cells outside the window)."""
    ld = cols + pad_cols
    ld += (-ld) % 8  # rows stay 16-byte aligned for bf16
    buf = torch.full((rows + 2 * pad_rows, ld), SENTINEL, dtype=dtype, device="cuda")
    view = buf[pad_rows:pad_rows + rows, :cols]
    outside = torch.ones_like(buf, dtype=torch.bool)
    outside[pad_rows:pad_rows + rows, :cols] = False
    return view, buf, outside


def _intact(buf, outside):
    return bool((buf[outside] == SENTINEL).all())


@pytest.mark.parametrize("M,N,K", [(384, 512, 256), (300, 200, 136), (130, 72, 64)])
def test_gemm_outputs_stay_inside_their_window(M, N, K):
    a, w, bias = _rand(M, K), _rand(N, K, scale=0.1, seed=1), _rand(N, seed=2)
    out, buf, outside = _window(M, N, torch.bfloat16)
    gemm(a, w, bias=bias, out=out)
    torch.cuda.synchronize()
    assert _intact(buf, outside)
    ref = gemm_reference(a, w, bias=bias, out_dtype=torch.float32)
    assert (out.float() - ref).abs().max() / ref.abs().max() < 2e-2
    # two-output epilogue: both windows
    o1, b1, m1 = _window(M, N, torch.bfloat16)
    o2, b2, m2 = _window(M, N, torch.bfloat16, pad_cols=40)
    gemm(a, w, bias=bias, epi=EPI_GELU_GRAD, out=o1, out2=o2)
    torch.cuda.synchronize()
    assert _intact(b1, m1) and _intact(b2, m2)
    # fp32 split-K accumulation into a window (weight-gradient form)
    dy, x = _rand(2048, N, scale=0.1, seed=3), _rand(2048, K, seed=4)
    g, bg, mg = _window(N, K, torch.float32)
    g.zero_()
    gemm(dy, x, a_mn=True, b_mn=True, out=g, accumulate=True)
    torch.cuda.synchronize()
    assert _intact(bg, mg)
    _lib.check_status()


def test_gemm_is_bitwise_repeatable_without_split_k():
    a, w = _rand(1024, 768), _rand(3072, 768, scale=0.05, seed=1)
    first = gemm(a, w)
    for _ in range(3):
        assert torch.equal(gemm(a, w), first)
    g1, a1 = gemm(a, w, epi=EPI_GELU_GRAD)
    g2, a2 = gemm(a, w, epi=EPI_GELU_GRAD)
    assert torch.equal(g1, g2) and torch.equal(a1, a2)
    dy = _rand(1024, 768, seed=2)
    w2 = _rand(768, 3072, scale=0.05, seed=3)
    assert torch.equal(gemm(dy, w2, b_mn=True, epi=EPI_MUL, aux=g1), gemm(dy, w2, b_mn=True, epi=EPI_MUL, aux=g1))
    # split-K reduces with fp32 atomics: equal within rounding, not necessarily bit for bit
    x = _rand(16384, 768, seed=4)
    dyl = _rand(16384, 768, scale=0.1, seed=5)
    r1 = gemm(dyl, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
    r2 = gemm(dyl, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
    assert (r1 - r2).abs().max() <= 1e-4 * r1.abs().max()
    _lib.check_status()


@pytest.mark.parametrize("mask", ["none", "pad", "doc"])
def test_attention_forward_is_bitwise_repeatable_and_backward_within_rounding(mask):
    from deberta_b200.ops.attention import disentangled_attention

    B, S, heads, span = 2, 384, 2, 256
    q, k, v = (_rand(B, S, heads * 64, scale=0.5, seed=s).requires_grad_(True) for s in (0, 1, 2))
    pk, pq = (_rand(2 * span, heads * 64, scale=0.5, seed=s).requires_grad_(True) for s in (3, 4))
    kw = {}
    if mask == "pad":
        keep = torch.ones(B, S, dtype=torch.bool, device="cuda")
        keep[1, 300:] = False
        kw["key_keep"] = keep
    elif mask == "doc":
        doc = torch.ones(B, S, dtype=torch.long, device="cuda")
        doc[:, 150:] = 2
        doc[0, 350:] = 0
        kw["doc_ids"] = doc
    run = lambda: disentangled_attention(q, k, v, pk, pq, heads=heads, scale_factor=3, bucket_size=256,  # noqa: E731
                                         max_position=512, att_span=span, **kw)
    o1, o2 = run(), run()
    assert torch.equal(o1, o2)
    w = torch.randn_like(o1)
    grads = []
    for o in (o1, o2):
        for t in (q, k, v, pk, pq):
            t.grad = None
        (o.float() * w.float()).sum().backward()
        grads.append([t.grad.clone() for t in (q, k, v, pk, pq)])
    names = "q k v pos_k pos_q".split()
    for n, a, b in zip(names, *grads):
        if n in ("k", "v"):
            assert torch.equal(a, b), n  # accumulated in TMEM by one CTA per key tile: order is fixed
        else:
            assert (a.float() - b.float()).abs().max() <= 2e-2 * a.float().abs().max() + 1e-6, n  # fp32 atomics across CTAs
    _lib.check_status()


def test_position_bias_kernels_stay_inside_their_buffers_and_repeat():
    from deberta_b200.ops.attention_cuda import _luts, _ranges

    B, S, h, span2 = 2, 256, 3, 512
    c_int = ctypes.c_int
    luts = _luts(S, 256, 512, 256, torch.device("cuda"))
    edges = _ranges(luts, S, span2)
    c2p, p2c = _rand(B * S, h, span2, seed=1), _rand(B * S, h, span2, seed=2)
    n = B * h * S * S
    buf = torch.full((n + 512,), SENTINEL, dtype=torch.bfloat16, device="cuda")
    bias = buf[256:256 + n].view(B, h, S, S)
    call = lambda: _lib.call("db200_posbias_build", _lib.ptr(c2p), _lib.ptr(p2c), _lib.ptr(luts[0]), _lib.ptr(luts[1]),  # noqa: E731
                             _lib.ptr(bias), c_int(B), c_int(S), c_int(S), c_int(h), c_int(span2), _lib.stream_ptr())
    call()
    first = bias.clone()
    call()
    torch.cuda.synchronize()
    assert torch.equal(first, bias) and bool((buf[:256] == SENTINEL).all()) and bool((buf[256 + n:] == SENTINEL).all())
    dbias = _rand(B, h, S, S, seed=3)
    m = B * S * h * span2
    for which in (0, 1):
        tab = torch.full((m + 512,), SENTINEL, dtype=torch.bfloat16, device="cuda")
        dst = tab[256:256 + m]
        outs = []
        for _ in range(2):
            _lib.call("db200_posbias_scatter_ranges", _lib.ptr(dbias), _lib.ptr(edges[which]), _lib.ptr(dst), c_int(which),
                      c_int(B), c_int(S), c_int(S), c_int(h), c_int(span2), _lib.stream_ptr())
            outs.append(dst.clone())
        torch.cuda.synchronize()
        assert torch.equal(outs[0], outs[1])  # prefix sums in a fixed order: no atomics
        assert bool((tab[:256] == SENTINEL).all()) and bool((tab[256 + m:] == SENTINEL).all())
    _lib.check_status()


def test_norm_and_vocab_head_repeat_bit_for_bit():
    from deberta_b200.ops.heads import mlm_loss_and_sample
    from deberta_b200.ops.norm import layer_norm, rms_norm

    x = _rand(1000, 768, seed=1)
    w, b = _rand(768, seed=2), _rand(768, seed=3)
    assert torch.equal(layer_norm(x, w, b, 1e-7), layer_norm(x, w, b, 1e-7))
    assert torch.equal(rms_norm(x, w, 1e-6), rms_norm(x, w, 1e-6))
    h = _rand(500, 768, scale=0.5, seed=4)
    table = _rand(4096, 768, scale=0.05, seed=5)
    labels = torch.randint(5, 4096, (500,), device="cuda")
    l1, _ = mlm_loss_and_sample(h, table, None, labels, None, 1.0)
    l2, _ = mlm_loss_and_sample(h, table, None, labels, None, 1.0)
    assert torch.equal(l1, l2)  # the loss does not depend on the sampling seed, and its reduction order is fixed
    _lib.check_status()


def test_dependent_launch_chains_match_ordinary_launches_bit_for_bit():
    """A chain of short kernels in which each one reads what the previous one wrote and overwrites what the one before
    that read (GEMM -> LayerNorm -> GEMM -> cast, ping-ponging two buffers, 40 rounds, plus a backward chain): with
    programmatic dependent launch the kernels' set-up overlaps their predecessors, and the results must still be the
    ones of ordinary stream-ordered launches, bit for bit, every time."""
    from deberta_b200.ops.linear import linear
    from deberta_b200.ops.norm import layer_norm

    T, H = 2048, 768
    x0 = _rand(T, H, seed=3)
    w1, w2 = _rand(H, H, scale=0.03, seed=4), _rand(H, H, scale=0.03, seed=5)
    b1 = _rand(H, scale=0.1, seed=6)
    gamma, beta = _rand(H, seed=7) * 0 + 1, _rand(H, scale=0.1, seed=8)

    def chain():
        torch.manual_seed(0)
        x = x0.clone().requires_grad_(True)
        h = x
        for _ in range(40):
            h = layer_norm(linear(h, w1, b1, residual=h), gamma, beta, 1e-6)
            h = linear(h, w2, None)
        (h.float().square().mean()).backward()
        return h.detach().clone(), x.grad.detach().clone()

    old = _lib.set_dependent_launch(False)
    try:
        ref = chain()
        _lib.set_dependent_launch(True)
        for _ in range(3):
            got = chain()
            assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1])
    finally:
        _lib.set_dependent_launch(old)
    _lib.check_status()
