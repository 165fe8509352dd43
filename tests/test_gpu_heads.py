"""Fused vocabulary cross-entropy + sampling kernel vs. the PyTorch statement."""

from __future__ import annotations

import pytest
import torch

from deberta_b200.ops import _lib
from deberta_b200.ops.heads import mlm_loss_and_sample, mlm_loss_and_sample_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("buffers", [False, True], ids=["grads", "main_grad"])
@pytest.mark.parametrize("N,V,E", [(300, 5000, 128), (77, 128100, 768), (130, 1000, 64)])
def test_vocab_ce_matches_reference(N, V, E, buffers):
    """``buffers``: the parameters carry the engine's fp32 accumulation buffers, so the table's gradient GEMM also sums
    the bias gradient (one launch) and both are ADDED to what the buffers held."""
    torch.manual_seed(0)
    x = (torch.randn(N, E, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(V, E, device="cuda") * 0.2).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn(V, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    if buffers:
        w.main_grad = torch.full((V, E), 0.25, dtype=torch.float32, device="cuda")
        b.main_grad = torch.full((V,), -0.5, dtype=torch.float32, device="cuda")
    labels = torch.randint(5, V, (N,), device="cuda")
    forb = torch.zeros(V, dtype=torch.bool, device="cuda")
    forb[:5] = True
    loss, sampled = mlm_loss_and_sample(x, w, b, labels, forb, 1.0)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    ref_loss, _ = mlm_loss_and_sample_reference(xr, wr, br, labels, forb, 1.0)
    _lib.check_status()
    assert abs(float(loss) - float(ref_loss)) / float(ref_loss) < 5e-3
    assert sampled.shape == (N,) and int(sampled.min()) >= 5 and int(sampled.max()) < V
    (loss * 3.0).backward()
    (ref_loss * 3.0).backward()
    _lib.check_status()
    got = {"x": x.grad.float()}
    if buffers:
        assert w.grad is None and b.grad is None
        got["w"], got["b"] = w.main_grad - 0.25, b.main_grad + 0.5
    else:
        got["w"], got["b"] = w.grad.float(), b.grad.float()
    for name, r in (("x", xr), ("w", wr), ("b", br)):
        err = (got[name] - r.grad).abs().max().item() / (r.grad.abs().max().item() + 1e-9)
        assert err < 3e-2, (name, err)


def test_sampling_follows_softmax():
    """With a sharply peaked distribution the Gumbel-max sample is the mode; with a flat one it spreads out."""
    torch.manual_seed(1)
    N, V, E = 512, 2048, 64
    w = torch.zeros(V, E, device="cuda", dtype=torch.bfloat16)
    x = torch.zeros(N, E, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(V, device="cuda", dtype=torch.bfloat16)
    b[100] = 30.0
    labels = torch.full((N,), 100, device="cuda")
    _, s = mlm_loss_and_sample(x, w, b, labels, None, 1.0)
    assert bool((s == 100).all())
    b[100] = 0.0
    _, s = mlm_loss_and_sample(x, w, b, labels, None, 1.0)
    assert s.unique().numel() > 300
    _, s2 = mlm_loss_and_sample(x, w, b, labels, None, 1.0)
    assert not torch.equal(s, s2)
    _lib.check_status()


def test_embedding_lookup_kernel_matches_pytorch():
    import torch
    from deberta_b200.ops.embedding import embedding_lookup

    dev = torch.device("cuda")
    torch.manual_seed(0)
    vocab, hidden = 1000, 256
    base = torch.nn.Parameter((torch.randn(vocab, hidden, device=dev) * 0.1).to(torch.bfloat16), requires_grad=False)
    delta = torch.nn.Parameter((torch.randn(vocab, hidden, device=dev) * 0.1).to(torch.bfloat16))
    delta.main_grad = torch.zeros(vocab, hidden, device=dev)
    ids = torch.randint(0, vocab, (4, 77), device=dev)
    ids[0, :20] = 5  # a hot row
    ids[1, :5] = 0   # padding
    out = embedding_lookup(ids, base, delta, padding_idx=0)
    ref = (base.float()[ids] + delta.float()[ids])
    assert (out.float() - ref).abs().max() <= 1e-2
    g = torch.randn_like(out)
    out.backward(g)
    want = torch.zeros(vocab, hidden, device=dev)
    keep = ids.reshape(-1) != 0
    want.index_add_(0, ids.reshape(-1)[keep], g.float().reshape(-1, hidden)[keep])
    assert (delta.main_grad - want).abs().max() <= 1e-3 * want.abs().max() + 1e-4
    assert float(delta.main_grad[0].abs().max()) == 0.0
    # single table, no autograd
    with torch.no_grad():
        out2 = embedding_lookup(ids, base)
    assert torch.equal(out2, base[ids])


def test_rtd_head_kernel_matches_composition():
    import torch
    from deberta_b200.ops.heads import rtd_loss
    from deberta_b200.ops.heads_cuda import rtd_head_loss_cuda, rtd_head_supported

    dev = torch.device("cuda")
    torch.manual_seed(0)
    B, S, H = 3, 50, 256
    x = (torch.randn(B, S, H, device=dev) * 0.7).to(torch.bfloat16).requires_grad_(True)
    dense_w = torch.nn.Parameter((torch.randn(H, H, device=dev) * 0.06).to(torch.bfloat16))
    dense_b = torch.nn.Parameter((torch.randn(H, device=dev) * 0.1).to(torch.bfloat16))
    cls_w = torch.nn.Parameter((torch.randn(1, H, device=dev) * 0.1).to(torch.bfloat16))
    cls_b = torch.nn.Parameter(torch.tensor([0.05], device=dev).to(torch.bfloat16))
    labels = (torch.rand(B, S, device=dev) < 0.2).float()
    active = torch.rand(B, S, device=dev) < 0.9
    assert rtd_head_supported(x, dense_w, cls_w, "gelu")
    loss, acc, count, pos = rtd_head_loss_cuda(x, dense_w, dense_b, cls_w, cls_b, labels, active)
    (loss * 3.0).backward()
    got = [x.grad.float(), dense_w.grad.float(), dense_b.grad.float(), cls_w.grad.float(), cls_b.grad.float()]
    xr = x.detach().float().requires_grad_(True)
    ps = [p.detach().float().requires_grad_(True) for p in (dense_w, dense_b, cls_w, cls_b)]
    h = torch.nn.functional.gelu(torch.nn.functional.linear(xr, ps[0], ps[1]))
    logits = torch.nn.functional.linear(h, ps[2], ps[3]).squeeze(-1)
    ref = rtd_loss(logits, labels, active)
    (ref.loss * 3.0).backward()
    assert abs(float(loss) - float(ref.loss)) < 2e-2 * float(ref.loss)
    assert abs(float(acc) - float(ref.accuracy)) < 0.02
    assert float(count) == float(ref.token_count) and float(pos) == float(ref.positive_count)
    want = [xr.grad] + [p.grad for p in ps]
    for g, w in zip(got, want):
        assert (g - w).abs().max() <= 6e-2 * w.abs().max() + 1e-5, (float((g - w).abs().max()), float(w.abs().max()))


@pytest.mark.parametrize("M,H,frac", [(4096, 768, 0.15), (1000, 64, 0.5), (512, 256, 0.0)])
def test_masked_row_gather_matches_index_select(M, H, frac):
    """Forward equals ``index_select`` bit for bit; the gradient equals the zero-filled ``index_add`` of the reference
    and covers every row (the unselected ones are exact zeros), also for a strided source and an empty selection."""
    from deberta_b200.ops.gather import gather_rows

    torch.manual_seed(4)
    base = (torch.randn(M, H + 8, device="cuda")).to(torch.bfloat16)
    x = base[:, :H].detach().requires_grad_(True)  # row stride H + 8
    idx = torch.nonzero(torch.rand(M, device="cuda") < frac).flatten()
    out = gather_rows(x, idx)
    assert torch.equal(out, x.detach().index_select(0, idx))
    dout = torch.randn(idx.numel(), H, device="cuda").to(torch.bfloat16)
    out.backward(dout)
    _lib.check_status()
    ref = torch.zeros(M, H, device="cuda", dtype=torch.bfloat16).index_add_(0, idx, dout)
    assert torch.equal(x.grad, ref)
