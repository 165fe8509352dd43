"""tcgen05 GEMM kernel vs. the fp32 PyTorch statement of the same contract."""

from __future__ import annotations

import pytest
import torch

from deberta_b200.ops import _lib
from deberta_b200.ops.gemm import EPI_DGELU, EPI_GELU, EPI_GELU_GRAD, EPI_MUL, gemm, gemm_reference

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, ref, tol=2e-2):
    got = got.float()
    ref = ref.float()
    err = (got - ref).abs().max().item()
    denom = ref.abs().max().item() + 1e-6
    assert err / denom < tol, f"rel err {err / denom:.4g} (abs {err:.4g})"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (304, 264, 136), (1024, 768, 768), (640, 96, 2048)])
def test_gemm_majors(a_mn, b_mn, M, N, K):
    torch.manual_seed(0)
    a = _rand(K, M) if a_mn else _rand(M, K)
    b = _rand(K, N) if b_mn else _rand(N, K)
    out = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    _lib.check_status()
    ref = gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    _close(out, ref)


def test_gemm_bias_residual_gelu():
    torch.manual_seed(1)
    M, N, K = 520, 3072, 768
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    out = gemm(a, w, bias=bias, residual=res)
    _close(out, gemm_reference(a, w, bias=bias, residual=res, out_dtype=torch.float32))
    z, act = gemm(a, w, bias=bias, epi=EPI_GELU)
    zr, ar = gemm_reference(a, w, bias=bias, epi=EPI_GELU)
    _close(z, zr)
    _close(act, ar)
    dz = gemm(a, w, epi=EPI_DGELU, aux=z)
    _close(dz, gemm_reference(a, w, epi=EPI_DGELU, aux=z, out_dtype=torch.float32))
    _lib.check_status()


@pytest.mark.parametrize("M,N", [(520, 3072), (300, 200)])  # TMA-store path and the ragged scalar path
def test_gemm_gelu_with_stored_derivative(M, N):
    """EPI_GELU_GRAD writes (gelu'(z), gelu(z)); EPI_MUL with that factor equals the EPI_DGELU backward."""
    torch.manual_seed(4)
    K = 768
    a, w, bias = _rand(M, K), _rand(N, K, scale=0.05), _rand(N)
    g, act = gemm(a, w, bias=bias, epi=EPI_GELU_GRAD)
    gr, ar = gemm_reference(a, w, bias=bias, epi=EPI_GELU_GRAD)
    _close(g, gr)
    _close(act, ar)
    z, act_z = gemm(a, w, bias=bias, epi=EPI_GELU)
    assert torch.equal(act, act_z)  # the activation is the same in both forms
    dy, w2 = _rand(M, 256), _rand(256, N, scale=0.05)
    via_mul = gemm(dy, w2, b_mn=True, epi=EPI_MUL, aux=g)
    via_dgelu = gemm(dy, w2, b_mn=True, epi=EPI_DGELU, aux=z)
    _close(via_mul, gemm_reference(dy, w2, b_mn=True, epi=EPI_MUL, aux=g, out_dtype=torch.float32))
    _close(via_mul, via_dgelu.float(), tol=1e-2)  # the stored factor is rounded to bf16 once more
    _lib.check_status()


def test_ffn_gelu_block_matches_pytorch():
    from deberta_b200.ops.linear import ffn_gelu

    torch.manual_seed(5)
    T, H, I = 384, 768, 3072
    x = _rand(T, H).requires_grad_(True)
    w1, b1 = _rand(I, H, scale=0.03).requires_grad_(True), _rand(I, scale=0.1).requires_grad_(True)
    w2, b2 = _rand(H, I, scale=0.03).requires_grad_(True), _rand(H, scale=0.1).requires_grad_(True)
    res = _rand(T, H)
    y = ffn_gelu(x, w1, b1, w2, b2, residual=res)
    ref_in = [t.detach().float().requires_grad_(True) for t in (x, w1, b1, w2, b2)]
    xr, w1r, b1r, w2r, b2r = ref_in
    yr = torch.nn.functional.gelu(xr @ w1r.t() + b1r) @ w2r.t() + b2r + res.float()
    _close(y, yr)
    dy = torch.randn_like(yr)
    (y.float() * dy).sum().backward()
    (yr * dy).sum().backward()
    for name, a, b in zip("x w1 b1 w2 b2".split(), (x, w1, b1, w2, b2), ref_in):
        _close(a.grad, b.grad, tol=3e-2)
    _lib.check_status()


def test_gemm_fp32_accumulate_split_k():
    torch.manual_seed(2)
    T, O, I = 4096, 768, 768
    dy, x = _rand(T, O, scale=0.1), _rand(T, I)
    grad = torch.ones(O, I, device="cuda", dtype=torch.float32)
    gemm(dy, x, a_mn=True, b_mn=True, out=grad, accumulate=True)
    ref = 1.0 + dy.float().t() @ x.float()
    _close(grad, ref, tol=5e-3)
    fresh = gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
    _close(fresh, ref - 1.0, tol=5e-3)
    _lib.check_status()


@pytest.mark.parametrize("M,N,K", [(768, 768, 16384), (3072, 768, 4096), (768, 3072, 2048), (200, 96, 1000), (2304, 768, 512),
                                   (4000, 520, 192)])
def test_weight_gradient_gemm_also_sums_its_first_operand(M, N, K):
    """dW = dyᵀ·x with ``a_sum``: the bias gradient Σ_tokens dy comes out of the same launch, is added to what the
    buffer held, and matches an fp32 column sum; covers split-K, both tile widths, ragged edges and several work
    items per CTA (the single-buffer accumulator path)."""
    torch.manual_seed(5)
    dy = (torch.randn(K, M, device="cuda") * 0.5 + 0.1).to(torch.bfloat16)
    x = torch.randn(K, N, device="cuda").to(torch.bfloat16)
    w_acc = torch.randn(M, N, device="cuda")
    b_acc = torch.randn(M, device="cuda")
    w0, b0 = w_acc.clone(), b_acc.clone()
    gemm(dy, x, a_mn=True, b_mn=True, out=w_acc, accumulate=True, a_sum=b_acc)
    _lib.check_status()
    ref_w = w0 + dy.float().t() @ x.float()
    ref_b = b0 + dy.float().sum(0)
    assert (w_acc - ref_w).abs().max().item() < 2e-3 * ref_w.abs().max().item() + 1e-3
    assert (b_acc - ref_b).abs().max().item() < 1e-4 * ref_b.abs().max().item() + 1e-3
    # a second call keeps accumulating (no hidden state between launches)
    gemm(dy, x, a_mn=True, b_mn=True, out=w_acc, accumulate=True, a_sum=b_acc)
    assert (b_acc - (ref_b + dy.float().sum(0))).abs().max().item() < 1e-4 * ref_b.abs().max().item() + 2e-3


def test_gemm_batched_strided():
    torch.manual_seed(3)
    B, T, H, d, P = 3, 256, 4, 64, 512
    q = _rand(T, B * H * d).view(T, B, H * d)  # tokens x (batch of heads) with row stride
    qh = q[:, 0, :].view(T, H, d).permute(1, 0, 2)  # [H, T, d], inner stride 1, ld = B*H*d
    pos = _rand(P, H * d).view(P, H, d).permute(1, 0, 2)  # [H, P, d]
    out = gemm(qh, pos)
    ref = torch.einsum("htd,hpd->htp", qh.float(), pos.float())
    _close(out, ref)
    _lib.check_status()


def test_gemm_speed_report():
    """Not a pass/fail perf gate: prints achieved TFLOP/s next to cuBLAS for the log."""
    M, N, K = 16384, 3072, 768
    a, w = _rand(M, K), _rand(N, K, scale=0.05)
    for fn, name in ((lambda: gemm(a, w), "tcgen05"), (lambda: a @ w.t(), "cublas")):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(10):
            fn()
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / 10
        print(f"\n[gemm {M}x{N}x{K}] {name}: {ms * 1e3:.1f} us, {2 * M * N * K / ms / 1e9:.1f} TFLOP/s")
    _lib.check_status()


def test_fused_qkv_projection_matches_three_linears():
    """Weights laid out back to back (as the engine does) take the one-GEMM path; results and gradients must agree."""
    from deberta_b200.ops.linear import _qkv_fusable, linear_qkv

    dev = torch.device("cuda")
    torch.manual_seed(0)
    n, k, t = 128, 64, 300
    flat_w = (torch.randn(3 * n * k, device=dev) * 0.1).to(torch.bfloat16)
    flat_b = (torch.randn(3 * n, device=dev) * 0.1).to(torch.bfloat16)
    gw = torch.zeros(3 * n * k, device=dev)
    gb = torch.zeros(3 * n, device=dev)
    ws, bs = [], []
    for i in range(3):
        w = torch.nn.Parameter(flat_w[i * n * k:(i + 1) * n * k].view(n, k))
        b = torch.nn.Parameter(flat_b[i * n:(i + 1) * n])
        w.main_grad = gw[i * n * k:(i + 1) * n * k].view(n, k)
        b.main_grad = gb[i * n:(i + 1) * n]
        ws.append(w)
        bs.append(b)
    x = (torch.randn(2, t // 2, k, device=dev) * 0.5).to(torch.bfloat16).requires_grad_(True)
    assert _qkv_fusable(x, ws[0], bs[0], ws[1], bs[1], ws[2], bs[2])
    q, kk, v = linear_qkv(x, ws[0], bs[0], ws[1], bs[1], ws[2], bs[2])
    gq, gk, gv = (torch.randn_like(q) for _ in range(3))
    (q * gq + kk * gk + v * gv).sum().backward()
    xr = x.detach().float().requires_grad_(True)
    outs = [torch.nn.functional.linear(xr, w.detach().float(), b.detach().float()) for w, b in zip(ws, bs)]
    sum((o * g.float()).sum() for o, g in zip(outs, (gq, gk, gv))).backward()
    for got, want in zip((q, kk, v), outs):
        assert (got.float() - want).abs().max() <= 2e-2 * want.abs().max()
    assert (x.grad.float() - xr.grad).abs().max() <= 3e-2 * xr.grad.abs().max()
    x2 = x.detach().float().reshape(-1, k)
    for i, g in enumerate((gq, gk, gv)):
        want_w = g.float().reshape(-1, n).t() @ x2
        assert (ws[i].main_grad - want_w).abs().max() <= 3e-2 * want_w.abs().max()
        want_b = g.float().reshape(-1, n).sum(0)
        assert (bs[i].main_grad - want_b).abs().max() <= 3e-2 * want_b.abs().max()


def test_linear_backward_reads_a_column_slice_in_place():
    """The upstream gradient of a projection can be a column slice of a wider buffer (the attention backward writes
    dQ | dK | dV side by side): data, weight and bias gradients must equal those of a contiguous copy, also into
    ``main_grad`` buffers."""
    from deberta_b200.ops.linear import linear

    torch.manual_seed(5)
    T, K, N = 1000, 256, 384
    x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
    wide = (torch.randn(T, 3 * N, device="cuda") * 0.5).to(torch.bfloat16)
    results = []
    for contiguous in (True, False):
        xx = x.clone().requires_grad_(True)
        w = torch.nn.Parameter((torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16))
        b = torch.nn.Parameter(torch.zeros(N, device="cuda", dtype=torch.bfloat16))
        torch.manual_seed(6)
        w.data.copy_((torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16))
        w.main_grad = torch.zeros(N, K, device="cuda")
        b.main_grad = torch.zeros(N, device="cuda")
        dy = wide[:, N : 2 * N]
        assert not dy.is_contiguous()
        linear(xx, w, b).backward(dy.contiguous() if contiguous else dy)
        results.append((xx.grad.clone(), w.main_grad.clone(), b.main_grad.clone()))
    _lib.check_status()
    assert torch.equal(results[0][0], results[1][0])
    for a_, b_ in zip(results[0][1:], results[1][1:]):  # split-K adds in fp32: equal up to the order of the additions
        assert (a_ - b_).abs().max() <= 1e-4 * a_.abs().max()


def test_residual_gradient_rides_into_the_qkv_data_gradient_gemm():
    """y = W_o·(q + k + v) + x with (q, k, v) from the fused projection of x: with a ResidualGradSink the closing
    projection reports no gradient for its residual and the opening projection's backward adds it in its GEMM epilogue.
    The gradient of x must equal the one autograd builds with its own add, and the fp32 statement."""
    from deberta_b200.ops.linear import ResidualGradSink, linear, linear_qkv

    dev = torch.device("cuda")
    torch.manual_seed(3)
    n, t = 128, 320
    flat_w = (torch.randn(3 * n * n, device=dev) * 0.05).to(torch.bfloat16)
    gw = torch.zeros(3 * n * n, device=dev)
    ws = []
    for i in range(3):
        w = torch.nn.Parameter(flat_w[i * n * n:(i + 1) * n * n].view(n, n))
        w.main_grad = gw[i * n * n:(i + 1) * n * n].view(n, n)
        ws.append(w)
    wo = (torch.randn(n, n, device=dev) * 0.05).to(torch.bfloat16)
    x0 = (torch.randn(2, t // 2, n, device=dev) * 0.5).to(torch.bfloat16)
    gy = torch.randn(2, t // 2, n, device=dev).to(torch.bfloat16)

    def run(with_sink):
        x = x0.clone().requires_grad_(True)
        sink = ResidualGradSink() if with_sink else None
        q, k, v = linear_qkv(x, ws[0], None, ws[1], None, ws[2], None, residual_sink=sink)
        assert (sink is None) or sink.armed
        y = linear(q + k + v, wo, None, residual=x, residual_sink=sink)
        y.backward(gy)
        assert sink is None or sink.grad is None  # collected
        return y.detach(), x.grad.detach()

    y_a, g_a = run(False)
    y_b, g_b = run(True)
    assert torch.equal(y_a, y_b)
    xr = x0.float().requires_grad_(True)
    h = sum(torch.nn.functional.linear(xr, w.detach().float()) for w in ws)
    yr = torch.nn.functional.linear(h, wo.float()) + xr
    yr.backward(gy.float())
    for g in (g_a, g_b):
        assert (g.float() - xr.grad).abs().max() <= 3e-2 * xr.grad.abs().max()
    # fused: one rounding of (dx + residual gradient); unfused: each rounded, then added and rounded again
    assert (g_a.float() - g_b.float()).abs().max() <= 2e-2 * xr.grad.abs().max()
    _lib.check_status()


@pytest.mark.parametrize("T,H,F,bias", [(1024, 768, 2048, False), (300, 256, 200, True), (640, 768, 3072, True)])
def test_swiglu_ffn_in_gemm_epilogues_matches_pytorch(T, H, F, bias):
    """SwiGLU forward inside the W12 GEMM (writes [gate | up] and silu(gate)·up) and its backward inside the W3
    data-gradient GEMM, against the fp32 statement; ragged F exercises the scalar tails."""
    from deberta_b200.ops.linear import ffn_swiglu

    torch.manual_seed(11)
    x = _rand(T, H, scale=0.5).requires_grad_(True)
    w12, w3 = _rand(2 * F, H, scale=0.05).requires_grad_(True), _rand(H, F, scale=0.05).requires_grad_(True)
    b12 = _rand(2 * F, scale=0.1).requires_grad_(True) if bias else None
    b3 = _rand(H, scale=0.1).requires_grad_(True) if bias else None
    y = ffn_swiglu(x, w12, b12, w3, b3)
    ref_in = [t.detach().float().requires_grad_(True) if t is not None else None for t in (x, w12, b12, w3, b3)]
    xr, w12r, b12r, w3r, b3r = ref_in
    gu = torch.nn.functional.linear(xr, w12r, b12r)
    yr = torch.nn.functional.linear(torch.nn.functional.silu(gu[:, :F]) * gu[:, F:], w3r, b3r)
    _close(y, yr, tol=3e-2)
    g = torch.randn_like(yr)
    y.backward(g.to(torch.bfloat16))
    yr.backward(g)
    _lib.check_status()
    for got, ref in ((x, xr), (w12, w12r), (w3, w3r)) + (((b12, b12r), (b3, b3r)) if bias else ()):
        _close(got.grad, ref.grad, tol=4e-2)
