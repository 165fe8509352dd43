"""Operator micro-benchmarks: ``python -m deberta_b200.ops.microbench <op> [--batch B] [--seq S] [--iters N]``.

Times one operator with CUDA events after warm-up (inputs of the DeBERTa-v3-base shapes are far
larger than the 126 MB L2) and prints achieved throughput. Used for the kernel profiles:
the same command line runs under ``ncu`` to capture a single kernel.
"""

from __future__ import annotations

import argparse

import torch


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters * 1e3  # microseconds


def _rand(*shape, scale=0.3, grad=False):
    t = (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)
    return t.requires_grad_(True) if grad else t


def bench_gemm(a) -> None:
    from deberta_b200.ops.gemm import gemm

    M = a.batch * a.seq
    for N, K in ((768, 768), (3072, 768), (768, 3072)):
        x, w = _rand(M, K), _rand(N, K, scale=0.05)
        us = _time(lambda: gemm(x, w), a.iters)
        ref = _time(lambda: x @ w.t(), a.iters)
        print(f"gemm {M}x{N}x{K}: tcgen05 {us:.1f} us ({2 * M * N * K / us / 1e6:.0f} TFLOP/s) | cuBLAS {ref:.1f} us")
        # the two gradients of the same layer: dX = dY·W (bf16) and dW += dYᵀ·X with the bias gradient from the same launch
        dy = _rand(M, N)
        us = _time(lambda: gemm(dy, w, b_mn=True), a.iters)
        ref = _time(lambda: dy @ w, a.iters)
        print(f"  dgrad {M}x{K}x{N}: tcgen05 {us:.1f} us ({2 * M * N * K / us / 1e6:.0f} TFLOP/s) | cuBLAS {ref:.1f} us")
        dw, db = torch.zeros(N, K, device="cuda"), torch.zeros(N, device="cuda")
        us = _time(lambda: gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True, a_sum=db), a.iters)
        plain = _time(lambda: gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True), a.iters)
        dw16 = torch.zeros(N, K, device="cuda", dtype=torch.bfloat16)
        ref = _time(lambda: (torch.addmm(dw16, dy.t(), x, out=dw16), dy.sum(0)), a.iters)
        print(f"  wgrad {N}x{K}x{M}: tcgen05 with bias sum {us:.1f} us ({2 * M * N * K / us / 1e6:.0f} TFLOP/s), without "
              f"{plain:.1f} us | cuBLAS bf16 addmm + column sum {ref:.1f} us")


def bench_ffn(a) -> None:
    """The four GELU-epilogue forms of the FFN GEMMs (M = batch*seq, 768 -> 3072 -> 768)."""
    from deberta_b200.ops.gemm import EPI_DGELU, EPI_GELU, EPI_GELU_GRAD, EPI_MUL, gemm

    M, H, I = a.batch * a.seq, 768, 3072
    x, w1, b1 = _rand(M, H), _rand(I, H, scale=0.03), _rand(I)
    dy, w2 = _rand(M, H), _rand(H, I, scale=0.03)
    z, _ = gemm(x, w1, bias=b1, epi=EPI_GELU)
    g, _ = gemm(x, w1, bias=b1, epi=EPI_GELU_GRAD)
    for name, fn in (("forward, outputs z and gelu(z)", lambda: gemm(x, w1, bias=b1, epi=EPI_GELU)),
                     ("forward, outputs gelu'(z) and gelu(z)", lambda: gemm(x, w1, bias=b1, epi=EPI_GELU_GRAD)),
                     ("backward, dy.W2 * gelu'(z) computed from z", lambda: gemm(dy, w2, b_mn=True, epi=EPI_DGELU, aux=z)),
                     ("backward, dy.W2 * stored gelu'(z)", lambda: gemm(dy, w2, b_mn=True, epi=EPI_MUL, aux=g)),
                     ("backward, dy.W2 alone", lambda: gemm(dy, w2, b_mn=True))):
        print(f"ffn {M}x{I}x{H} {name}: {_time(fn, a.iters):.1f} us")


def bench_attention(a) -> None:
    from deberta_b200.ops.attention import disentangled_attention

    h, span = a.heads, 256
    H = h * 64
    q, k, v = (_rand(a.batch, a.seq, H, grad=True) for _ in range(3))
    pk, pq = (_rand(2 * span, H, grad=True) for _ in range(2))
    from deberta_b200.ops.attention_cuda import set_forward_key_tile

    kw = dict(heads=h, scale_factor=3, bucket_size=256, max_position=512, att_span=span)
    for tile in ((64, 65, 128) if a.key_tile == 0 else (a.key_tile,)):
        set_forward_key_tile(tile)
        for name, pkk, pqq in (("content only", None, None), ("disentangled", pk, pq)):
            f = lambda: disentangled_attention(q, k, v, pkk, pqq, **kw)  # noqa: E731
            g = torch.randn_like(f())
            with torch.no_grad():
                fwd = _time(f, a.iters)
            both = _time(lambda: f().backward(g), a.iters)
            flops = 4 * a.batch * h * a.seq * a.seq * 64
            print(f"attention [{name}, {tile} keys per tile] B={a.batch} S={a.seq} h={h}: fwd {fwd:.0f} us "
                  f"({flops / fwd / 1e6:.0f} TFLOP/s), fwd+bwd {both:.0f} us")
    set_forward_key_tile(64)


def bench_posbias(a) -> None:
    """Position-bias kernels in isolation: tensor-core tile kernels against the score-table path."""
    import ctypes

    from deberta_b200.ops import _lib, attention_cuda as ac

    h, span = a.heads, 256
    H = h * 64
    q, k = _rand(a.batch, a.seq, H), _rand(a.batch, a.seq, H)
    pk, pq = _rand(2 * span, H), _rand(2 * span, H)
    luts = ac._luts(a.seq, 256, 512, span, q.device)
    for name, tc in (("tensor cores", True), ("score tables + gather", False)):
        us = _time(lambda: ac.position_bias(q, k, pk, pq, luts, h, tensor_core=tc), a.iters)
        print(f"position bias fwd [{name}] B={a.batch} S={a.seq} h={h}: {us:.0f} us")
    bias, _ = ac.position_bias(q, k, pk, pq, luts, h, tensor_core=True)
    dbias = _rand(*bias.shape, scale=0.1)
    T = a.batch * a.seq
    dq_acc = torch.zeros(T, H, dtype=torch.float32, device="cuda")
    dk = torch.zeros(T, 3 * H, dtype=torch.bfloat16, device="cuda")[:, H:2 * H]
    gk, gq = (torch.zeros(2 * span, H, dtype=torch.float32, device="cuda") for _ in range(2))
    pa = ac._posbias_args(q, k, pk, pq, luts, h, 2 * span)
    pa.dbias, pa.ldb = dbias.data_ptr(), bias.shape[-1]
    pa.dq_acc, pa.dk, pa.ld_dk = dq_acc.data_ptr(), dk.data_ptr(), 3 * H
    pa.d_pos_k, pa.d_pos_q = gk.data_ptr(), gq.data_ptr()
    us = _time(lambda: _lib.call("db200_posbias_tc_bwd", ctypes.byref(pa), _lib.stream_ptr()), a.iters)
    print(f"position bias bwd [tensor cores] B={a.batch} S={a.seq} h={h}: {us:.0f} us")
    _lib.check_status()


def bench_vocab_ce(a) -> None:
    from deberta_b200.ops.heads import mlm_loss_and_sample, mlm_loss_and_sample_reference

    N, V, E = a.batch * 77, 128100, 768
    x, w, b = _rand(N, E, grad=True), _rand(V, E, scale=0.02, grad=True), _rand(V, scale=0.01, grad=True)
    labels = torch.randint(5, V, (N,), device="cuda")
    forb = torch.zeros(V, dtype=torch.bool, device="cuda")
    for name, fn in (("fused", mlm_loss_and_sample), ("aten", mlm_loss_and_sample_reference)):
        f = lambda: fn(x, w, b, labels, forb, 1.0)  # noqa: E731
        fwd = _time(f, a.iters)
        both = _time(lambda: f()[0].backward(), a.iters)
        print(f"vocab CE+sample [{name}] N={N} V={V}: fwd {fwd:.0f} us, fwd+bwd {both:.0f} us")


def bench_layer(a) -> None:
    from deberta_b200.models.deberta_v2 import DebertaV2Layer
    from deberta_b200.models.builder import build_repo_hf_deberta_v2_config

    cfg = build_repo_hf_deberta_v2_config("base")
    cfg.hidden_dropout_prob = cfg.attention_probs_dropout_prob = 0.0
    layer = DebertaV2Layer(cfg).cuda().to(torch.bfloat16)
    x = _rand(a.batch, a.seq, 768, scale=1.0, grad=True)
    rel = _rand(512, 768, scale=1.0)
    f = lambda: layer(x, None, rel_embeddings=rel)[0]  # noqa: E731
    g = torch.randn_like(f())
    fwd = _time(f, a.iters)
    both = _time(lambda: f().backward(g), a.iters)
    print(f"DeBERTa-v3-base layer B={a.batch} S={a.seq}: fwd {fwd:.0f} us, fwd+bwd {both:.0f} us")


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("op", choices=("gemm", "ffn", "attention", "posbias", "vocab_ce", "layer"))
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--seq", type=int, default=512)
    p.add_argument("--heads", type=int, default=12)
    p.add_argument("--iters", type=int, default=5)
    p.add_argument("--key-tile", type=int, default=0, help="attention forward: 64 (warp-specialised), 65 (64 keys, block barriers) or 128 keys per tile (0: all)")
    a = p.parse_args()
    {"gemm": bench_gemm, "ffn": bench_ffn, "attention": bench_attention, "posbias": bench_posbias, "vocab_ce": bench_vocab_ce, "layer": bench_layer}[a.op](a)


if __name__ == "__main__":
    main()
