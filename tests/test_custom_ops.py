"""The ``db200`` custom ops on CPU: ``torch.library.opcheck`` (schema, fake kernels, autograd registration, AOT
dispatch) for every forward/backward pair, and a compiled tiny model step through the public operator functions."""

from __future__ import annotations

import pytest
import torch
from torch.library import opcheck

from deberta_b200.ops import library as L


def _t(*shape, grad=False, dtype=torch.float32):
    return torch.randn(*shape, dtype=dtype).requires_grad_(grad)


def _cases():
    x, w, b = _t(6, 8, grad=True), _t(16, 8, grad=True), _t(16, grad=True)
    wg, bg = torch.zeros(16, 8), torch.zeros(16)
    yield "linear", L.linear, (x, w, b, _t(6, 16), None, None)
    yield "linear-main-grad", L.linear, (x, w, b, None, wg, bg)
    yield "linear_bwd", L.linear_bwd, (_t(6, 16), x.detach(), w.detach(), wg, None, True, True)
    w2, b2 = _t(8, 16, grad=True), _t(8, grad=True)
    yield "ffn_gelu", L.ffn_gelu, (x, w, b, w2, b2, _t(6, 8), None, None, None, None)
    g, a = _t(6, 16), _t(6, 16)
    yield "ffn_gelu_bwd", L.ffn_gelu_bwd, (_t(6, 8), x.detach(), w.detach(), w2.detach(), g, a, wg, None, None,
                                            torch.zeros(8), True, True, True)
    gamma, beta = _t(8, grad=True), _t(8, grad=True)
    keep = torch.tensor([1, 1, 0, 1, 1, 1], dtype=torch.uint8)
    yield "layer_norm", L.norm, (x, gamma, beta, keep, 1e-6, False, None, None)
    yield "rms_norm", L.norm, (x, gamma, None, None, 1e-6, True, None, None)
    y, mean, rstd = L.norm(x.detach(), gamma.detach(), beta.detach(), None, 1e-6, False, None, None)
    yield "norm_bwd", L.norm_bwd, (_t(6, 8), x.detach(), gamma.detach(), mean, rstd, None, False, True, torch.zeros(8), None)
    table = _t(11, 8)
    ids = torch.randint(0, 11, (2, 3))
    yield "embed", L.embed, (ids, table, _t(11, 8), 0, torch.zeros(11, 8), None)
    yield "embed_bwd", L.embed_bwd, (_t(2, 3, 8), ids, 11, 0, torch.zeros(11, 8), torch.zeros(11, 8))
    ang = torch.repeat_interleave(torch.outer(torch.arange(5.0), 1.0 / 10 ** torch.arange(0, 4.0, 2) ), 2, dim=-1)
    yield "rotary", L.rotary, (_t(2, 5, 16, grad=True), ang.cos(), ang.sin(), 2, 4, False)
    gu = _t(6, 16, grad=True)
    yield "swiglu", L.swiglu, (gu,)
    yield "swiglu_bwd", L.swiglu_bwd, (gu.detach(), _t(6, 8))
    q, k, v = (_t(2, 12, 128, grad=True) for _ in range(3))
    pk, pq = _t(16, 128, grad=True), _t(16, 128, grad=True)
    keep2 = torch.ones(2, 12, dtype=torch.bool)
    keep2[1, 9:] = False
    yield "flash_attn-disentangled", L.flash_attn, (q, k, v, pk, pq, keep2, None, 2, 13.86, 8, 16, 8)
    yield "flash_attn-content", L.flash_attn, (q, k, v, None, None, None, None, 2, 8.0, 0, 0, 0)


CASES = list(_cases())


@pytest.mark.parametrize("name,op,args", CASES, ids=[c[0] for c in CASES])
def test_opcheck(name, op, args):
    opcheck(op, args)


def test_linear_op_matches_eager_and_fills_main_grad():
    x, w, b = _t(5, 8, grad=True), _t(4, 8, grad=True), _t(4, grad=True)
    wg, bg = torch.zeros(4, 8), torch.zeros(4)
    y = L.linear(x, w, b, None, wg, bg)
    ref = torch.nn.functional.linear(x, w, b)
    torch.testing.assert_close(y, ref)
    gy = torch.randn_like(y)
    y.backward(gy)
    gx, gw, gb = torch.autograd.grad(ref, (x, w, b), gy)
    torch.testing.assert_close(x.grad, gx)
    torch.testing.assert_close(wg, gw)
    torch.testing.assert_close(bg, gb)
    assert w.grad is None and b.grad is None  # the buffers took the parameter gradients


def test_norm_ops_match_functional():
    x, g, b = _t(7, 16, grad=True), _t(16, grad=True), _t(16, grad=True)
    y = L.norm(x, g, b, None, 1e-5, False, None, None)[0]
    ref = torch.nn.functional.layer_norm(x, (16,), g, b, 1e-5)
    torch.testing.assert_close(y, ref)
    gy = torch.randn_like(y)
    got = torch.autograd.grad(y, (x, g, b), gy)
    want = torch.autograd.grad(ref, (x, g, b), gy)
    for a_, b_ in zip(got, want):
        torch.testing.assert_close(a_, b_, rtol=1e-4, atol=1e-5)
    y2 = L.norm(x, g, None, None, 1e-6, True, None, None)[0]
    ref2 = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * g
    torch.testing.assert_close(y2, ref2)
    for a_, b_ in zip(torch.autograd.grad(y2, (x, g), gy), torch.autograd.grad(ref2, (x, g), gy)):
        torch.testing.assert_close(a_, b_, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("backend", ["aot_eager"])
def test_ops_trace_as_single_nodes_without_graph_breaks(backend):
    """What ``train.compile`` relies on: the ops pass through Dynamo + AOTAutograd with ``fullgraph=True``, and the
    parameter gradients still reach the ``main_grad`` buffers."""

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(8, 8)
            self.ln_w = torch.nn.Parameter(torch.ones(8))
            self.ln_b = torch.nn.Parameter(torch.zeros(8))
            for p in self.parameters():
                p.main_grad = torch.zeros_like(p)

        def forward(self, x):
            mg = lambda p: p.main_grad  # noqa: E731
            h = L.linear(x, self.fc.weight, self.fc.bias, x, mg(self.fc.weight), mg(self.fc.bias))
            return L.norm(h, self.ln_w, self.ln_b, None, 1e-6, False, mg(self.ln_w), mg(self.ln_b))[0].square().sum()

    torch.manual_seed(0)
    m = Block()
    x = torch.randn(4, 8, requires_grad=True)
    m(x).backward()
    want = {n: p.main_grad.clone() for n, p in m.named_parameters()}
    gx = x.grad.clone()
    for p in m.parameters():
        p.main_grad.zero_()
    x.grad = None
    torch._dynamo.reset()
    torch.compile(m, backend=backend, fullgraph=True)(x).backward()
    torch.testing.assert_close(x.grad, gx)
    for n, p in m.named_parameters():
        torch.testing.assert_close(p.main_grad, want[n])
        assert p.grad is None


def test_compile_scopes_resolve_and_replace_forwards():
    from deberta_b200 import config as C
    from deberta_b200.data.synthetic import SyntheticTokenizer
    from deberta_b200.training.compile import compile_model_for_scope, maybe_compile_model, resolve_compile_scope
    from deberta_b200.training.runtime import build_model

    assert resolve_compile_scope(requested_scope="auto", backbone_type="hf_deberta_v2") == ("backbones", None)
    scope, why = resolve_compile_scope(requested_scope="auto", backbone_type="rope", block_cross_document_attention=True)
    assert scope == "ffn" and "doc-blocking" in why
    assert resolve_compile_scope(requested_scope="gen_ffn", backbone_type="rope")[0] == "gen_ffn"
    mc = C.ModelConfig(backbone_type="rope", hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                       intermediate_size=64, tokenizer_name_or_path="synthetic:200")
    model, _, _ = build_model(model_cfg=mc, tokenizer=SyntheticTokenizer(200), max_seq_length=32)
    names = compile_model_for_scope(model, "ffn", backend="aot_eager")
    assert names and all(".mlp" in n for n in names) and any(n.startswith("generator") for n in names)
    assert compile_model_for_scope(model, "encoder", backend="aot_eager") == ["generator.encoder", "discriminator.encoder"]
    with pytest.raises(ValueError):
        compile_model_for_scope(model, "nonsense", backend="aot_eager")
    tc = C.TrainConfig(mixed_precision="no")
    assert maybe_compile_model(model, train_cfg=tc, model_cfg=mc) == (None, None, [])


def test_compiled_backbones_train_step_matches_eager_on_cpu():
    """One decoupled window with ``train.compile`` (aot_eager, scope backbones) against the same window in eager mode."""
    from deberta_b200 import config as C
    from deberta_b200.data.synthetic import SyntheticTokenizer
    from deberta_b200.parallel.dist import DistContext
    from deberta_b200.training.compile import maybe_compile_model
    from deberta_b200.training.runtime import build_engine, build_model
    from deberta_b200.training.trainer import Trainer

    def run(compiled: bool):
        torch.manual_seed(0)
        torch._dynamo.reset()
        mc = C.ModelConfig(backbone_type="rope", hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                           intermediate_size=64, tokenizer_name_or_path="synthetic:200")
        tc = C.TrainConfig(max_steps=4, per_device_train_batch_size=2, gradient_accumulation_steps=1, mixed_precision="no",
                           torch_compile=compiled, torch_compile_backend="aot_eager", torch_compile_scope="backbones")
        oc = C.OptimConfig(learning_rate=1e-3, warmup_steps=0, lr_scheduler_type="constant")
        model, _, _ = build_model(model_cfg=mc, tokenizer=SyntheticTokenizer(200), max_seq_length=32)
        ctx = DistContext()
        engine = build_engine(model=model, ctx=ctx, train_cfg=tc, optim_cfg=oc, parallelism="ddp")
        trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=tc, optim_cfg=oc, pad_token_id=0)
        scope, _, targets = maybe_compile_model(model, train_cfg=tc, model_cfg=mc)
        assert (scope == "backbones" and targets == ["generator", "discriminator"]) if compiled else scope is None
        g = torch.Generator().manual_seed(1)
        ids = torch.randint(5, 200, (2, 16), generator=g)
        labels = torch.full_like(ids, -100)
        labels[:, 3] = ids[:, 3]
        labels[:, 9] = ids[:, 9]
        ids = ids.clone()
        ids[:, 3] = 4
        ids[:, 9] = 4
        stats = trainer.train_window([{"input_ids": ids, "labels": labels}])
        return float(stats.gen_loss_tokens), engine.master.clone()

    loss_e, w_e = run(False)
    loss_c, w_c = run(True)
    assert abs(loss_e - loss_c) < 1e-4 * max(1.0, abs(loss_e))
    torch.testing.assert_close(w_c, w_e, rtol=1e-4, atol=1e-6)


def test_gemm_reference_swiglu_epilogues_are_consistent_with_autograd():
    """The fp32 statements of the two SwiGLU epilogues (the oracle of the GPU test): forward halves and product, and a
    backward that equals autograd's through ``silu(gate) * up``."""
    from deberta_b200.ops.gemm import EPI_SWIGLU, EPI_SWIGLU_BWD, gemm_reference

    torch.manual_seed(2)
    x, w12, b12 = _t(5, 8), _t(12, 8), _t(12)
    gu, h = gemm_reference(x, w12, bias=b12, epi=EPI_SWIGLU)
    ref_gu = torch.nn.functional.linear(x, w12, b12)
    torch.testing.assert_close(gu, ref_gu)
    torch.testing.assert_close(h, torch.nn.functional.silu(ref_gu[:, :6]) * ref_gu[:, 6:])
    dy, w3 = _t(5, 4), _t(4, 6)
    dgu = gemm_reference(dy, w3, b_mn=True, epi=EPI_SWIGLU_BWD, aux=gu)
    gu_ad = ref_gu.clone().requires_grad_(True)
    (torch.nn.functional.silu(gu_ad[:, :6]) * gu_ad[:, 6:] @ w3.t() * dy).sum().backward()
    torch.testing.assert_close(dgu, gu_ad.grad, rtol=1e-4, atol=1e-5)
