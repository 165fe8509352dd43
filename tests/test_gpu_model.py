"""Kernels against PyTorch above the single-operator level: norms, AdamW, one DeBERTa-v3 layer, one whole RTD step,
the fused sampler's distribution, and a compiled training step."""

from __future__ import annotations

import ctypes
import math

import pytest
import torch
import torch.nn.functional as F

from deberta_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-9)


@pytest.mark.parametrize("rows,H", [(1000, 768), (333, 200), (64, 1024), (5, 8)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_kernels_match_pytorch_values_and_gradients(rows, H, rms):
    from deberta_b200.ops.norm import layer_norm, rms_norm

    torch.manual_seed(0)
    x = (torch.randn(rows, H, device="cuda") * 2 + 0.5).to(torch.bfloat16).requires_grad_(True)
    g = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    keep = torch.rand(rows, device="cuda") > 0.1
    xr, gr, br = (t.detach().float().requires_grad_(True) for t in (x, g, b))
    if rms:
        y = rms_norm(x, g, 1e-6, keep)
        ref = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * gr * keep[:, None]
    else:
        y = layer_norm(x, g, b, 1e-7, keep)
        ref = F.layer_norm(xr, (H,), gr, br, 1e-7) * keep[:, None]
    _lib.check_status()
    assert _rel(y, ref) < 1e-2
    w = torch.randn_like(ref)
    (y.float() * w).sum().backward()
    (ref * w).sum().backward()
    _lib.check_status()
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(g.grad, gr.grad) < 2e-2
    if not rms:
        assert _rel(b.grad, br.grad) < 2e-2


def test_adamw_and_sumsq_kernels_match_torch_adamw_with_clipping_and_skip():
    torch.manual_seed(0)
    n, lr, wd, b1, b2, eps, max_norm = 10_000 + 4, 1e-2, 0.1, 0.9, 0.98, 1e-6, 0.5
    p = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=lr, betas=(b1, b2), eps=eps, weight_decay=wd, fused=False, foreach=False)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    shadow = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    norm_sq = torch.zeros(1, device="cuda")
    cf, cl = ctypes.c_float, ctypes.c_longlong
    step = 0
    for it in range(6):
        g = torch.randn(n, device="cuda") * (3.0 if it % 2 else 0.3)
        if it == 3:
            g[17] = float("inf")  # this step must leave parameters and moments untouched
        norm_sq.zero_()
        _lib.call("db200_sumsq", _lib.ptr(g), cl(n), _lib.ptr(norm_sq), _lib.stream_ptr())
        if it != 3:
            assert abs(float(norm_sq) - float(g.double().pow(2).sum())) < 1e-4 * float(g.double().pow(2).sum())
            step += 1
        before = (p.clone(), m.clone(), v.clone())
        t = step if it != 3 else step + 1
        _lib.call("db200_adamw", _lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), _lib.ptr(shadow), cl(n), cf(lr), cf(wd),
                  cf(b1), cf(b2), cf(eps), cf(1 / (1 - b1 ** t)), cf(1 / math.sqrt(1 - b2 ** t)), _lib.ptr(norm_sq),
                  cf(max_norm), cf(1.0), None, _lib.stream_ptr())
        if it == 3:
            assert all(torch.equal(a, b) for a, b in zip(before, (p, m, v)))
            continue
        ref_p.grad = g.clone()
        torch.nn.utils.clip_grad_norm_([ref_p], max_norm)
        opt.step()
        assert (p - ref_p.data).abs().max() < 2e-6
        assert torch.equal(shadow, p.to(torch.bfloat16))
    gate = torch.zeros(1, device="cuda")  # a device-side gate of 0 switches the update off
    before = p.clone()
    _lib.call("db200_adamw", _lib.ptr(p), _lib.ptr(g), _lib.ptr(m), _lib.ptr(v), _lib.ptr(shadow), cl(n), cf(lr), cf(wd),
              cf(b1), cf(b2), cf(eps), cf(1.0), cf(1.0), None, cf(0.0), cf(1.0), _lib.ptr(gate), _lib.stream_ptr())
    assert torch.equal(p, before)
    _lib.check_status()


def _layer_pair(seed=0):
    from deberta_b200.models.builder import build_repo_hf_deberta_v2_config
    from deberta_b200.models.deberta_v2 import DebertaV2Layer

    cfg = build_repo_hf_deberta_v2_config("base")
    cfg.hidden_dropout_prob = cfg.attention_probs_dropout_prob = 0.0
    torch.manual_seed(seed)
    ref = DebertaV2Layer(cfg).cuda().float()
    for p in ref.parameters():  # bf16-representable weights: both arms then start from identical numbers
        p.data = p.data.to(torch.bfloat16).float() if p.dim() < 2 else (p.data * 2).to(torch.bfloat16).float()
    fast = DebertaV2Layer(cfg).cuda().to(torch.bfloat16)
    fast.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()})
    return cfg, ref, fast


def test_one_deberta_v3_base_layer_kernels_match_fp32_modules():
    _, ref, fast = _layer_pair()
    B, S = 2, 384
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(B, S, 768, device="cuda", generator=g).to(torch.bfloat16)
    rel = (torch.randn(512, 768, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    keep = torch.ones(B, S, dtype=torch.bool, device="cuda")
    keep[1, 300:] = False
    xf, xr = x.clone().requires_grad_(True), x.float().requires_grad_(True)
    relf, relr = rel.clone().requires_grad_(True), rel.float().requires_grad_(True)
    y = fast(xf, keep, rel_embeddings=relf)[0]
    yr = ref(xr, keep, rel_embeddings=relr)[0]
    _lib.check_status()
    live = keep[:, :, None]
    assert _rel(y * live, yr * live) < 3e-2
    w = torch.randn_like(yr) * live
    (y.float() * w).sum().backward()
    (yr * w).sum().backward()
    _lib.check_status()
    assert _rel(xf.grad, xr.grad) < 5e-2 and _rel(relf.grad, relr.grad) < 8e-2
    grads = dict(ref.named_parameters())
    for name, p in fast.named_parameters():
        assert p.grad is not None and _rel(p.grad, grads[name].grad) < 8e-2, name


def _tiny_step(precision: str, compile_backend: str | None = None, synchronous: bool = True, overlap: bool = True,
               windows: int = 2, return_engine: bool = False, grad_ckpt: bool = False):
    from deberta_b200.config import Config, DataConfig, ModelConfig, OptimConfig, TrainConfig, validate_config
    from deberta_b200.parallel.dist import DistContext
    from deberta_b200.training.compile import maybe_compile_model
    from deberta_b200.training.runtime import build_engine, build_model, build_tokenizer
    from deberta_b200.training.trainer import Trainer

    train_kw = {}
    if compile_backend:
        train_kw = dict(torch_compile=True, torch_compile_backend=compile_backend, torch_compile_scope="backbones")
    cfg = Config(model=ModelConfig(hf={"model_size": "xsmall"}, tokenizer={"name_or_path": "synthetic:4096"},
                                   gradient_checkpointing=grad_ckpt),
                 data=DataConfig(dataset_name="synthetic", max_seq_length=256),
                 train=TrainConfig(mixed_precision=precision, per_device_train_batch_size=4, gradient_accumulation_steps=1,
                                   max_steps=10, dataloader_num_workers=0, distributed={"overlap_backward": overlap},
                                   **train_kw),
                 optim=OptimConfig(warmup_steps=1))
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        validate_config(cfg)
    torch.manual_seed(0)
    tok = build_tokenizer(cfg.model)
    model, _, _ = build_model(model_cfg=cfg.model, tokenizer=tok, max_seq_length=256)
    ctx = DistContext(device=torch.device("cuda", 0))
    engine = build_engine(model=model, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim)
    trainer = Trainer(model=model, engine=engine, ctx=ctx, train_cfg=cfg.train, optim_cfg=cfg.optim, pad_token_id=0,
                      synchronous=synchronous)
    maybe_compile_model(model, train_cfg=cfg.train, model_cfg=cfg.model, data_cfg=cfg.data)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(5, 4096, (4, 256), generator=g)
    labels = torch.full_like(ids, -100)
    pick = torch.rand(4, 256, generator=g) < 0.15
    labels[pick] = ids[pick]
    ids[pick] = tok.mask_token_id
    out = []
    for w in range(windows):
        torch.manual_seed(50 + w)
        st = trainer.train_window([{"input_ids": ids, "labels": labels}])
        if not synchronous:
            continue
        out.append((float(st.gen_loss_tokens) / st.gen_tokens, float(st.disc_loss_tokens) / st.disc_tokens,
                    float(st.grad_norms["generator"]), float(st.grad_norms["discriminator"])))
    trainer.wait_for_side_stream()
    trainer.resolve_pending()
    _lib.check_status()
    if return_engine:
        return trainer, engine
    return out


def test_discriminator_update_on_the_side_stream_matches_the_serial_schedule():
    """Four windows with the discriminator's collective + AdamW queued on a side stream (outcomes read one window
    late) end in the same masters and step counters as the fully serial schedule."""
    t_ser, e_ser = _tiny_step("bf16", synchronous=False, overlap=False, windows=4, return_engine=True)
    _, e_again = _tiny_step("bf16", synchronous=False, overlap=False, windows=4, return_engine=True)
    t_ovl, e_ovl = _tiny_step("bf16", synchronous=False, overlap=True, windows=4, return_engine=True)
    assert t_ovl.overlap and not t_ser.overlap
    torch.cuda.synchronize()
    # Two serial runs already differ: dQ and embedding gradients are summed with floating-point atomics, and Adam turns
    # a sign flip of a tiny gradient into a full learning-rate step. The side-stream schedule must stay inside that noise.
    noise = (e_ser.master - e_again.master).abs()
    diff = (e_ser.master - e_ovl.master).abs()
    assert float(diff.mean()) <= 3 * float(noise.mean()) + 1e-7, (float(diff.mean()), float(noise.mean()))
    assert float(diff.max()) <= 3 * float(noise.max()) + 1e-4, (float(diff.max()), float(noise.max()))
    assert [o.step for o in e_ser.optimizers.values()] == [o.step for o in e_ovl.optimizers.values()] == [4, 4]
    assert float(e_ovl.grads.abs().max()) == 0.0  # both ranges were cleared after their updates


def test_whole_rtd_step_bf16_kernels_match_fp32_modules():
    fast, ref = _tiny_step("bf16"), _tiny_step("no")
    for (gl, dl, gn, dn), (rgl, rdl, rgn, rdn) in zip(fast, ref):
        assert abs(gl - rgl) < 2e-2 * rgl and abs(dl - rdl) < 5e-2 * rdl
        assert abs(gn - rgn) < 0.15 * rgn and abs(dn - rdn) < 0.25 * rdn  # the discriminator sees sampled tokens


def test_activation_checkpointing_leaves_the_step_unchanged():
    """Per-layer recomputation (non-reentrant checkpoints) with the fused blocks: the residual-gradient hand-over
    between the attention block's two projections, the side-by-side QKV gradients and the saved position bias all have
    to survive a forward that runs twice. Losses and gradient norms must match the plain step within atomics noise."""
    from deberta_b200.ops import heads_cuda

    heads_cuda._SEED_STATE["counter"] = 0  # both runs draw the same replacement tokens
    plain = _tiny_step("bf16")
    heads_cuda._SEED_STATE["counter"] = 0
    ckpt = _tiny_step("bf16", grad_ckpt=True)
    for (gl, dl, gn, dn), (cgl, cdl, cgn, cdn) in zip(plain, ckpt):
        assert abs(gl - cgl) < 5e-3 * gl and abs(dl - cdl) < 1e-2 * dl
        assert abs(gn - cgn) < 3e-2 * gn and abs(dn - cdn) < 3e-2 * dn


@pytest.mark.parametrize("backend", ["aot_eager", "inductor"])
def test_compiled_train_step_has_no_graph_breaks_and_matches_eager(backend):
    import torch._dynamo as dynamo

    dynamo.reset()
    from torch._dynamo.utils import counters

    counters.clear()
    eager = _tiny_step("bf16")
    compiled = _tiny_step("bf16", compile_backend=backend)
    breaks = sum(counters["graph_break"].values())
    assert counters["stats"]["unique_graphs"] >= 2, "nothing was compiled"
    assert breaks == 0, dict(counters["graph_break"])
    for (gl, dl, _, _), (cgl, cdl, _, _) in zip(eager, compiled):
        assert math.isfinite(cgl) and math.isfinite(cdl)
        assert abs(gl - cgl) < 2e-2 * gl and abs(dl - cdl) < 5e-2 * dl
    dynamo.reset()


@pytest.mark.parametrize("V,T,banned", [(64, 0.7, True), (64, 1.0, True), (1000, 1.0, False), (1000, 1.3, True)])
def test_fused_sampler_frequencies_follow_softmax_chi_square(V, T, banned):
    """The sample frequencies of 40 000 draws must pass a chi-square test against ``softmax(logits / T)`` renormalised
    over the allowed ids: one and several vocabulary tiles (V = 1000 ends in a ragged 8-column chunk), unit and other
    temperatures (two code paths in the kernel), with and without forbidden ids."""
    from deberta_b200.ops.heads import mlm_loss_and_sample

    torch.manual_seed(3)
    E = 64
    w = (torch.randn(V, E, device="cuda") * 0.3).to(torch.bfloat16)
    b = (torch.randn(V, device="cuda") * 0.5).to(torch.bfloat16)
    x_row = (torch.randn(E, device="cuda") * 0.5).to(torch.bfloat16)
    forb = torch.zeros(V, dtype=torch.bool, device="cuda")
    if banned:
        forb[[0, 1, 2, 3, 17, 40]] = True
    logits = (x_row.float() @ w.float().t() + b.float()) / T
    probs = torch.softmax(logits.masked_fill(forb, -1e9), dim=-1).double().cpu()
    N, rounds = 4000, 10
    x = x_row[None].expand(N, E).contiguous()
    labels = torch.full((N,), 5, device="cuda")
    counts = torch.zeros(V, dtype=torch.float64)
    for _ in range(rounds):
        _, s = mlm_loss_and_sample(x, w, b, labels, forb if banned else None, T)
        counts += torch.bincount(s.cpu(), minlength=V).double()
    _lib.check_status()
    assert float(counts[forb.cpu()].sum()) == 0.0
    total = N * rounds
    exp = probs * total
    use = exp > 5  # the usual validity rule of the test; rare ids are pooled
    chi = float((((counts - exp) ** 2) / exp)[use].sum())
    rest_exp, rest_obs = float(exp[~use].sum()), float(counts[~use].sum())
    dof = int(use.sum()) - 1
    if rest_exp > 5:
        chi += (rest_obs - rest_exp) ** 2 / rest_exp
        dof += 1
    # 99.9 % quantile of chi-square by the Wilson-Hilferty approximation
    z = 3.09
    crit = dof * (1 - 2 / (9 * dof) + z * math.sqrt(2 / (9 * dof))) ** 3
    assert chi < crit, (chi, crit, dof)
