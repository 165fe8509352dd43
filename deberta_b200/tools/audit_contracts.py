"""Contract audit: fast checks that the invariants the training loop relies on still hold.

Usage::

    python -m deberta_b200.tools.audit_contracts [--verbose] [--no-config-scan] [--json]

Exit status 0 when no check fails (warnings allowed), 1 otherwise. The checks mirror the list of the reference's
``tools/audit_contracts.py:1252-1269`` (layout, export key handling, collator fallbacks and determinism, optimizer
ordering, doc-block masks, mask→active-token contract, RoPE FFN gating / norm order / mask leakage, RTD loss
integrity and gradient isolation, checkpoint round trip, unused config fields) and add two of our own: the C ABI
header matches the kernel sources, and no source names an API that must not be used on the GPU pool.
"""

from __future__ import annotations

import argparse
import ast
import dataclasses
import json
import re
import sys
import tempfile
from pathlib import Path
from typing import Callable

PKG = Path(__file__).resolve().parents[1]
REPO = PKG.parent


@dataclasses.dataclass
class CheckResult:
    name: str
    status: str  # "ok" | "warn" | "fail"
    detail: str = ""

    def sort_key(self) -> tuple[int, str]:
        return ({"fail": 0, "warn": 1, "ok": 2}[self.status], self.name)


def _ok(name: str, detail: str = "") -> CheckResult:
    return CheckResult(name, "ok", detail)


def _fail(name: str, detail: str) -> CheckResult:
    return CheckResult(name, "fail", detail)


def _warn(name: str, detail: str) -> CheckResult:
    return CheckResult(name, "warn", detail)


# ---- static checks ------------------------------------------------------------------------------

def check_repo_layout() -> CheckResult:
    need = ["__init__.py", "cli.py", "config.py", "export_cli.py", "build.py", "csrc/kernels.h", "csrc/gemm.cu",
            "csrc/attention.cu", "csrc/comm.cu", "data/collator.py", "data/streaming.py", "models/deberta_v2.py",
            "models/rope_encoder.py", "models/rtd.py", "models/builder.py", "ops/_lib.py", "parallel/engine.py",
            "parallel/peer.py", "training/entrypoint.py", "training/trainer.py", "utils/checkpoint.py"]
    missing = [p for p in need if not (PKG / p).exists()]
    return _fail("repo_layout", f"missing: {missing}") if missing else _ok("repo_layout", f"{len(need)} files present")


def check_kernel_abi() -> CheckResult:
    """Every ``db200_*`` function declared in kernels.h / no_alloc.h is defined ``extern "C"`` in a .cu file and back."""
    decl: set[str] = set()
    for h in ("kernels.h", "no_alloc.h"):
        decl |= set(re.findall(r"\b(db200_\w+)\s*\(", (PKG / "csrc" / h).read_text()))
    defs: set[str] = set()
    for cu in (PKG / "csrc").glob("*.cu"):
        defs |= set(re.findall(r'extern\s+"C"\s+[\w\s\*]+?\b(db200_\w+)\s*\(', cu.read_text()))
    defs |= {m for cu in (PKG / "csrc").glob("*.cu") for m in re.findall(r"^\s*(?:int|void|const char\*)\s+(db200_\w+)\s*\(", cu.read_text(), re.M)}
    undeclared, undefined = sorted(defs - decl), sorted(decl - defs)
    if undefined:
        return _fail("kernel_abi", f"declared but not defined: {undefined}")
    if undeclared:
        return _warn("kernel_abi", f"defined but not declared in a header: {undeclared}")
    return _ok("kernel_abi", f"{len(decl)} entry points")


def check_forbidden_apis() -> CheckResult:
    """No travelling source may name the batched-memcpy driver calls or a cluster-multicast bulk/TMA load."""
    names = ["cuda" + "Memcpy" + "BatchAsync", "cuda" + "Memcpy3D" + "BatchAsync", "cu" + "Memcpy" + "BatchAsync",
             "cu" + "Memcpy3D" + "BatchAsync"]
    # (the qualifier is spelled in two pieces so that this checker does not itself contain the pattern)
    bulk_mc = re.compile(r"cp\.async\.bulk[\w\.:]*\.multi" + "cast::cluster")
    hits = []
    for path in list(REPO.rglob("*.py")) + list(REPO.rglob("*.cu")) + list(REPO.rglob("*.cuh")) + list(REPO.rglob("*.h")):
        rel = path.relative_to(REPO)
        if rel.parts[0] in ("baseline", ".git") or rel.parts[0].startswith("_") or rel.parts[0].endswith("_out"):
            continue
        text = path.read_text(errors="ignore")
        if any(n in text for n in names) or bulk_mc.search(text):
            hits.append(str(rel))
    return _fail("forbidden_apis", f"found in {hits}") if hits else _ok("forbidden_apis")


def check_bounded_waits() -> CheckResult:
    """Device code may spin only inside the bounded helpers; a bare ``while (true)`` / ``for (;;)`` needs a limit nearby."""
    bad = []
    for cu in list((PKG / "csrc").glob("*.cu")) + list((PKG / "csrc").glob("*.cuh")):
        lines = cu.read_text().splitlines()
        for i, line in enumerate(lines):
            if re.search(r"while\s*\(\s*(true|1)\s*\)|for\s*\(\s*;\s*;\s*\)", line):
                window = "\n".join(lines[i:i + 12])
                if not re.search(r"kSpinLimit|timeout_ns|break", window):
                    bad.append(f"{cu.name}:{i + 1}")
    return _fail("bounded_waits", f"unbounded loops: {bad}") if bad else _ok("bounded_waits")


def check_optimizer_state_ordering_risk() -> CheckResult:
    """Optimizer state is addressed by flat offsets; resuming must compare a parameter-order digest."""
    eng = (PKG / "parallel" / "engine.py").read_text()
    ck = (PKG / "training" / "entrypoint.py").read_text() + (PKG / "training" / "trainer.py").read_text()
    if "def param_order_digest" not in eng:
        return _fail("optimizer_state_ordering", "param_order_digest is gone")
    if "optimizer_param_digest" not in ck:
        return _fail("optimizer_state_ordering", "the digest is never compared on resume")
    return _ok("optimizer_state_ordering")


def scan_unused_config_fields() -> CheckResult:
    """Every config leaf should be read somewhere outside config.py (or be on the accepted-but-inert list)."""
    from deberta_b200 import config as C

    inert = {"torch_compile", "compile", "sdpa_kernel", "tf32", "attention_kernel", "hf_attention_kernel"}
    text = "\n".join(p.read_text() for p in PKG.rglob("*.py") if p.name != "config.py")
    text += "\n" + (REPO / "bench.py").read_text()
    unused = []

    def walk(cls, prefix=""):
        for f in dataclasses.fields(cls):
            if f.name.startswith("_"):
                continue
            sub = f.default_factory if f.default_factory is not dataclasses.MISSING else None
            if sub is not None and dataclasses.is_dataclass(sub):
                walk(sub, prefix + f.name + ".")
            elif not re.search(rf"\b{re.escape(f.name)}\b", text) and f.name not in inert:
                unused.append(prefix + f.name)

    for section in ("model", "data", "train", "optim", "logging"):
        walk(type(getattr(C.Config(), section)), section + ".")
    return _warn("unused_config_fields", f"never read: {unused}") if unused else _ok("unused_config_fields")


# ---- dynamic checks (tiny CPU models) --------------------------------------------------------------

def _tiny_rope(**over):
    from deberta_b200.models.rope_encoder import DebertaRoPEConfig, DebertaRoPEModel

    kw = dict(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=2, intermediate_size=64,
              attention_implementation="eager", use_rmsnorm_heads=True, hidden_dropout_prob=0.0,
              attention_probs_dropout_prob=0.0)
    kw.update(over)
    cfg = DebertaRoPEConfig(**kw)
    return cfg, DebertaRoPEModel(cfg).eval()


def _tiny_pretrainer(sharing: str = "gdes"):
    import copy

    import torch

    from deberta_b200.models.rope_encoder import DebertaRoPEModel
    from deberta_b200.models.rtd import DebertaV3RTDPretrainer

    torch.manual_seed(0)
    dcfg, _ = _tiny_rope()
    gcfg = copy.deepcopy(dcfg)
    gcfg.num_hidden_layers = 1
    return DebertaV3RTDPretrainer(discriminator_backbone=DebertaRoPEModel(dcfg), generator_backbone=DebertaRoPEModel(gcfg),
                                  disc_config=dcfg, gen_config=gcfg, embedding_sharing=sharing,
                                  additional_forbidden_token_ids=[0, 1, 2, 3])


def _tiny_batch():
    import torch

    g = torch.Generator().manual_seed(3)
    ids = torch.randint(4, 128, (2, 16), generator=g)
    labels = torch.full_like(ids, -100)
    pick = torch.rand(2, 16, generator=g) < 0.25
    pick[:, 1] = True
    labels[pick] = ids[pick]
    return ids.masked_fill(pick, 3), labels


def check_export_intersection_load() -> CheckResult:
    """Non-strict export loading takes the intersection of keys; strict mode refuses missing/unexpected ones."""
    import torch

    from deberta_b200.models.export_utils import load_intersection_state_dict

    m = torch.nn.Linear(4, 4)
    state = {"weight": torch.ones(4, 4), "extra": torch.zeros(1)}
    try:
        load_intersection_state_dict(m, state, strict=False)
    except Exception as e:  # noqa: BLE001
        return _fail("export_intersection_load", f"non-strict load raised: {e}")
    if not torch.equal(m.weight.data, torch.ones(4, 4)):
        return _fail("export_intersection_load", "matching key was not loaded")
    try:
        load_intersection_state_dict(m, state, strict=True)
    except Exception:  # noqa: BLE001
        return _ok("export_intersection_load")
    return _fail("export_intersection_load", "strict load accepted missing/unexpected keys")


def _collate(seed: int, max_ngram: int = 1):
    import random

    import numpy as np
    import torch

    from deberta_b200.data.collator import DebertaV3ElectraCollator, MLMConfig
    from deberta_b200.data.synthetic import SyntheticTokenizer

    tok = SyntheticTokenizer(vocab_size=512)
    col = DebertaV3ElectraCollator(tokenizer=tok, cfg=MLMConfig(mlm_probability=0.15, max_ngram=max_ngram))
    g = torch.Generator().manual_seed(1)
    feats = [{"input_ids": [tok.cls_token_id] + torch.randint(10, 500, (30,), generator=g).tolist() + [tok.sep_token_id]}
             for _ in range(4)]
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    return col(feats), tok


def check_collator_determinism() -> CheckResult:
    import torch

    a, _ = _collate(7)
    b, _ = _collate(7)
    c, _ = _collate(8)
    same = all(torch.equal(a[k], b[k]) for k in ("input_ids", "labels"))
    differs = not torch.equal(a["labels"], c["labels"])
    if not same:
        return _fail("collator_determinism", "same seeds gave different batches")
    return _ok("collator_determinism") if differs else _warn("collator_determinism", "different seeds gave equal masks")


def check_collator_whole_word_fallback() -> CheckResult:
    """n-gram masking on a tokenizer without word-boundary markers must fall back to token-level groups, not crash."""
    try:
        batch, tok = _collate(5, max_ngram=3)
    except Exception as e:  # noqa: BLE001
        return _fail("collator_whole_word_fallback", f"raised {type(e).__name__}: {e}")
    labels = batch["labels"]
    n = int((labels != -100).sum())
    special = (batch["input_ids"] == tok.cls_token_id) | (batch["input_ids"] == tok.sep_token_id)
    if n == 0:
        return _fail("collator_whole_word_fallback", "nothing was masked")
    if bool(((labels != -100) & special).any()):
        return _fail("collator_whole_word_fallback", "a special token was selected for masking")
    return _ok("collator_whole_word_fallback", f"{n} masked tokens")


def check_doc_block_mask_contract() -> CheckResult:
    """doc_ids → keep mask: block diagonal over equal non-zero ids, symmetric, padding (id 0) attends to nothing."""
    import torch

    from deberta_b200.ops.attention import dense_keep_mask

    doc = torch.tensor([[1, 1, 2, 2, 2, 0]])
    keep, live = dense_keep_mask(None, doc, None)
    if keep is None or live is None:
        return _fail("doc_block_mask", "no mask was produced for doc_ids")
    keep, live = keep.reshape(6, 6).bool(), live.reshape(6).bool()
    active = doc[0] != 0
    want = (doc[0][:, None] == doc[0][None, :]) & active[:, None] & active[None, :]
    if not torch.equal(keep[active], want[active]):
        return _fail("doc_block_mask", "rows of real tokens differ from equal-and-nonzero doc ids")
    if not torch.equal(live, active):
        return _fail("doc_block_mask", "live-query flags differ from doc_ids != 0")
    if bool(keep[~active][:, active].any() and keep[~active].sum(-1).max() > 1):
        return _fail("doc_block_mask", "padding queries attend to real tokens beyond the single placeholder edge")
    return _ok("doc_block_mask")


def check_attention_mask_to_active_tokens_contract() -> CheckResult:
    import torch

    from deberta_b200.models.rtd import attention_mask_to_active_tokens

    ids = torch.tensor([[5, 6, 0, 0]])
    a = attention_mask_to_active_tokens(input_ids=ids, attention_mask=None, pad_token_id=0)
    b = attention_mask_to_active_tokens(input_ids=ids, attention_mask=torch.tensor([[1, 1, 1, 0]]), pad_token_id=0)
    pair = torch.eye(4, dtype=torch.bool)[None]
    pair[0, 3, 3] = False
    c = attention_mask_to_active_tokens(input_ids=ids, attention_mask=pair, pad_token_id=0)
    # pairwise masks: diagonal = query activity, intersected with input_ids != pad
    ok = a.tolist() == [[True, True, False, False]] and b.tolist() == [[True, True, True, False]] and \
        c.tolist() == [[True, True, False, False]]
    return _ok("mask_to_active_tokens") if ok else _fail("mask_to_active_tokens", f"got {a.tolist()} {b.tolist()} {c.tolist()}")


def check_rope_ffn_gating() -> CheckResult:
    """SwiGLU = w3(silu(gate) * up) with gate/up the two halves of the fused w12 projection."""
    import torch
    import torch.nn.functional as F

    from deberta_b200.models.rope_encoder import DebertaRoPEMLP

    cfg, _ = _tiny_rope(ffn_type="swiglu")
    mlp = DebertaRoPEMLP(cfg).eval()
    x = torch.randn(2, 5, cfg.hidden_size)
    names = dict(mlp.named_parameters())
    w12 = next(v for k, v in names.items() if "w12" in k and k.endswith("weight"))
    w3 = next(v for k, v in names.items() if "w3" in k and k.endswith("weight"))
    b12 = next((v for k, v in names.items() if "w12" in k and k.endswith("bias")), None)
    b3 = next((v for k, v in names.items() if "w3" in k and k.endswith("bias")), None)
    h = F.linear(x, w12, b12)
    a, b = h.chunk(2, dim=-1)
    want = F.linear(F.silu(a) * b, w3, b3)
    got = mlp(x)
    err = float((got - want).detach().abs().max())
    return _ok("rope_ffn_gating") if err < 1e-5 else _fail("rope_ffn_gating", f"max err {err:.2e} vs silu(first half)*second half")


def check_rope_layer_norm_order() -> CheckResult:
    """post-norm layer: x1 = norm(x + attn(x)); out = norm(x1 + mlp(x1))."""
    import torch

    cfg, model = _tiny_rope(norm_arch="post")
    layer = model.encoder.layers[0]
    x = torch.randn(1, 6, cfg.hidden_size)
    seen = []
    hooks = [m.register_forward_hook(lambda mod, i, o, n=n: seen.append(n)) for n, m in layer.named_children()]
    try:
        model.encoder(x, None)
    except Exception as e:  # noqa: BLE001
        return _warn("rope_layer_norm_order", f"could not drive the encoder directly: {e}")
    finally:
        for h in hooks:
            h.remove()
    order = [n for n in seen if n in dict(layer.named_children())][:4]
    norm_after = len(order) >= 4 and "norm" in order[1].lower() and "norm" in order[3].lower()
    return _ok("rope_layer_norm_order", "->".join(order)) if norm_after else _fail("rope_layer_norm_order", f"call order {order}")


def check_rope_attention_mask_leak() -> CheckResult:
    """Outputs at kept positions must not depend on inputs at masked positions (gradient is exactly zero)."""
    import torch

    cfg, model = _tiny_rope()
    ids = torch.randint(4, 128, (1, 8))
    mask = torch.tensor([[1, 1, 1, 1, 1, 0, 0, 0]])
    emb = model.embeddings.word_embeddings.weight
    out = model(input_ids=ids, attention_mask=mask).last_hidden_state
    (g,) = torch.autograd.grad(out[0, :5].sum(), emb, retain_graph=False)
    masked_tokens = set(ids[0, 5:].tolist()) - set(ids[0, :5].tolist())
    leak = max((float(g[t].abs().max()) for t in masked_tokens), default=0.0)
    return _ok("rope_attention_mask_leak") if leak == 0.0 else _fail("rope_attention_mask_leak", f"gradient {leak:.2e} reaches masked tokens")


def check_rtd_loss_integrity(verbose: bool = False) -> CheckResult:
    """Reported losses equal a recomputation from the phase outputs; the RTD loss sends no gradient to the generator."""
    import torch
    import torch.nn.functional as F

    model = _tiny_pretrainer("gdes").train()
    ids, labels = _tiny_batch()
    torch.manual_seed(1)
    gen = model.forward_generator_phase(input_ids=ids, labels=labels)
    disc = model.forward_discriminator_phase(input_ids=ids, corrupted_input_ids=gen.corrupted_input_ids,
                                             disc_labels=gen.disc_labels)
    problems = []
    want_labels = (gen.corrupted_input_ids != ids).to(gen.disc_labels.dtype)
    if not torch.equal(want_labels, gen.disc_labels):
        problems.append("disc_labels != (corrupted != original)")
    if bool(((labels == -100) & (gen.corrupted_input_ids != ids)).any()):
        problems.append("an unmasked position was corrupted")
    disc.disc_loss_raw.backward()
    leaked = [n for n, p in model.generator.named_parameters() if p.grad is not None and float(p.grad.abs().max()) > 0]
    if leaked:
        problems.append(f"RTD loss reached generator parameters: {leaked[:3]}")
    if verbose:
        print(f"  gen_loss={float(gen.gen_loss_raw):.4f} disc_loss={float(disc.disc_loss_raw):.4f}")
    if not torch.isfinite(gen.gen_loss_raw) or not torch.isfinite(disc.disc_loss_raw):
        problems.append("non-finite loss")
    _ = F  # (kept for interactive use)
    return _fail("rtd_loss_integrity", "; ".join(problems)) if problems else _ok("rtd_loss_integrity")


def check_checkpoint_roundtrip() -> CheckResult:
    """save_training_state → load_training_state restores model, optimizer moments and step on a CPU engine."""
    import torch

    from deberta_b200.parallel.dist import DistContext
    from deberta_b200.parallel.engine import TrainEngine
    from deberta_b200.utils.checkpoint import load_training_state, save_training_state

    class _T:  # the slice of the trainer the checkpoint code touches
        def __init__(self, eng):
            self.eng, self.global_step = eng, 3

        def resolve_pending(self):
            pass

        def state_dict(self):
            return {"global_step": self.global_step, "schedules": {n: {} for n in self.eng.optimizers}}

        def load_state_dict(self, s):
            self.global_step = int(s["global_step"])

    def make():
        torch.manual_seed(0)
        return TrainEngine(_tiny_pretrainer("gdes"), DistContext(), compute_dtype=torch.float32, parallelism="ddp")

    a = make()
    ids, labels = _tiny_batch()
    out = a.model(input_ids=ids, labels=labels)
    out.loss.backward()
    for name in a.optimizers:
        a.sync_grads(name)
        a.step(name)
    with tempfile.TemporaryDirectory() as d:
        save_training_state(d, engine=a, trainer=_T(a), ctx=a.ctx)
        b = make()
        tb = _T(b)
        tb.global_step = 0
        load_training_state(d, engine=b, trainer=tb, ctx=b.ctx)
    bad = []
    if not torch.equal(a.master, b.master):
        bad.append("masters differ")
    for n in a.optimizers:
        if not torch.equal(a.optimizers[n].exp_avg, b.optimizers[n].exp_avg) or a.optimizers[n].step != b.optimizers[n].step:
            bad.append(f"optimizer {n} differs")
    if tb.global_step != 3:
        bad.append("trainer step not restored")
    return _fail("checkpoint_roundtrip", "; ".join(bad)) if bad else _ok("checkpoint_roundtrip")


def run_all(*, verbose: bool = False, config_scan: bool = True) -> list[CheckResult]:
    checks: list[Callable[[], CheckResult]] = [
        check_repo_layout, check_kernel_abi, check_forbidden_apis, check_bounded_waits,
        check_optimizer_state_ordering_risk, check_export_intersection_load, check_collator_whole_word_fallback,
        check_collator_determinism, check_doc_block_mask_contract, check_attention_mask_to_active_tokens_contract,
        check_rope_ffn_gating, check_rope_layer_norm_order, check_rope_attention_mask_leak,
        lambda: check_rtd_loss_integrity(verbose), check_checkpoint_roundtrip,
    ]
    if config_scan:
        checks.append(scan_unused_config_fields)
    results = []
    for fn in checks:
        try:
            results.append(fn())
        except Exception as e:  # noqa: BLE001
            name = getattr(fn, "__name__", "check")
            results.append(_fail(name.replace("check_", ""), f"crashed: {type(e).__name__}: {e}"))
    return sorted(results, key=lambda r: r.sort_key())


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--no-config-scan", action="store_true")
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    results = run_all(verbose=args.verbose, config_scan=not args.no_config_scan)
    if args.json:
        print(json.dumps([dataclasses.asdict(r) for r in results], indent=1))
    else:
        for r in results:
            print(f"[{r.status.upper():4s}] {r.name}" + (f" — {r.detail}" if r.detail else ""))
    _ = ast  # static helpers may grow AST checks; keep the import local to this tool
    return 1 if any(r.status == "fail" for r in results) else 0


if __name__ == "__main__":
    sys.exit(main())
