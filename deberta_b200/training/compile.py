"""``train.compile``: compile the Python glue of chosen sub-modules around the kernel ops.

The hot operators are precompiled sm_100a kernels and stay exactly that: while a compiler traces, the operator
functions of ``deberta_b200.ops`` hand it their ``db200::*`` custom ops (``ops/library.py``), which Dynamo,
AOTAutograd and Inductor carry as opaque nodes. What ``torch.compile`` then owns is what lies between them —
reshapes, residual bookkeeping, mask handling, module dispatch — as in the reference, which compiles its eager
modules scope by scope (``training/compile.py:129-265`` there). Off by default.

Scopes: ``backbones`` (both backbone modules), ``encoder`` / ``gen_encoder`` / ``disc_encoder`` (the layer stacks),
``ffn`` / ``gen_ffn`` / ``disc_ffn`` (the feed-forward modules of every layer); ``auto`` picks ``backbones``, or ``ffn``
for the rope backbone with cross-document blocking (document ids change the traced mask structure from batch to batch).
A module's ``forward`` attribute is replaced in place, so parameter names (and checkpoints) do not change.
"""

from __future__ import annotations

import logging
from typing import Any

import torch

logger = logging.getLogger(__name__)

__all__ = ["resolve_compile_scope", "compile_model_for_scope", "maybe_compile_model"]


def resolve_compile_scope(*, requested_scope: str, backbone_type: str, block_cross_document_attention: bool = False):
    """(effective scope, reason or ``None``) for a requested scope; only ``auto`` is ever changed."""
    scope = str(requested_scope).strip().lower()
    if scope != "auto":
        return scope, None
    if block_cross_document_attention and str(backbone_type).strip().lower() == "rope":
        return "ffn", "auto scope selected FFN-only for rope + doc-blocking (mask shape churn under compile)"
    return "backbones", None


def _ffn_modules(backbone: torch.nn.Module, branch: str) -> list[tuple[str, torch.nn.Module]]:
    enc = getattr(backbone, "encoder", None)
    if not isinstance(enc, torch.nn.Module):
        raise RuntimeError(f"{branch}.encoder is required for ffn-only compile scope.")
    for attr in ("layer", "layers"):
        layers = getattr(enc, attr, None)
        if isinstance(layers, torch.nn.ModuleList):
            break
    else:
        raise RuntimeError(f"{branch}.encoder.layer/layers is required for ffn-only compile scope.")
    if len(layers) == 0:
        raise RuntimeError(f"{branch}.encoder.{attr} is empty; cannot apply ffn-only compile scope.")
    out: list[tuple[str, torch.nn.Module]] = []
    for i, layer in enumerate(layers):
        pfx = f"{branch}.encoder.{attr}[{i}]"
        if isinstance(getattr(layer, "intermediate", None), torch.nn.Module) and \
                isinstance(getattr(layer, "output", None), torch.nn.Module):
            out += [(f"{pfx}.intermediate", layer.intermediate), (f"{pfx}.output", layer.output)]
            if hasattr(layer, "call_ffn_modules"):
                layer.call_ffn_modules = True  # the layer otherwise runs both as one fused operator
        elif isinstance(getattr(layer, "mlp", None), torch.nn.Module):
            out.append((f"{pfx}.mlp", layer.mlp))
        else:
            raise RuntimeError(f"{pfx} has no recognized FFN module (expected intermediate+output or mlp).")
    return out


def compile_model_for_scope(model: torch.nn.Module, scope: str, **compile_kwargs: Any) -> list[str]:
    """Replace ``forward`` of the modules the scope names by its compiled form; returns the names of what was compiled."""
    gen, disc = getattr(model, "generator", None), getattr(model, "discriminator", None)
    if not isinstance(gen, torch.nn.Module) or not isinstance(disc, torch.nn.Module):
        raise RuntimeError("RTD model must expose generator and discriminator modules for compilation.")
    todo: list[tuple[str, torch.nn.Module]] = []
    if scope == "backbones":
        todo = [("generator", gen), ("discriminator", disc)]
    else:
        for branch, backbone, tags in (("generator", gen, ("encoder", "gen_encoder")),
                                       ("discriminator", disc, ("encoder", "disc_encoder"))):
            if scope in tags:
                enc = getattr(backbone, "encoder", None)
                if not isinstance(enc, torch.nn.Module):
                    raise RuntimeError(f"{branch}.encoder is required for encoder-only compile scope.")
                todo.append((f"{branch}.encoder", enc))
        if scope in ("ffn", "gen_ffn"):
            todo += _ffn_modules(gen, "generator")
        if scope in ("ffn", "disc_ffn"):
            todo += _ffn_modules(disc, "discriminator")
    if not todo:
        raise ValueError(f"Unsupported compile scope: {scope}")
    for _name, module in todo:
        module.forward = torch.compile(module.forward, **compile_kwargs)  # identity of the module stays the same
    return [n for n, _ in todo]


def maybe_compile_model(model: torch.nn.Module, *, train_cfg: Any, model_cfg: Any, data_cfg: Any = None):
    """Apply ``train.compile`` to ``model``: (effective scope or ``None`` when disabled, reason, compiled targets)."""
    cc = train_cfg.compile
    if not bool(cc.enabled):
        return None, None, []
    blocking = bool(getattr(getattr(data_cfg, "packing", None), "block_cross_document_attention", False))
    scope, reason = resolve_compile_scope(requested_scope=cc.scope, backbone_type=model_cfg.backbone_type,
                                          block_cross_document_attention=blocking)
    kwargs: dict[str, Any] = {"backend": str(cc.backend), "dynamic": False}
    if str(cc.backend) == "inductor" and str(cc.mode) != "default":
        kwargs["mode"] = str(cc.mode)
    targets = compile_model_for_scope(model, scope, **kwargs)
    logger.info("torch.compile enabled (scope=%s, backend=%s, mode=%s): %d module(s)%s", scope, cc.backend, cc.mode,
                len(targets), f" — {reason}" if reason else "")
    return scope, reason, targets
