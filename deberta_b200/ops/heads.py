"""Objective heads: vocabulary cross-entropy fused with Gumbel-max sampling, and the RTD loss.

``mlm_loss_and_sample`` evaluates, for the N masked rows only, the tied-embedding
vocabulary projection, the mean fp32 cross-entropy and one sample per row from
``softmax(logits / T)`` with forbidden ids excluded (the reference draws it by Gumbel-max) — the
three steps of ``rtd.py:1066-1078`` of the reference. The PyTorch implementation materialises the
``[N, V]`` logits; the sm_100a kernel (the cross-entropy epilogue of ``csrc/gemm.cu``, behind
``ops/heads_cuda.py``) sweeps vocabulary tiles once with online log-sum-exp and a two-level exact
sampler (an id per 32-column chunk by inverse CDF, Gumbel-max over the chunks' masses), so the
logits never reach HBM.

``rtd_loss`` is the masked-mean binary cross-entropy of the discriminator with its
accuracy / count statistics (``rtd.py:1123-1145``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

__all__ = ["mlm_loss_and_sample", "mlm_loss_and_sample_reference", "gumbel_sample", "rtd_loss", "RTDStats"]


def gumbel_sample(logits: torch.Tensor, *, temperature: float, forbidden_vocab_mask: torch.Tensor | None) -> torch.Tensor:
    """``argmax(logits/T − 1e9·forbidden + G)``, ``G = −ln(−ln U)``, ``U ∈ [1e-6, 1−1e-6]`` (``rtd.py:935-982``)."""
    temp = float(temperature)
    if temp <= 0:
        raise ValueError("sampling_temperature must be > 0")
    x = logits.float() / temp
    if forbidden_vocab_mask is not None and forbidden_vocab_mask.numel() != 0:
        mask = forbidden_vocab_mask.to(device=x.device, dtype=torch.bool)
        if int(mask.shape[-1]) != int(x.shape[-1]):
            raise ValueError(
                "forbidden_vocab_mask length must match logits vocabulary dimension: "
                f"{int(mask.shape[-1])} vs {int(x.shape[-1])}."
            )
        try:
            x = x.masked_fill(mask if mask.ndim == 1 else mask.expand_as(x), -1e9)
        except RuntimeError as exc:
            raise ValueError("forbidden_vocab_mask with rank > 1 must be broadcastable to logits.") from exc
    u = torch.rand_like(x).clamp_(min=1e-6, max=1.0 - 1e-6)
    return torch.argmax(x - torch.log(-torch.log(u)), dim=-1)


def mlm_loss_and_sample_reference(x, weight, bias, labels, forbidden_mask, temperature: float):
    """PyTorch statement: returns (mean CE over rows, sampled ids ``[N]`` int64)."""
    logits = F.linear(x, weight.to(x.dtype), None if bias is None else bias.to(x.dtype))
    loss = F.cross_entropy(logits.float(), labels)
    with torch.no_grad():
        sampled = gumbel_sample(logits, temperature=temperature, forbidden_vocab_mask=forbidden_mask)
    return loss, sampled


def mlm_loss_and_sample(x, weight, bias, labels, forbidden_mask, temperature: float):
    """Dispatch: fused sm_100a vocabulary sweep on bf16 CUDA inputs, PyTorch otherwise."""
    from . import heads_cuda

    if heads_cuda.vocab_ce_supported(x, weight):
        return heads_cuda.mlm_loss_and_sample_cuda(x, weight, bias, labels, forbidden_mask, temperature)
    return mlm_loss_and_sample_reference(x, weight, bias, labels, forbidden_mask, temperature)


@dataclass
class RTDStats:
    loss: torch.Tensor
    accuracy: torch.Tensor
    token_count: torch.Tensor
    positive_count: torch.Tensor


def rtd_loss(logits: torch.Tensor, labels: torch.Tensor, active: torch.Tensor) -> RTDStats:
    """Masked-mean BCE-with-logits over ``active`` tokens plus accuracy and counts (all fp32 scalars)."""
    act = active.to(torch.float32)
    count = act.sum()
    denom = count.clamp(min=1.0)
    per_tok = F.binary_cross_entropy_with_logits(logits.float(), labels.float(), reduction="none")
    loss = (per_tok * act).sum() / denom
    with torch.no_grad():
        truth = labels.gt(0.5)
        positive = (truth.to(torch.float32) * act).sum()
        acc = ((logits.gt(0) == truth).to(torch.float32) * act).sum() / denom
    return RTDStats(loss=loss, accuracy=acc.detach(), token_count=count.detach(), positive_count=positive.detach())
