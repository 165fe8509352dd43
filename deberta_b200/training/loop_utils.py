"""Per-window arithmetic of the training loop (``training/loop_utils.py`` of the reference).

Token-weighted gradient accumulation: with per-micro-batch counts ``g_i`` (masked tokens)
and ``d_i`` (active tokens) and window totals per rank ``G``, ``D`` (mean over ranks), the
window objective is ``Σ_i w_g·(g_i/G)·gen_i + w_d·(d_i/D)·disc_i``; averaging gradients over
ranks then completes the global per-token normalisation.
"""

from __future__ import annotations

import torch

from deberta_b200.models.rtd import attention_mask_to_active_tokens

NONFINITE_LR_BACKOFF = 0.5
NONFINITE_LR_MULT_FLOOR = 0.01
NONFINITE_LR_MULT_RECOVERY = 1.1
NONFINITE_OPT_STATE_RESET_EVERY = 4


def count_rtd_tokens_for_batch(batch: dict[str, torch.Tensor], *, pad_token_id: int | None) -> tuple[float, float]:
    """(masked-token count, active-token count) of one micro-batch (host tensors: no device sync)."""
    gen = float(batch["labels"].ne(-100).sum().item())
    mask = batch.get("attention_mask")
    doc = batch.get("doc_ids")
    if doc is not None:
        active = doc.ne(0)
        if pad_token_id is not None:
            active = active & batch["input_ids"].ne(int(pad_token_id))
    else:
        active = attention_mask_to_active_tokens(input_ids=batch["input_ids"], attention_mask=mask, pad_token_id=pad_token_id)
    return gen, float(active.sum().item())


def count_input_tokens_for_batch(batch: dict[str, torch.Tensor]) -> float:
    """Non-padding input tokens (throughput accounting)."""
    if batch.get("doc_ids") is not None:
        return float(batch["doc_ids"].ne(0).sum().item())
    active = attention_mask_to_active_tokens(input_ids=batch["input_ids"], attention_mask=batch.get("attention_mask"),
                                             pad_token_id=None)
    return float(active.sum().item())


def token_weighted_micro_objective(*, gen_loss, disc_loss, gen_count: float, disc_count: float,
                                   gen_window_tokens_per_rank: float, disc_window_tokens_per_rank: float,
                                   gen_loss_weight: float, disc_loss_weight: float):
    gs = float(gen_count) / max(float(gen_window_tokens_per_rank), 1.0)
    ds = float(disc_count) / max(float(disc_window_tokens_per_rank), 1.0)
    return float(gen_loss_weight) * gs * gen_loss + float(disc_loss_weight) * ds * disc_loss


def resolve_window_token_denominators(*, gen_window_tokens_per_rank_raw: float, disc_window_tokens_per_rank_raw: float):
    """(gen denom ≥ 1, disc denom ≥ 1, gen window empty?, disc window empty?)."""
    g, d = float(gen_window_tokens_per_rank_raw), float(disc_window_tokens_per_rank_raw)
    return max(g, 1.0), max(d, 1.0), g <= 0.0, d <= 0.0


def micro_loss_scale(*, ga_steps: int, token_weighted_ga: bool) -> float:
    """Factor applied to a micro-batch objective before backward.

    Token-weighted objectives already sum to the window objective; plain means are divided
    by the number of micro-batches. (The reference reaches the same values by multiplying
    with ``ga_steps`` to cancel Accelerate's implicit division, ``loop_utils.py:113-125``.)
    """
    return 1.0 if token_weighted_ga else 1.0 / float(max(1, int(ga_steps)))


def finalize_window_metric_loss(*, accumulated_loss, ga_steps: int, token_weighted_ga: bool):
    return accumulated_loss if token_weighted_ga else accumulated_loss / float(max(1, int(ga_steps)))


def should_clip_gradients(*, sync_gradients: bool, max_grad_norm) -> bool:
    return bool(sync_gradients) and max_grad_norm is not None and float(max_grad_norm) > 0.0


def apply_nonfinite_recovery(*, lr_mult: float, skip_streak: int) -> tuple[float, bool]:
    """After a non-finite window: halve the persistent LR multiplier (floor 1 %); every 4th
    consecutive skip also asks for the optimizer moments to be cleared."""
    new = max(float(lr_mult) * NONFINITE_LR_BACKOFF, NONFINITE_LR_MULT_FLOOR)
    return new, int(skip_streak) % NONFINITE_OPT_STATE_RESET_EVERY == 0


def recover_lr_mult(lr_mult: float) -> float:
    """Gradual recovery (×1.1 per good step, capped at 1)."""
    return min(1.0, float(lr_mult) * NONFINITE_LR_MULT_RECOVERY)
