"""Replaced-token-detection pretraining module: generator + discriminator with embedding sharing.

Same module/parameter names and phase API as ``modeling/rtd.py`` of the reference
(``generator.*``, ``discriminator.*``, ``generator_lm_head.*``, ``discriminator_head.*``),
so checkpoints interchange. The per-step hot work — masked-row vocabulary projection +
cross-entropy + Gumbel sampling, RTD head + loss — goes through ``deberta_b200.ops``.
"""

from __future__ import annotations

from collections.abc import Iterable
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

from deberta_b200.ops.gather import gather_rows
from deberta_b200.ops.heads import gumbel_sample, mlm_loss_and_sample, rtd_loss
from deberta_b200.ops.linear import linear
from deberta_b200.ops.norm import layer_norm

from .activations import get_act_fn
from .mask_utils import AttnMask, normalize_keep_mask
from .norm import RMSNorm

__all__ = [
    "RTDOutput", "RTDGeneratorPhaseOutput", "RTDDiscriminatorPhaseOutput", "DebertaV3RTDPretrainer",
    "MaskedLMHead", "MLMTransform", "EnhancedMaskDecoder", "RTDHead", "attention_mask_to_active_tokens",
]


def attention_mask_to_active_tokens(*, input_ids, attention_mask, pad_token_id: int | None) -> torch.Tensor:
    """[B,S] bool activity from ``None`` / (B,S) / (B,S,S) / (B,H,S,S) masks (``rtd.py:55-102``).

    Pairwise masks carry query activity on their diagonal and are additionally
    intersected with ``input_ids != pad``.
    """
    if attention_mask is None:
        return torch.ones_like(input_ids, dtype=torch.bool) if pad_token_id is None else input_ids.ne(int(pad_token_id))
    if isinstance(attention_mask, AttnMask):
        m = attention_mask
    else:
        if attention_mask.ndim not in (2, 3, 4):
            raise ValueError("attention_mask must have shape (B,S), (B,S,S), or (B,H,S,S).")
        m = AttnMask.from_any(attention_mask)
    if m.key_keep is not None and not (isinstance(attention_mask, torch.Tensor) and attention_mask.ndim == 4):
        return m.key_keep
    active = m.token_keep()
    if active is None:
        return torch.ones_like(input_ids, dtype=torch.bool) if pad_token_id is None else input_ids.ne(int(pad_token_id))
    return active & input_ids.ne(int(pad_token_id)) if pad_token_id is not None else active


def _norm(mod: nn.Module, x: torch.Tensor) -> torch.Tensor:
    if isinstance(mod, nn.LayerNorm):
        return layer_norm(x, mod.weight, mod.bias, mod.eps)
    return mod(x)


def _is_sharded_dtensor(t: torch.Tensor) -> bool:
    t = t.detach()
    return bool(hasattr(t, "_local_tensor") and hasattr(t, "placements") and getattr(t, "placements", ()))


class _SyncedBufferEmbedding(nn.Module):
    """GDES embedding ``E(ids) = base_weight[ids] + bias[ids]`` (``rtd.py:157-226``).

    ``base_weight`` is a frozen copy of the generator table (refreshed after every
    generator step), ``bias`` is the discriminator's trainable delta. Gradients therefore
    reach only the delta: the discriminator loss never pulls on the generator embeddings.
    """

    def __init__(self, *, init_weight: torch.Tensor, padding_idx: int | None, add_bias: bool) -> None:
        super().__init__()
        if not isinstance(init_weight, torch.Tensor) or init_weight.ndim != 2:
            raise ValueError("init_weight must be a rank-2 tensor")
        self.base_weight = nn.Parameter(init_weight.detach().clone(), requires_grad=False)
        self.padding_idx = int(padding_idx) if padding_idx is not None else None
        self.bias = nn.Parameter(torch.zeros_like(init_weight)) if add_bias else None

    @torch.no_grad()
    def sync_from(self, weight: torch.Tensor) -> None:
        if _is_sharded_dtensor(weight) or _is_sharded_dtensor(self.base_weight):
            raise RuntimeError("sync_from received a sharded DTensor; gather full parameters first.")
        if weight.shape != self.base_weight.shape:
            raise ValueError(f"sync_from shape mismatch: src={tuple(weight.shape)} dst={tuple(self.base_weight.shape)}")
        if weight.data_ptr() == self.base_weight.data_ptr():
            return  # the engine aliased base_weight onto the generator table: nothing to copy
        self.base_weight.copy_(weight.detach().to(device=self.base_weight.device, dtype=self.base_weight.dtype))

    @property
    def weight(self) -> torch.Tensor:
        """Effective table (base + delta); exported checkpoints store this merged matrix."""
        return self.base_weight if self.bias is None else self.base_weight + self.bias

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        from deberta_b200.ops.embedding import embedding_lookup

        return embedding_lookup(input_ids, self.base_weight, self.bias, self.padding_idx)


class MLMTransform(nn.Module):
    """Dense(hidden→embedding) → act → LayerNorm/RMSNorm (``rtd.py:234-275``)."""

    def __init__(self, config: Any) -> None:
        super().__init__()
        self.hidden_size = int(config.hidden_size)
        self.embedding_size = int(getattr(config, "embedding_size", None) or self.hidden_size)
        self.dense = nn.Linear(self.hidden_size, self.embedding_size)
        self.act = get_act_fn(getattr(config, "hidden_act", "gelu"))
        eps = float(getattr(config, "norm_eps", getattr(config, "layer_norm_eps", 1e-6)))
        self.norm = (RMSNorm(self.embedding_size, eps=eps) if bool(getattr(config, "use_rmsnorm_heads", False))
                     else nn.LayerNorm(self.embedding_size, eps=eps))

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return _norm(self.norm, self.act(linear(hidden_states, self.dense.weight, self.dense.bias)))


class MaskedLMHead(nn.Module):
    """MLM head, tied (``logits = transform(h)·Eᵀ + bias``) or with its own decoder (``rtd.py:278-344``)."""

    def __init__(self, config: Any, *, tie_word_embeddings: bool = True) -> None:
        super().__init__()
        self.transform = MLMTransform(config)
        self.vocab_size = int(config.vocab_size)
        self.tie_word_embeddings = bool(tie_word_embeddings)
        if self.tie_word_embeddings:
            self.decoder = None
            self.bias = nn.Parameter(torch.zeros(self.vocab_size))
        else:
            self.decoder = nn.Linear(self.transform.embedding_size, self.vocab_size, bias=True)
            self.bias = self.decoder.bias

    def projection(self, word_embedding_weight: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:
        """(weight ``[V,E]``, bias ``[V]``) of the vocabulary projection."""
        if not self.tie_word_embeddings:
            return self.decoder.weight, self.decoder.bias
        if word_embedding_weight is None:
            raise RuntimeError("MaskedLMHead requires `word_embedding_weight` when tie_word_embeddings=True.")
        if word_embedding_weight.shape[1] != self.transform.embedding_size:
            raise RuntimeError(
                "Tied word_embedding_weight hidden size mismatch: "
                f"got {word_embedding_weight.shape[1]}, expected {self.transform.embedding_size}."
            )
        return word_embedding_weight, self.bias

    def forward(self, hidden_states: torch.Tensor, *, word_embedding_weight: torch.Tensor | None = None) -> torch.Tensor:
        x = self.transform(hidden_states)
        w, b = self.projection(word_embedding_weight)
        return F.linear(x, w.to(x.dtype), b.to(x.dtype))


class EnhancedMaskDecoder(nn.Module):
    """Enhanced Mask Decoder (``rtd.py:347-544``).

    When the backbone does not add absolute positions to its input, masked-token states
    are refined by running the *last* encoder layer ``num_passes`` times with
    ``query = LN_emb(position_embeddings) + hs[-2]`` and keys/values from ``hs[-2]``.
    A 2-D padding mask stays a compact key mask here: the reference's outer-product
    expansion has identical semantics (dead queries are zeroed either way).
    """

    def __init__(self, config: Any, *, num_last_layer_passes: int = 2) -> None:
        super().__init__()
        self.position_biased_input = bool(getattr(config, "position_biased_input", True))
        self.num_passes = int(num_last_layer_passes)
        if self.num_passes < 1:
            raise ValueError("num_last_layer_passes must be >= 1")

    def forward(self, *, encoder_hidden_states, masked_positions, attention_mask, embeddings, encoder,
                position_ids=None, relative_pos=None, masked_idx=None) -> torch.Tensor:
        hs = list(encoder_hidden_states)
        if len(hs) < 2:
            raise RuntimeError(
                "EnhancedMaskDecoder requires output_hidden_states=True on the generator "
                "so we can access penultimate-layer states."
            )
        if masked_idx is None:  # (data-dependent size: the host waits for the device here)
            masked_idx = torch.nonzero(masked_positions.reshape(-1), as_tuple=False).squeeze(-1)
        if masked_idx.numel() == 0 or self.position_biased_input:
            return gather_rows(hs[-1].reshape(-1, hs[-1].shape[-1]), masked_idx)
        final = self.decode(hs[-2], attention_mask, embeddings, encoder, position_ids, relative_pos)
        return gather_rows(final.reshape(-1, final.shape[-1]), masked_idx)

    def decode(self, kv_states, attention_mask, embeddings, encoder, position_ids=None, relative_pos=None):
        """Full-sequence ``[B,S,H]`` output of the EMD passes."""
        bsz, seq_len, hidden = kv_states.shape
        pos_mod = getattr(embeddings, "position_embeddings", None)
        if pos_mod is None:
            raise RuntimeError("EnhancedMaskDecoder requires embeddings.position_embeddings.")
        pos_w = pos_mod.weight if hasattr(pos_mod, "weight") else None
        if position_ids is None and pos_w is not None:
            z = pos_w[:seq_len].unsqueeze(0)  # same for every row: [1,S,E]
        else:
            if position_ids is None:
                position_ids = torch.arange(seq_len, device=kv_states.device).unsqueeze(0).expand(bsz, -1)
            z = pos_mod(position_ids.to(kv_states.device).long())
        proj = getattr(embeddings, "embed_proj", None)
        if isinstance(proj, nn.Linear):
            z = linear(z, proj.weight)
        if z.shape[-1] != hidden:
            raise RuntimeError(f"Position embedding hidden size mismatch: got {z.shape[-1]}, expected {hidden}.")
        emb_ln = getattr(embeddings, "LayerNorm", None)
        if emb_ln is not None:
            z = _norm(emb_ln, z.to(kv_states.dtype))
        query = z.to(kv_states.dtype) + kv_states
        rel_embeddings = encoder.get_rel_embedding() if hasattr(encoder, "get_rel_embedding") else None
        mask = AttnMask.from_any(attention_mask)
        layers = getattr(encoder, "layer", None)
        if layers is None or len(layers) == 0:
            raise RuntimeError("EnhancedMaskDecoder expects encoder.layer to be a non-empty sequence")
        for _ in range(self.num_passes):
            query, _ = layers[-1](kv_states, mask, query_states=query, relative_pos=relative_pos,
                                  rel_embeddings=rel_embeddings)
        return query


class RTDHead(nn.Module):
    """``logit = w·act(W·Norm(h + h_cls) + b) + c`` (``rtd.py:552-626``).

    The global CLS vector is left out under pairwise (document-block) masks, where adding
    it to every token would leak information across packed documents.
    """

    def __init__(self, config: Any) -> None:
        super().__init__()
        hidden = int(config.hidden_size)
        self.dense = nn.Linear(hidden, hidden)
        self.act_name = str(getattr(config, "hidden_act", "gelu"))
        self.act = get_act_fn(self.act_name)
        eps = float(getattr(config, "norm_eps", getattr(config, "layer_norm_eps", 1e-6)))
        self.norm = (RMSNorm(hidden, eps=eps) if bool(getattr(config, "use_rmsnorm_heads", False))
                     else nn.LayerNorm(hidden, eps=eps))
        self.classifier = nn.Linear(hidden, 1)

    @staticmethod
    def _use_global_cls_context(attention_mask) -> bool:
        if attention_mask is None:
            return True
        if isinstance(attention_mask, AttnMask):
            return not attention_mask.is_pairwise
        m = attention_mask
        if m.ndim == 4:
            m = m[:, 0] if m.shape[1] == 1 else m.any(dim=1)
        return not (m.ndim == 3 and m.shape[-2] != 1)

    def forward(self, hidden_states: torch.Tensor, attention_mask=None) -> torch.Tensor:
        x = hidden_states + hidden_states[:, 0:1, :] if self._use_global_cls_context(attention_mask) else hidden_states
        x = self.act(linear(_norm(self.norm, x), self.dense.weight, self.dense.bias))
        return F.linear(x, self.classifier.weight.to(x.dtype), self.classifier.bias.to(x.dtype)).squeeze(-1)

    def loss_stats(self, hidden_states: torch.Tensor, attention_mask, labels: torch.Tensor, active: torch.Tensor):
        """Head + masked BCE in one go: ``RTDStats`` of ``rtd_loss(self(hidden_states), labels, active)``.

        On bf16 CUDA tensors with a GELU head the dense layer runs with the GELU epilogue and the classifier, the
        loss and the counts come from one kernel; otherwise this is the composition above.
        """
        from deberta_b200.ops.heads import RTDStats
        from deberta_b200.ops.heads_cuda import rtd_head_loss_cuda, rtd_head_supported

        if not rtd_head_supported(hidden_states, self.dense.weight, self.classifier.weight, self.act_name):
            return rtd_loss(self(hidden_states, attention_mask=attention_mask), labels, active)
        x = hidden_states + hidden_states[:, 0:1, :] if self._use_global_cls_context(attention_mask) else hidden_states
        loss, acc, count, positive = rtd_head_loss_cuda(_norm(self.norm, x), self.dense.weight, self.dense.bias,
                                                        self.classifier.weight, self.classifier.bias, labels, active)
        return RTDStats(loss=loss, accuracy=acc, token_count=count, positive_count=positive)


@dataclass
class RTDOutput:
    loss: torch.Tensor
    gen_loss: torch.Tensor
    disc_loss: torch.Tensor
    disc_accuracy: torch.Tensor
    gen_token_count: torch.Tensor
    disc_token_count: torch.Tensor
    disc_positive_count: torch.Tensor
    gen_loss_raw: torch.Tensor
    disc_loss_raw: torch.Tensor


@dataclass
class RTDGeneratorPhaseOutput:
    gen_loss_raw: torch.Tensor
    gen_token_count: torch.Tensor
    corrupted_input_ids: torch.Tensor
    disc_labels: torch.Tensor
    has_masked_targets: bool


@dataclass
class RTDDiscriminatorPhaseOutput:
    disc_loss_raw: torch.Tensor
    disc_accuracy: torch.Tensor
    disc_token_count: torch.Tensor
    disc_positive_count: torch.Tensor


class DebertaV3RTDPretrainer(nn.Module):
    """Generator (MLM) + discriminator (RTD) with ES/GDES embedding sharing (``rtd.py:675-1256``)."""

    _SPECIAL_ID_ATTRS = ("pad_token_id", "cls_token_id", "sep_token_id", "mask_token_id", "unk_token_id",
                         "bos_token_id", "eos_token_id")

    def __init__(self, *, discriminator_backbone: nn.Module, generator_backbone: nn.Module, disc_config: Any,
                 gen_config: Any, embedding_sharing: str = "gdes", tie_generator_word_embeddings: bool = True,
                 use_enhanced_mask_decoder: bool = True,
                 additional_forbidden_token_ids: Iterable[int] | None = None) -> None:
        super().__init__()
        self.disc_config, self.gen_config = disc_config, gen_config
        self.generator, self.discriminator = generator_backbone, discriminator_backbone
        self.generator_lm_head = MaskedLMHead(gen_config, tie_word_embeddings=tie_generator_word_embeddings)
        self.use_enhanced_mask_decoder = bool(use_enhanced_mask_decoder)
        self.enhanced_mask_decoder = EnhancedMaskDecoder(gen_config, num_last_layer_passes=2)
        self.discriminator_head = RTDHead(disc_config)
        self.embedding_sharing = str(embedding_sharing or "none")
        self._forbidden_sample_token_ids = self._collect_forbidden_sample_token_ids(additional_forbidden_token_ids)
        vocab = int(getattr(gen_config, "vocab_size", 0) or 0)
        self.register_buffer(
            "_forbidden_sample_token_mask",
            self._build_forbidden_token_mask(vocab_size=vocab, forbidden_ids=self._forbidden_sample_token_ids),
            persistent=False,
        )
        self._gdes_synced_embeddings: list[tuple[str, _SyncedBufferEmbedding, nn.Module]] = []
        self._patch_discriminator_embeddings_for_sharing()

    # ---- sampling exclusions -------------------------------------------------------------
    @staticmethod
    def _build_forbidden_token_mask(*, vocab_size: int, forbidden_ids: set[int]) -> torch.Tensor:
        if vocab_size <= 0:
            return torch.empty(0, dtype=torch.bool)
        mask = torch.zeros(vocab_size, dtype=torch.bool)
        valid = [int(t) for t in forbidden_ids if 0 <= int(t) < vocab_size]
        if valid:
            mask[valid] = True
        if bool(mask.all()):
            raise ValueError(
                "forbidden token mask excludes all vocabulary ids; at least one token must remain sampleable."
            )
        return mask

    def _collect_forbidden_sample_token_ids(self, additional: Iterable[int] | None) -> set[int]:
        vocab = int(getattr(self.gen_config, "vocab_size", 0) or 0)
        if vocab <= 0:
            return set()
        cands: list[Any] = [getattr(cfg, a, None) for cfg in (self.gen_config, self.disc_config)
                            for a in self._SPECIAL_ID_ATTRS]
        if additional is not None:
            cands.extend(additional)
        out: set[int] = set()
        for sid in cands:
            try:
                i = int(sid)
            except (TypeError, ValueError):
                continue
            if 0 <= i < vocab:
                out.add(i)
        return out

    # ---- embedding sharing ------------------------------------------------------------------
    def _patch_discriminator_embeddings_for_sharing(self) -> None:
        mode = (self.embedding_sharing or "none").lower()
        if mode not in {"none", "es", "gdes"}:
            raise ValueError("embedding_sharing must be one of: none|es|gdes")
        if mode == "none":
            return
        try:
            gen_emb, disc_emb = self.generator.embeddings, self.discriminator.embeddings
        except AttributeError as e:
            raise RuntimeError("Expected backbones with an `.embeddings` module containing word_embeddings.") from e
        for attr in ("word_embeddings", "position_embeddings", "token_type_embeddings"):
            g, d = getattr(gen_emb, attr, None), getattr(disc_emb, attr, None)
            if g is None or d is None:
                continue
            gw, dw = getattr(g, "weight", None), getattr(d, "weight", None)
            if not isinstance(gw, torch.Tensor) or not isinstance(dw, torch.Tensor):
                raise RuntimeError("Embedding module must expose .weight tensor")
            if gw.shape != dw.shape:
                raise ValueError(
                    f"Cannot share embeddings for '{attr}': generator shape {tuple(gw.shape)} != "
                    f"discriminator shape {tuple(dw.shape)}."
                )
            if mode == "es":
                d.weight = gw  # one Parameter object used by both branches
                continue
            pad = getattr(d, "padding_idx", None)
            synced = _SyncedBufferEmbedding(init_weight=gw, padding_idx=pad, add_bias=True)
            setattr(disc_emb, attr, synced)
            self._gdes_synced_embeddings.append((attr, synced, g))

    @torch.no_grad()
    def sync_discriminator_embeddings_from_generator(self) -> None:
        """Refresh every GDES ``base_weight`` from the generator table (after generator steps / loads)."""
        if (self.embedding_sharing or "none").lower() != "gdes":
            return
        for attr, disc_mod, gen_mod in self._gdes_synced_embeddings:
            w = getattr(gen_mod, "weight", None)
            if not isinstance(w, torch.Tensor):
                raise RuntimeError(f"Generator embedding '{attr}' no longer exposes .weight")
            disc_mod.sync_from(w)

    def _get_generator_word_embedding_weight(self) -> torch.Tensor:
        emb = getattr(self.generator, "embeddings", None)
        word = getattr(emb, "word_embeddings", None) if emb is not None else None
        w = getattr(word, "weight", None)
        if not isinstance(w, torch.Tensor):
            raise RuntimeError("Generator word_embeddings must expose a `.weight` tensor for LM-head tying.")
        return w

    _gumbel_sample = staticmethod(gumbel_sample)

    # ---- forward phases ------------------------------------------------------------------------
    def _uses_emd(self) -> bool:
        pos_biased = bool(getattr(self.gen_config, "position_biased_input", True))
        z_steps = int(getattr(self.generator, "z_steps", getattr(self.gen_config, "z_steps", 0)) or 0)
        return self.use_enhanced_mask_decoder and (not pos_biased) and z_steps <= 1

    def forward_generator_phase(self, *, input_ids, attention_mask=None, labels, token_type_ids=None,
                                sampling_temperature: float = 1.0, masked_idx=None) -> RTDGeneratorPhaseOutput:
        """Generator MLM loss on masked rows + sampled corruption for the discriminator (``:988-1093``).

        ``masked_idx`` (optional): the flat positions where ``labels != -100``, already on the device. The training
        loop computes them on the host copy of the batch, so that the forward never has to wait for the device to
        learn how many rows are masked; without it they come from ``torch.nonzero`` (one host-device round trip)."""
        if labels is None:
            raise ValueError("labels must be provided (MLM labels with -100 for unmasked positions)")
        masked_positions = labels.ne(-100)
        masked_flat = masked_positions.view(-1)
        if masked_idx is None:
            masked_idx = torch.nonzero(masked_flat, as_tuple=False).squeeze(-1)
        gen_token_count = masked_flat.sum().to(torch.float32)
        use_emd = self._uses_emd()
        kw: dict[str, Any] = {"input_ids": input_ids, "attention_mask": attention_mask,
                              "token_type_ids": token_type_ids, "return_dict": True}
        if use_emd:
            kw["output_hidden_states"] = True
        gen_out = self.generator(**kw)
        if masked_idx.numel() == 0:
            return RTDGeneratorPhaseOutput(
                gen_loss_raw=gen_out.last_hidden_state.sum() * 0.0, gen_token_count=gen_token_count.detach(),
                corrupted_input_ids=input_ids.detach(),
                disc_labels=torch.zeros_like(input_ids, dtype=torch.float32), has_masked_targets=False,
            )
        if use_emd:
            hidden = self.enhanced_mask_decoder(
                encoder_hidden_states=gen_out.hidden_states, masked_positions=masked_positions,
                attention_mask=attention_mask, embeddings=self.generator.embeddings, encoder=self.generator.encoder,
                masked_idx=masked_idx,
            )
        else:
            last = gen_out.last_hidden_state
            hidden = gather_rows(last.reshape(-1, last.shape[-1]), masked_idx)
        masked_labels = labels.view(-1).index_select(0, masked_idx)
        head = self.generator_lm_head
        w, b = head.projection(self._get_generator_word_embedding_weight() if head.tie_word_embeddings else None)
        gen_loss, sampled = mlm_loss_and_sample(
            head.transform(hidden), w, b, masked_labels, getattr(self, "_forbidden_sample_token_mask", None),
            float(sampling_temperature),
        )
        with torch.no_grad():
            sampled = sampled.to(input_ids.dtype)
            corrupted = input_ids.view(-1).scatter(0, masked_idx, sampled).view_as(input_ids)
            replaced = sampled.ne(masked_labels.to(sampled.dtype)).to(torch.float32)
            disc_labels = torch.zeros(input_ids.numel(), dtype=torch.float32, device=input_ids.device)
            disc_labels = disc_labels.scatter_(0, masked_idx, replaced).view_as(input_ids)
        return RTDGeneratorPhaseOutput(
            gen_loss_raw=gen_loss, gen_token_count=gen_token_count.detach(), corrupted_input_ids=corrupted.detach(),
            disc_labels=disc_labels.detach(), has_masked_targets=True,
        )

    def forward_discriminator_phase(self, *, input_ids, corrupted_input_ids, disc_labels, attention_mask=None,
                                    token_type_ids=None) -> RTDDiscriminatorPhaseOutput:
        """Discriminator pass over the corrupted ids + masked-mean BCE over active tokens (``:1095-1152``)."""
        out = self.discriminator(input_ids=corrupted_input_ids, attention_mask=attention_mask,
                                 token_type_ids=token_type_ids, return_dict=True)
        pad = getattr(self.disc_config, "pad_token_id", None)
        active = attention_mask_to_active_tokens(input_ids=input_ids, attention_mask=attention_mask,
                                                 pad_token_id=int(pad) if pad is not None else None)
        st = self.discriminator_head.loss_stats(out.last_hidden_state, attention_mask, disc_labels, active)
        return RTDDiscriminatorPhaseOutput(disc_loss_raw=st.loss, disc_accuracy=st.accuracy,
                                           disc_token_count=st.token_count, disc_positive_count=st.positive_count)

    def forward(self, *, input_ids, attention_mask=None, labels=None, token_type_ids=None,
                sampling_temperature: float = 1.0, gen_loss_weight: float = 1.0, disc_loss_weight: float = 50.0,
                phase: str = "both", corrupted_input_ids=None, disc_labels=None, masked_idx=None):
        """``phase='generator' | 'discriminator'`` run one branch; ``'both'`` returns the weighted ``RTDOutput``."""
        phase = str(phase or "both").strip().lower()
        if phase == "generator":
            if labels is None:
                raise ValueError("labels must be provided for phase='generator'.")
            return self.forward_generator_phase(input_ids=input_ids, attention_mask=attention_mask, labels=labels,
                                                token_type_ids=token_type_ids,
                                                sampling_temperature=sampling_temperature, masked_idx=masked_idx)
        if phase == "discriminator":
            if corrupted_input_ids is None:
                raise ValueError("corrupted_input_ids must be provided for phase='discriminator'.")
            if disc_labels is None:
                raise ValueError("disc_labels must be provided for phase='discriminator'.")
            return self.forward_discriminator_phase(input_ids=input_ids, corrupted_input_ids=corrupted_input_ids,
                                                    disc_labels=disc_labels, attention_mask=attention_mask,
                                                    token_type_ids=token_type_ids)
        if phase != "both":
            raise ValueError("phase must be one of: both|generator|discriminator.")
        if labels is None:
            raise ValueError("labels must be provided for phase='both'.")
        g = self.forward_generator_phase(input_ids=input_ids, attention_mask=attention_mask, labels=labels,
                                         token_type_ids=token_type_ids, sampling_temperature=sampling_temperature,
                                         masked_idx=masked_idx)
        if not g.has_masked_targets:
            zero = torch.zeros((), device=input_ids.device, dtype=torch.float32)
            return RTDOutput(loss=float(gen_loss_weight) * g.gen_loss_raw, gen_loss=g.gen_loss_raw.detach(),
                             disc_loss=zero, disc_accuracy=zero, gen_token_count=g.gen_token_count.detach(),
                             disc_token_count=zero, disc_positive_count=zero, gen_loss_raw=g.gen_loss_raw,
                             disc_loss_raw=zero)
        d = self.forward_discriminator_phase(input_ids=input_ids, corrupted_input_ids=g.corrupted_input_ids,
                                             disc_labels=g.disc_labels, attention_mask=attention_mask,
                                             token_type_ids=token_type_ids)
        total = float(gen_loss_weight) * g.gen_loss_raw + float(disc_loss_weight) * d.disc_loss_raw
        return RTDOutput(loss=total, gen_loss=g.gen_loss_raw.detach(), disc_loss=d.disc_loss_raw.detach(),
                         disc_accuracy=d.disc_accuracy.detach(), gen_token_count=g.gen_token_count.detach(),
                         disc_token_count=d.disc_token_count.detach(),
                         disc_positive_count=d.disc_positive_count.detach(), gen_loss_raw=g.gen_loss_raw,
                         disc_loss_raw=d.disc_loss_raw)
