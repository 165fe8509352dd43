"""DeBERTa-v2/v3 encoder backbone (disentangled attention, post-LN blocks).

Parameter names equal Hugging Face ``DebertaV2Model`` (and the reference's
``deberta_v2_native.py``), so checkpoints and exports interchange. The forward pass is
written against the operator layer (``deberta_b200.ops``): one fused attention
operator per layer that takes a compact mask instead of a dense S×S tensor, GEMMs with
bias/residual/GELU epilogues, and fp32-statistics LayerNorm. On CPU those operators are
plain PyTorch, on a B200 they are the sm_100a kernels.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn.functional as F
from torch import nn
from transformers import DebertaV2Config, PreTrainedModel
from transformers.modeling_outputs import BaseModelOutput

from deberta_b200.ops.attention import disentangled_attention
from deberta_b200.ops.linear import ResidualGradSink, ffn_gelu, linear, linear_qkv
from deberta_b200.ops.norm import layer_norm

from .activations import get_act_fn
from .mask_utils import AttnMask

__all__ = [
    "DebertaV2Config",
    "DebertaV2Model",
    "DebertaV2Embeddings",
    "DebertaV2Encoder",
    "DebertaV2Layer",
    "DisentangledSelfAttention",
]

_HF_ATTN_KERNELS = {"dynamic", "cached_bmm", "stable"}


def normalize_pos_att_type(raw: Any) -> list[str]:
    """``"p2c|c2p"`` / ``["p2c", "c2p"]`` / ``None`` → lower-case list of position-attention terms."""
    if raw is None:
        return []
    chunks = raw.replace(",", "|").split("|") if isinstance(raw, str) else [str(x) for x in raw]
    return [c.strip().lower() for c in chunks if c and c.strip()]


def _ln(mod: nn.LayerNorm, x: torch.Tensor, row_keep: torch.Tensor | None = None) -> torch.Tensor:
    return layer_norm(x, mod.weight, mod.bias, mod.eps, row_keep)


def _drop(x: torch.Tensor, p: float, training: bool) -> torch.Tensor:
    return F.dropout(x, p, True) if (training and p > 0.0) else x



def _embed(module: nn.Module, input_ids: torch.Tensor) -> torch.Tensor:
    """Word-embedding lookup: plain ``nn.Embedding`` tables go through the gather kernel, wrapped ones keep their forward."""
    if type(module) is nn.Embedding and module.max_norm is None and not module.sparse:
        from deberta_b200.ops.embedding import embedding_lookup

        return embedding_lookup(input_ids, module.weight, None, module.padding_idx)
    return module(input_ids)

class DisentangledSelfAttention(nn.Module):
    """Content/position attention of DeBERTa (``deberta_v2_native.py:168-652``).

    The three "attention kernel" names the reference accepts (``dynamic``, ``cached_bmm``,
    ``stable``) are numerically equivalent formulations there; here all of them select
    the same fused operator.
    """

    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        hidden, heads = int(config.hidden_size), int(config.num_attention_heads)
        if hidden % heads:
            raise ValueError(f"hidden_size ({hidden}) must be divisible by num_attention_heads ({heads}).")
        self.num_attention_heads = heads
        self.attention_head_size = int(getattr(config, "attention_head_size", hidden // heads))
        self.all_head_size = heads * self.attention_head_size
        self.query_proj = nn.Linear(hidden, self.all_head_size)
        self.key_proj = nn.Linear(hidden, self.all_head_size)
        self.value_proj = nn.Linear(hidden, self.all_head_size)
        self.share_att_key = bool(getattr(config, "share_att_key", False))
        self.pos_att_type = normalize_pos_att_type(getattr(config, "pos_att_type", None))
        self.relative_attention = bool(getattr(config, "relative_attention", False))
        self.position_buckets = int(getattr(config, "position_buckets", -1))
        self.max_relative_positions = int(getattr(config, "max_relative_positions", -1))
        if self.max_relative_positions < 1:
            self.max_relative_positions = int(config.max_position_embeddings)
        self.pos_ebd_size = self.position_buckets if self.position_buckets > 0 else self.max_relative_positions
        self.pos_dropout_p = float(config.hidden_dropout_prob)
        self.attn_dropout_p = float(config.attention_probs_dropout_prob)
        kernel = str(getattr(config, "hf_attention_kernel", "dynamic")).strip().lower()
        if kernel not in _HF_ATTN_KERNELS:
            raise ValueError(f"hf_attention_kernel must be one of {sorted(_HF_ATTN_KERNELS)}, got {kernel!r}")
        self.attn_kernel = kernel
        self.pos_key_proj = self.pos_query_proj = None
        if self.relative_attention and not self.share_att_key:
            if "c2p" in self.pos_att_type or "p2p" in self.pos_att_type:
                self.pos_key_proj = nn.Linear(hidden, self.all_head_size)
            if "p2c" in self.pos_att_type or "p2p" in self.pos_att_type:
                self.pos_query_proj = nn.Linear(hidden, self.all_head_size)

    @property
    def scale_factor(self) -> int:
        return 1 + sum(t in self.pos_att_type for t in ("c2p", "p2c", "p2p"))

    def project_positions(self, rel_embeddings: torch.Tensor, *, use_query: bool) -> torch.Tensor:
        """``[2·span, H]`` projection of the relative-embedding table with the key/query weights."""
        # (a slice of the whole table is still an autograd node: its backward would zero-fill and copy a full table per layer)
        rows = 2 * self.pos_ebd_size
        rel = rel_embeddings if rel_embeddings.shape[0] == rows else rel_embeddings[:rows]
        proj = (self.query_proj if self.share_att_key else self.pos_query_proj) if use_query else (
            self.key_proj if self.share_att_key else self.pos_key_proj
        )
        if proj is None:
            raise RuntimeError("Requested relative projection is not configured for this attention module.")
        return linear(rel, proj.weight, proj.bias)

    def forward(
        self,
        hidden_states: torch.Tensor,
        mask: AttnMask,
        query_states: torch.Tensor | None = None,
        relative_pos: torch.Tensor | None = None,
        rel_embeddings: torch.Tensor | None = None,
        residual_sink=None,
    ) -> torch.Tensor:
        if query_states is None:
            q, k, v = linear_qkv(hidden_states, self.query_proj.weight, self.query_proj.bias, self.key_proj.weight,
                                 self.key_proj.bias, self.value_proj.weight, self.value_proj.bias,
                                 residual_sink=residual_sink)
        else:
            q = linear(query_states, self.query_proj.weight, self.query_proj.bias)
            k = linear(hidden_states, self.key_proj.weight, self.key_proj.bias)
            v = linear(hidden_states, self.value_proj.weight, self.value_proj.bias)
        pos_k = pos_q = None
        if self.relative_attention and rel_embeddings is not None:
            rel = _drop(rel_embeddings, self.pos_dropout_p, self.training)
            if "c2p" in self.pos_att_type or "p2p" in self.pos_att_type:
                pos_k = self.project_positions(rel, use_query=False)
            if "p2c" in self.pos_att_type or "p2p" in self.pos_att_type:
                pos_q = self.project_positions(rel, use_query=True)
        if "p2p" in self.pos_att_type:
            return self._forward_with_p2p(q, k, v, pos_k, pos_q, mask, relative_pos)
        return disentangled_attention(
            q, k, v,
            pos_k if "c2p" in self.pos_att_type else None,
            pos_q if "p2c" in self.pos_att_type else None,
            heads=self.num_attention_heads, scale_factor=self.scale_factor, bucket_size=self.position_buckets,
            max_position=self.max_relative_positions, att_span=self.pos_ebd_size,
            dropout_p=self.attn_dropout_p, training=self.training, rel_pos=relative_pos, **mask.kwargs(),
        )

    def _forward_with_p2p(self, q, k, v, pos_k, pos_q, mask: AttnMask, relative_pos):
        """Position→position term (not used by any preset; PyTorch path only, ``:298-347``)."""
        import math

        from deberta_b200.ops.attention import dense_keep_mask, relative_positions

        h, d, span = self.num_attention_heads, self.attention_head_size, self.pos_ebd_size
        B, Sq, _ = q.shape
        Sk = k.shape[1]
        rel = relative_pos if relative_pos is not None else relative_positions(
            Sq, Sk, self.position_buckets, self.max_relative_positions, device=q.device)
        rel = rel.clamp(-span, span)
        scale = math.sqrt(float(d * self.scale_factor))
        split = lambda x: x.view(x.shape[0], x.shape[1], h, d).permute(0, 2, 1, 3).float()  # noqa: E731
        qf, kf, vf = split(q), split(k), split(v)
        scores = torch.matmul(qf, kf.transpose(-1, -2)) / scale
        pk = pos_k.view(2 * span, h, d).permute(1, 0, 2).float()
        pq = pos_q.view(2 * span, h, d).permute(1, 0, 2).float()
        idx = (rel + span).clamp(0, 2 * span - 1)
        if "c2p" in self.pos_att_type:
            c2p = torch.einsum("bhqd,hpd->bhqp", qf, pk)
            scores = scores + c2p.gather(-1, idx[None, None].expand(B, h, Sq, Sk)) / scale
        if "p2c" in self.pos_att_type:
            p2c = torch.einsum("bhkd,hpd->bhkp", kf, pq)
            idx_t = (span - rel.transpose(0, 1)).clamp(0, 2 * span - 1)
            scores = scores + p2c.gather(-1, idx_t[None, None].expand(B, h, Sk, Sq)).transpose(-1, -2) / scale
        table = torch.einsum("hqd,hkd->hqk", pq[:, span:], pk)  # positive half of the query table
        rows = torch.arange(Sq, device=q.device).clamp(max=table.shape[1] - 1)
        p2p = table.index_select(1, rows).gather(-1, idx[None].expand(h, Sq, Sk)) / scale
        scores = scores + p2p[None]
        keep, live = dense_keep_mask(**mask.kwargs())
        if keep is not None:
            scores = scores.masked_fill(~keep, torch.finfo(scores.dtype).min)
            scores = torch.where(live, scores, torch.zeros_like(scores))
        probs = _drop(torch.softmax(scores, dim=-1), self.attn_dropout_p, self.training)
        if keep is not None:
            probs = probs * live.to(probs.dtype)
        ctx = torch.matmul(probs, vf)
        return ctx.permute(0, 2, 1, 3).reshape(B, Sq, h * d).to(q.dtype)


class DebertaV2SelfOutput(nn.Module):
    """Attention output projection + residual LayerNorm (parameters only; the layer runs the math)."""

    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        self.dense = nn.Linear(int(config.hidden_size), int(config.hidden_size))
        self.LayerNorm = nn.LayerNorm(int(config.hidden_size), eps=float(config.layer_norm_eps))
        self.dropout_p = float(config.hidden_dropout_prob)

    def forward(self, hidden_states: torch.Tensor, input_tensor: torch.Tensor, residual_sink=None) -> torch.Tensor:
        if self.training and self.dropout_p > 0.0:
            x = _drop(linear(hidden_states, self.dense.weight, self.dense.bias), self.dropout_p, True) + input_tensor
        else:
            x = linear(hidden_states, self.dense.weight, self.dense.bias, residual=input_tensor,
                       residual_sink=residual_sink)
        return _ln(self.LayerNorm, x)


class DebertaV2Attention(nn.Module):
    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        self.self = DisentangledSelfAttention(config)
        self.output = DebertaV2SelfOutput(config)

    def forward(self, hidden_states, mask: AttnMask, query_states=None, relative_pos=None, rel_embeddings=None):
        if query_states is not None:
            ctx = self.self(hidden_states, mask, query_states=query_states, relative_pos=relative_pos,
                            rel_embeddings=rel_embeddings)
            return self.output(ctx, query_states)
        # x feeds the QKV projection and the block's residual: the residual's gradient rides into the QKV projection's
        # data-gradient GEMM instead of meeting it in a separate add (ops/linear.py::ResidualGradSink)
        sink = ResidualGradSink()
        ctx = self.self(hidden_states, mask, relative_pos=relative_pos, rel_embeddings=rel_embeddings, residual_sink=sink)
        return self.output(ctx, hidden_states, residual_sink=sink)


class DebertaV2Intermediate(nn.Module):
    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        self.dense = nn.Linear(int(config.hidden_size), int(config.intermediate_size))
        self.act_name = config.hidden_act if isinstance(config.hidden_act, str) else None
        self.intermediate_act_fn = get_act_fn(config.hidden_act)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.intermediate_act_fn(linear(hidden_states, self.dense.weight, self.dense.bias))


class DebertaV2Output(nn.Module):
    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        self.dense = nn.Linear(int(config.intermediate_size), int(config.hidden_size))
        self.LayerNorm = nn.LayerNorm(int(config.hidden_size), eps=float(config.layer_norm_eps))
        self.dropout_p = float(config.hidden_dropout_prob)

    def forward(self, hidden_states: torch.Tensor, input_tensor: torch.Tensor) -> torch.Tensor:
        x = _drop(linear(hidden_states, self.dense.weight, self.dense.bias), self.dropout_p, self.training)
        return _ln(self.LayerNorm, x + input_tensor)


class DebertaV2Layer(nn.Module):
    """One post-LN block: ``a = LN(Wo·attn + x_q)``, ``y = LN(W2·gelu(W1·a) + a)`` (``:774-807``)."""

    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        self.attention = DebertaV2Attention(config)
        self.intermediate = DebertaV2Intermediate(config)
        self.output = DebertaV2Output(config)
        self.call_ffn_modules = False

    def forward(
        self,
        hidden_states: torch.Tensor,
        attention_mask: AttnMask | torch.Tensor | None,
        query_states: torch.Tensor | None = None,
        relative_pos: torch.Tensor | None = None,
        rel_embeddings: torch.Tensor | None = None,
        output_attentions: bool = False,
    ) -> tuple[torch.Tensor, None]:
        mask = AttnMask.from_any(attention_mask)
        a = self.attention(hidden_states, mask, query_states=query_states, relative_pos=relative_pos,
                           rel_embeddings=rel_embeddings)
        inter, out = self.intermediate, self.output
        # (a layer whose FFN modules were compiled one by one, ``train.compile.scope: ffn``, has to call them)
        fused = inter.act_name == "gelu" and not (self.training and out.dropout_p > 0.0) and not self.call_ffn_modules
        if fused:
            y = ffn_gelu(a, inter.dense.weight, inter.dense.bias, out.dense.weight, out.dense.bias, residual=a)
            y = _ln(out.LayerNorm, y)
        else:
            y = out(inter(a), a)
        return y, None


class ConvLayer(nn.Module):
    """Optional Conv1d refinement after layer 0 (only when ``conv_kernel_size > 0``; ``:810-860``)."""

    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        hidden = int(config.hidden_size)
        ks = int(getattr(config, "conv_kernel_size", 3))
        self.conv_act = str(getattr(config, "conv_act", "tanh"))
        self.conv = nn.Conv1d(hidden, hidden, ks, padding=(ks - 1) // 2, groups=int(getattr(config, "conv_groups", 1)))
        self.LayerNorm = nn.LayerNorm(hidden, eps=float(config.layer_norm_eps))
        self.dropout_p = float(config.hidden_dropout_prob)

    def forward(self, hidden_states, residual_states, token_keep: torch.Tensor | None):
        out = self.conv(hidden_states.transpose(1, 2).contiguous()).transpose(1, 2).contiguous()
        if token_keep is not None:
            out = out.masked_fill(~token_keep.unsqueeze(-1), 0)
        out = get_act_fn(self.conv_act)(_drop(out, self.dropout_p, self.training))
        y = _ln(self.LayerNorm, residual_states + out)
        return y if token_keep is None else y * token_keep.to(y.dtype).unsqueeze(-1)


class DebertaV2Embeddings(nn.Module):
    """``LN(word [+pos] [+type] [·embed_proj]) · keep`` (``:863-995``).

    ``position_embeddings`` always exists because the Enhanced Mask Decoder reads it, but
    it is only added to the input when ``position_biased_input`` is set.
    """

    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        pad = int(getattr(config, "pad_token_id", 0) or 0)
        self.embedding_size = int(getattr(config, "embedding_size", None) or config.hidden_size)
        self.word_embeddings = nn.Embedding(int(config.vocab_size), self.embedding_size, padding_idx=pad)
        self.position_biased_input = bool(getattr(config, "position_biased_input", True))
        self.position_embeddings = nn.Embedding(int(config.max_position_embeddings), self.embedding_size)
        self.token_type_embeddings = (
            nn.Embedding(int(config.type_vocab_size), self.embedding_size) if int(config.type_vocab_size) > 0 else None
        )
        self.embed_proj = (
            nn.Linear(self.embedding_size, int(config.hidden_size), bias=False)
            if self.embedding_size != int(config.hidden_size) else None
        )
        self.LayerNorm = nn.LayerNorm(int(config.hidden_size), eps=float(config.layer_norm_eps))
        self.dropout_p = float(config.hidden_dropout_prob)
        self.register_buffer(
            "position_ids", torch.arange(int(config.max_position_embeddings)).unsqueeze(0), persistent=False
        )

    def forward(self, input_ids=None, token_type_ids=None, position_ids=None, mask=None, inputs_embeds=None):
        if input_ids is None and inputs_embeds is None:
            raise ValueError("Either input_ids or inputs_embeds must be provided.")
        shape = input_ids.shape if input_ids is not None else inputs_embeds.shape[:-1]
        device = input_ids.device if input_ids is not None else inputs_embeds.device
        seq_len = int(shape[1])
        x = _embed(self.word_embeddings, input_ids) if inputs_embeds is None else inputs_embeds
        if self.position_biased_input:
            pos = self.position_ids[:, :seq_len].to(device) if position_ids is None else position_ids.to(device)
            x = x + self.position_embeddings(pos.long())
        if self.token_type_embeddings is not None:
            if token_type_ids is None:
                token_type_ids = torch.zeros(shape, dtype=torch.long, device=device)
            x = x + self.token_type_embeddings(token_type_ids.long())
        if self.embed_proj is not None:
            x = linear(x, self.embed_proj.weight)
        keep = AttnMask.from_any(mask).token_keep() if mask is not None else None
        x = _ln(self.LayerNorm, x, None if keep is None else keep[:, :seq_len])
        return _drop(x, self.dropout_p, self.training)


class DebertaV2Encoder(nn.Module):
    """Layer stack + shared relative-embedding table (``:998-1227``)."""

    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__()
        self.layer = nn.ModuleList([DebertaV2Layer(config) for _ in range(int(config.num_hidden_layers))])
        self.relative_attention = bool(getattr(config, "relative_attention", False))
        self.max_relative_positions = int(getattr(config, "max_relative_positions", -1))
        if self.max_relative_positions < 1:
            self.max_relative_positions = int(config.max_position_embeddings)
        self.position_buckets = int(getattr(config, "position_buckets", -1))
        if self.relative_attention:
            span = self.position_buckets if self.position_buckets > 0 else self.max_relative_positions
            self.rel_embeddings = nn.Embedding(2 * span, int(config.hidden_size))
        else:
            self.rel_embeddings = None
        self.norm_rel_ebd = [x.strip() for x in str(getattr(config, "norm_rel_ebd", "none")).lower().split("|")]
        self.LayerNorm = (
            nn.LayerNorm(int(config.hidden_size), eps=float(config.layer_norm_eps))
            if "layer_norm" in self.norm_rel_ebd else None
        )
        ks = getattr(config, "conv_kernel_size", 0)
        self.conv = ConvLayer(config) if ks and int(ks) > 0 else None
        self.gradient_checkpointing = False

    def get_rel_embedding(self) -> torch.Tensor | None:
        if self.rel_embeddings is None:
            return None
        w = self.rel_embeddings.weight
        return _ln(self.LayerNorm, w) if self.LayerNorm is not None else w

    def get_attention_mask(self, attention_mask) -> AttnMask:
        return AttnMask.from_any(attention_mask)

    def get_rel_pos(self, hidden_states, query_states=None, relative_pos=None):
        """Explicit relative-position ids if the caller supplied them.

        The attention operator derives the log-bucket ids from (query_len, key_len) itself,
        so nothing is materialised per forward when ``relative_pos`` is ``None``.
        """
        return relative_pos if self.relative_attention else None

    def forward(
        self,
        hidden_states: torch.Tensor,
        attention_mask,
        output_hidden_states: bool = True,
        output_attentions: bool = False,
        query_states: torch.Tensor | None = None,
        relative_pos: torch.Tensor | None = None,
        return_dict: bool = True,
    ):
        mask = AttnMask.from_any(attention_mask)
        rel_embeddings = self.get_rel_embedding()
        all_hidden = (hidden_states,) if output_hidden_states else None
        next_kv = out = hidden_states
        for idx, layer in enumerate(self.layer):
            if self.gradient_checkpointing and self.training and query_states is None:
                out = torch.utils.checkpoint.checkpoint(
                    lambda hs, re, layer=layer: layer(hs, mask, relative_pos=relative_pos, rel_embeddings=re)[0],
                    next_kv, rel_embeddings, use_reentrant=False,
                )
            else:
                out, _ = layer(next_kv, mask, query_states=query_states, relative_pos=relative_pos,
                               rel_embeddings=rel_embeddings)
            if idx == 0 and self.conv is not None:
                out = self.conv(hidden_states, out, mask.token_keep())
            if output_hidden_states:
                all_hidden = all_hidden + (out,)
            if query_states is not None:
                query_states = out
            next_kv = out
        attn = () if output_attentions else None
        if not return_dict:
            return tuple(v for v in (out, all_hidden, attn) if v is not None)
        return BaseModelOutput(last_hidden_state=out, hidden_states=all_hidden, attentions=attn)


class DebertaV2PreTrainedModel(PreTrainedModel):
    config_class = DebertaV2Config
    base_model_prefix = "deberta"
    supports_gradient_checkpointing = True

    def _init_weights(self, module: nn.Module) -> None:
        """N(0, initializer_range) for matrices, zero biases and pad row, unit LayerNorm."""
        from ._hf_init import init_embedding_, init_linear_, init_norm_

        std = float(self.config.initializer_range)
        if isinstance(module, nn.Linear):
            init_linear_(module, std)
        elif isinstance(module, nn.Embedding):
            init_embedding_(module, std)
        elif isinstance(module, nn.LayerNorm):
            init_norm_(module.weight, module.bias)
        elif isinstance(module, DebertaV2Embeddings):
            # non-persistent buffer: absent from checkpoints, so it is rewritten after a load from the meta device
            module.position_ids.data.copy_(torch.arange(module.position_ids.shape[-1]).unsqueeze(0))

    def _set_gradient_checkpointing(self, module: nn.Module = None, value: bool = False, **_: Any) -> None:
        for m in self.modules():
            if isinstance(m, DebertaV2Encoder):
                m.gradient_checkpointing = bool(value)

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None) -> None:
        self._set_gradient_checkpointing(value=True)

    def gradient_checkpointing_disable(self) -> None:
        self._set_gradient_checkpointing(value=False)


class DebertaV2Model(DebertaV2PreTrainedModel):
    """Encoder-only DeBERTa-v2 returning ``BaseModelOutput`` (``:1266-1428``)."""

    def __init__(self, config: DebertaV2Config) -> None:
        super().__init__(config)
        self.embeddings = DebertaV2Embeddings(config)
        self.encoder = DebertaV2Encoder(config)
        self.z_steps = int(getattr(config, "z_steps", 0) or 0)
        self.post_init()

    def get_input_embeddings(self) -> nn.Module:
        return self.embeddings.word_embeddings

    def set_input_embeddings(self, new_embeddings: nn.Module) -> None:
        self.embeddings.word_embeddings = new_embeddings

    def forward(
        self,
        input_ids: torch.Tensor | None = None,
        attention_mask: torch.Tensor | None = None,
        token_type_ids: torch.Tensor | None = None,
        position_ids: torch.Tensor | None = None,
        inputs_embeds: torch.Tensor | None = None,
        output_attentions: bool | None = None,
        output_hidden_states: bool | None = None,
        return_dict: bool | None = None,
    ):
        if output_attentions:
            raise ValueError("output_attentions is not supported: attention probabilities are never materialised.")
        output_hidden_states = bool(
            getattr(self.config, "output_hidden_states", False) if output_hidden_states is None else output_hidden_states
        )
        return_dict = bool(getattr(self.config, "return_dict", True) if return_dict is None else return_dict)
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("Specify exactly one of input_ids or inputs_embeds.")
        mask = AttnMask.from_any(attention_mask)
        emb = self.embeddings(input_ids=input_ids, token_type_ids=token_type_ids, position_ids=position_ids,
                              mask=mask if attention_mask is not None else None, inputs_embeds=inputs_embeds)
        need_z = self.z_steps > 1
        enc = self.encoder(emb, mask, output_hidden_states=(output_hidden_states or need_z), return_dict=True)
        seq, hidden = enc.last_hidden_state, enc.hidden_states
        if need_z:
            # iterative refinement: re-run the last layer with the previous output as query
            base, query = hidden[-2], hidden[-1]
            rel_embeddings = self.encoder.get_rel_embedding()
            extras = []
            for _ in range(self.z_steps - 1):
                query, _ = self.encoder.layer[-1](base, mask, query_states=query, rel_embeddings=rel_embeddings)
                extras.append(query)
            seq = query
            if output_hidden_states:
                hidden = tuple(hidden) + tuple(extras)
        if not return_dict:
            return (seq, hidden) if output_hidden_states else (seq,)
        return BaseModelOutput(last_hidden_state=seq, hidden_states=hidden if output_hidden_states else None,
                               attentions=None)
