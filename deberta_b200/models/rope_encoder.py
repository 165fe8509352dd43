"""RoPE encoder backbone: fused-QKV rotary attention, RMSNorm (post or KEEL), MLP/SwiGLU.

State-dict names follow ``rope_encoder.py`` of the reference (``encoder.layers.{i}.attn.qkv`` …).
Attention runs through ``ops.attention.rope_attention``, which takes packed-document ids
or a padding mask directly, so no dense S×S mask is built for document blocking.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn
from transformers import PretrainedConfig, PreTrainedModel
from transformers.modeling_outputs import BaseModelOutput

from deberta_b200.ops.attention import rope_attention
from deberta_b200.ops.linear import ffn_gelu, ffn_swiglu, linear, split_qkv

from .activations import get_act_fn
from .mask_utils import AttnMask
from .norm import RMSNorm
from .rope import RotaryEmbedding

__all__ = ["DebertaRoPEConfig", "DebertaRoPEModel", "DebertaRoPELayer", "DebertaRoPEEncoder"]



def _embed(module: nn.Module, input_ids: torch.Tensor) -> torch.Tensor:
    """Word-embedding lookup: plain ``nn.Embedding`` tables go through the gather kernel, wrapped ones keep their forward."""
    if type(module) is nn.Embedding and module.max_norm is None and not module.sparse:
        from deberta_b200.ops.embedding import embedding_lookup

        return embedding_lookup(input_ids, module.weight, None, module.padding_idx)
    return module(input_ids)

class DebertaRoPEConfig(PretrainedConfig):
    model_type = "deberta-rope"

    def __init__(
        self, *, vocab_size: int = 50265, hidden_size: int = 768, num_hidden_layers: int = 12,
        num_attention_heads: int = 12, intermediate_size: int = 3072, hidden_act: str = "gelu",
        ffn_type: str = "swiglu", use_bias: bool = False, hidden_dropout_prob: float = 0.0,
        attention_probs_dropout_prob: float = 0.0, max_position_embeddings: int = 512, type_vocab_size: int = 2,
        pad_token_id: int = 0, rope_theta: float = 10000.0, rotary_pct: float = 1.0,
        use_absolute_position_embeddings: bool = False, norm_eps: float = 1e-6, norm_arch: str = "post",
        keel_alpha_init: float | None = None, keel_alpha_learnable: bool = False,
        attention_implementation: str = "sdpa", initializer_range: float = 0.02, **kwargs: Any,
    ) -> None:
        super().__init__(pad_token_id=pad_token_id, **kwargs)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.num_hidden_layers, self.num_attention_heads = int(num_hidden_layers), int(num_attention_heads)
        self.intermediate_size, self.hidden_act = int(intermediate_size), str(hidden_act)
        self.ffn_type, self.use_bias = str(ffn_type), bool(use_bias)
        self.hidden_dropout_prob = float(hidden_dropout_prob)
        self.attention_probs_dropout_prob = float(attention_probs_dropout_prob)
        self.max_position_embeddings, self.type_vocab_size = int(max_position_embeddings), int(type_vocab_size)
        self.rope_theta, self.rotary_pct = float(rope_theta), float(rotary_pct)
        self.use_absolute_position_embeddings = bool(use_absolute_position_embeddings)
        self.norm_eps, self.norm_arch = float(norm_eps), str(norm_arch)
        self.keel_alpha_init = None if keel_alpha_init is None else float(keel_alpha_init)
        self.keel_alpha_learnable = bool(keel_alpha_learnable)
        self.attention_implementation = str(attention_implementation)
        self.initializer_range = float(initializer_range)
        if self.hidden_size % self.num_attention_heads:
            raise ValueError(
                f"hidden_size ({self.hidden_size}) must be divisible by num_attention_heads ({self.num_attention_heads})."
            )
        if not 0.0 < self.rotary_pct <= 1.0:
            raise ValueError("rotary_pct must be in (0, 1].")
        if self.ffn_type not in {"swiglu", "mlp"}:
            raise ValueError("ffn_type must be one of: swiglu|mlp")
        if self.norm_arch not in {"post", "keel"}:
            raise ValueError("norm_arch must be one of: post|keel")
        if self.attention_implementation not in {"sdpa", "eager"}:
            raise ValueError("attention_implementation must be one of: sdpa|eager")


def _drop(x, p, training):
    return F.dropout(x, p, True) if (training and p > 0.0) else x


class DebertaRoPEEmbeddings(nn.Module):
    def __init__(self, config: DebertaRoPEConfig) -> None:
        super().__init__()
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size, padding_idx=config.pad_token_id)
        self.token_type_embeddings = (
            nn.Embedding(config.type_vocab_size, config.hidden_size) if config.type_vocab_size > 0 else None
        )
        self.position_embeddings = (
            nn.Embedding(config.max_position_embeddings, config.hidden_size)
            if config.use_absolute_position_embeddings else None
        )
        self.norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.dropout_p = float(config.hidden_dropout_prob)

    def forward(self, input_ids: torch.Tensor, token_type_ids: torch.Tensor | None = None) -> torch.Tensor:
        bsz, seq_len = input_ids.shape
        x = _embed(self.word_embeddings, input_ids)
        if self.token_type_embeddings is not None:
            if token_type_ids is None:
                token_type_ids = torch.zeros((bsz, seq_len), dtype=torch.long, device=input_ids.device)
            x = x + self.token_type_embeddings(token_type_ids)
        if self.position_embeddings is not None:
            x = x + self.position_embeddings(torch.arange(seq_len, device=input_ids.device))[None]
        return _drop(self.norm(x), self.dropout_p, self.training)


class DebertaRoPESelfAttention(nn.Module):
    """Fused-QKV rotary attention; inactive query rows are zero after ``out_proj`` (``:204-287``)."""

    def __init__(self, config: DebertaRoPEConfig) -> None:
        super().__init__()
        self.hidden_size = int(config.hidden_size)
        self.num_heads = int(config.num_attention_heads)
        self.head_dim = self.hidden_size // self.num_heads
        bias = bool(config.use_bias)
        self.qkv = nn.Linear(self.hidden_size, 3 * self.hidden_size, bias=bias)
        self.out_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=bias)
        self.attn_dropout = float(config.attention_probs_dropout_prob)
        self.attn_impl = str(config.attention_implementation)
        rd = int(self.head_dim * float(config.rotary_pct))
        self.rotary_dim = rd - (rd % 2)
        self.rope = (
            RotaryEmbedding(self.rotary_dim, base=float(config.rope_theta), full_dim=self.head_dim)
            if self.rotary_dim > 0 else None
        )

    def forward(self, x: torch.Tensor, attention_mask, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``out_proj(attention(x)) (+ residual)``; the residual is added in the projection's epilogue."""
        mask = AttnMask.from_any(attention_mask)
        q, k, v = split_qkv(linear(x, self.qkv.weight, self.qkv.bias))
        cos = sin = None
        if self.rope is not None:
            cos, sin = self.rope.get_cos_sin(x.shape[1], device=x.device, dtype=torch.float32)
        ctx = rope_attention(q, k, v, cos, sin, heads=self.num_heads, rotary_dim=self.rotary_dim,
                             dropout_p=self.attn_dropout, training=self.training, **mask.kwargs())
        keep = mask.token_keep()
        if keep is None or self.out_proj.bias is None:
            # (rows of inactive queries leave the attention as zeros: without a bias the projection keeps them zero)
            return linear(ctx, self.out_proj.weight, self.out_proj.bias, residual=residual)
        out = linear(ctx, self.out_proj.weight, self.out_proj.bias) * keep[:, :, None].to(ctx.dtype)
        return out if residual is None else out + residual


class DebertaRoPEMLP(nn.Module):
    """``mlp``: Linear→act→Linear; ``swiglu``: fused gate+up ``w12``, SiLU gate, ``w3`` (``:290-343``)."""

    def __init__(self, config: DebertaRoPEConfig) -> None:
        super().__init__()
        self.ffn_type = str(config.ffn_type).lower()
        bias = bool(config.use_bias)
        h, i = int(config.hidden_size), int(config.intermediate_size)
        if self.ffn_type == "swiglu":
            self.w12 = nn.Linear(h, 2 * i, bias=bias)
            self.w3 = nn.Linear(i, h, bias=bias)
        elif self.ffn_type == "mlp":
            self.dense_in = nn.Linear(h, i, bias=bias)
            self.act_name = str(config.hidden_act)
            self.act = get_act_fn(config.hidden_act)
            self.dense_out = nn.Linear(i, h, bias=bias)
        else:
            raise ValueError(f"Unsupported ffn_type: {self.ffn_type}")

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """``FFN(x) (+ residual)``; the residual is added in the epilogue of the second GEMM."""
        if self.ffn_type == "swiglu":
            return ffn_swiglu(x, self.w12.weight, self.w12.bias, self.w3.weight, self.w3.bias, residual=residual)
        if self.act_name == "gelu":
            return ffn_gelu(x, self.dense_in.weight, self.dense_in.bias, self.dense_out.weight, self.dense_out.bias,
                            residual=residual)
        return linear(self.act(linear(x, self.dense_in.weight, self.dense_in.bias)),
                      self.dense_out.weight, self.dense_out.bias, residual=residual)


class _KEELAlpha(nn.Module):
    def __init__(self, init: float, learnable: bool) -> None:
        super().__init__()
        self.init_value = float(init)
        if learnable:
            self.alpha = nn.Parameter(torch.tensor(float(init), dtype=torch.float32))
        else:
            self.register_buffer("alpha", torch.tensor(float(init), dtype=torch.float32), persistent=False)
        self.learnable = bool(learnable)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.alpha.to(dtype=x.dtype)


class DebertaRoPELayer(nn.Module):
    """post: ``x = N(x + F(x))``; keel: ``x = N_outer(α·x + F(N_inner(x)))`` per sub-layer (``:371-429``)."""

    def __init__(self, config: DebertaRoPEConfig, *, alpha_init: float) -> None:
        super().__init__()
        self.norm_arch = str(config.norm_arch)
        self.attn = DebertaRoPESelfAttention(config)
        self.mlp = DebertaRoPEMLP(config)
        self.dropout_p = float(config.hidden_dropout_prob)
        if self.norm_arch == "post":
            self.norm1 = RMSNorm(config.hidden_size, eps=config.norm_eps)
            self.norm2 = RMSNorm(config.hidden_size, eps=config.norm_eps)
        else:
            for name in ("inner_norm1", "outer_norm1", "inner_norm2", "outer_norm2"):
                setattr(self, name, RMSNorm(config.hidden_size, eps=config.norm_eps))
            self.alpha1 = _KEELAlpha(alpha_init, learnable=config.keel_alpha_learnable)
            self.alpha2 = _KEELAlpha(alpha_init, learnable=config.keel_alpha_learnable)

    def forward(self, x: torch.Tensor, attention_mask) -> torch.Tensor:
        d = lambda h: _drop(h, self.dropout_p, self.training)  # noqa: E731
        if not (self.training and self.dropout_p > 0.0):  # residual sums inside the GEMM epilogues
            if self.norm_arch == "post":
                x = self.norm1(self.attn(x, attention_mask, residual=x))
                return self.norm2(self.mlp(x, residual=x))
            x = self.outer_norm1(self.attn(self.inner_norm1(x), attention_mask, residual=self.alpha1(x) * x))
            return self.outer_norm2(self.mlp(self.inner_norm2(x), residual=self.alpha2(x) * x))
        if self.norm_arch == "post":
            x = self.norm1(x + d(self.attn(x, attention_mask)))
            return self.norm2(x + d(self.mlp(x)))
        x = self.outer_norm1(self.alpha1(x) * x + d(self.attn(self.inner_norm1(x), attention_mask)))
        return self.outer_norm2(self.alpha2(x) * x + d(self.mlp(self.inner_norm2(x))))


class DebertaRoPEEncoder(nn.Module):
    def __init__(self, config: DebertaRoPEConfig) -> None:
        super().__init__()
        # KEEL default: alpha = 1/sqrt(number of residual sub-layers) = 1/sqrt(2L)
        alpha = (float(config.keel_alpha_init) if config.keel_alpha_init is not None
                 else 1.0 / math.sqrt(2.0 * int(config.num_hidden_layers)))
        self.layers = nn.ModuleList([DebertaRoPELayer(config, alpha_init=alpha) for _ in range(config.num_hidden_layers)])
        self.gradient_checkpointing = False

    def forward(self, x: torch.Tensor, attention_mask, *, output_hidden_states: bool = False):
        mask = AttnMask.from_any(attention_mask)
        hidden = (x,) if output_hidden_states else None
        for layer in self.layers:
            if self.gradient_checkpointing and self.training:
                x = torch.utils.checkpoint.checkpoint(lambda h, layer=layer: layer(h, mask), x, use_reentrant=False)
            else:
                x = layer(x, mask)
            if output_hidden_states:
                hidden = hidden + (x,)
        return x, hidden


class DebertaRoPEPreTrainedModel(PreTrainedModel):
    config_class = DebertaRoPEConfig
    base_model_prefix = "deberta_rope"
    supports_gradient_checkpointing = True

    def _init_weights(self, module: nn.Module) -> None:
        from ._hf_init import init_embedding_, init_linear_, init_norm_

        std = float(self.config.initializer_range)
        if isinstance(module, nn.Linear):
            init_linear_(module, std)
        elif isinstance(module, nn.Embedding):
            init_embedding_(module, std)
        elif isinstance(module, RMSNorm):
            init_norm_(module.weight)
        elif isinstance(module, RotaryEmbedding):
            module.reset_buffers()
        elif isinstance(module, _KEELAlpha):
            # a fixed alpha is a non-persistent buffer: no checkpoint carries it, and a model materialised from the
            # meta device holds arbitrary memory there until it is written again
            if not module.learnable or not getattr(module.alpha, "_is_hf_initialized", False):
                module.alpha.data.fill_(module.init_value)

    def _set_gradient_checkpointing(self, module: nn.Module = None, value: bool = False, **_: Any) -> None:
        for m in self.modules():
            if isinstance(m, DebertaRoPEEncoder):
                m.gradient_checkpointing = bool(value)

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None) -> None:
        self._set_gradient_checkpointing(value=True)

    def gradient_checkpointing_disable(self) -> None:
        self._set_gradient_checkpointing(value=False)


class DebertaRoPEModel(DebertaRoPEPreTrainedModel):
    def __init__(self, config: DebertaRoPEConfig) -> None:
        super().__init__(config)
        self.embeddings = DebertaRoPEEmbeddings(config)
        self.encoder = DebertaRoPEEncoder(config)
        self.post_init()

    def get_input_embeddings(self) -> nn.Module:
        return self.embeddings.word_embeddings

    def set_input_embeddings(self, value: nn.Module) -> None:
        self.embeddings.word_embeddings = value

    def forward(self, input_ids, attention_mask=None, token_type_ids=None, output_hidden_states=None,
                output_attentions=None, return_dict=None):
        output_hidden_states = bool(
            getattr(self.config, "output_hidden_states", False) if output_hidden_states is None else output_hidden_states
        )
        return_dict = bool(getattr(self.config, "return_dict", True) if return_dict is None else return_dict)
        if output_attentions:
            raise NotImplementedError("DebertaRoPEModel does not expose attention maps; set output_attentions=False.")
        x = self.embeddings(input_ids=input_ids, token_type_ids=token_type_ids)
        x, hidden = self.encoder(x, attention_mask, output_hidden_states=output_hidden_states)
        if not return_dict:
            return (x, hidden) if output_hidden_states else (x,)
        return BaseModelOutput(last_hidden_state=x, hidden_states=hidden if output_hidden_states else None)
