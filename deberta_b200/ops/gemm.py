"""bf16 GEMM on the tcgen05 kernel (``csrc/gemm.cu``) with fused epilogues.

``gemm`` is the one entry point: ``out[M,N] = alpha * A @ B^T`` where the operand
"majors" say which axis of each 2-D (or batched 3-D) operand is contiguous, so that
forward, data-gradient and weight-gradient products of a linear layer all run on the
same kernel without transposed copies. On CPU tensors (or non-bf16 dtypes) the same
contract is evaluated with plain PyTorch in fp32, which is the oracle the GPU tests
compare against.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import EPI_DGELU, EPI_GELU, EPI_GELU_GRAD, EPI_MUL, EPI_NONE, EPI_SWIGLU, EPI_SWIGLU_BWD

__all__ = ["gemm", "gemm_reference", "EPI_NONE", "EPI_GELU", "EPI_DGELU", "EPI_GELU_GRAD", "EPI_MUL", "EPI_SWIGLU",
           "EPI_SWIGLU_BWD"]


def _gelu(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.gelu(x)


def _dgelu(x: torch.Tensor) -> torch.Tensor:
    cdf = 0.5 * (1.0 + torch.erf(x * 0.7071067811865476))
    pdf = torch.exp(-0.5 * x * x) * 0.3989422804014327
    return cdf + x * pdf


def gemm_reference(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    epi: int = EPI_NONE,
    aux: torch.Tensor | None = None,
    alpha: float = 1.0,
    out_dtype: torch.dtype | None = None,
):
    """fp32 PyTorch statement of the GEMM contract (any device)."""
    af = a.float().transpose(-1, -2) if a_mn else a.float()
    bf = b.float() if b_mn else b.float().transpose(-1, -2)
    acc = torch.matmul(af, bf) * alpha
    if bias is not None:
        acc = acc + bias.float()
    if residual is not None:
        acc = acc + residual.float()
    out_dtype = out_dtype or a.dtype
    if epi == EPI_DGELU:
        assert aux is not None
        acc = acc * _dgelu(aux.float())
    if epi == EPI_MUL:
        assert aux is not None
        acc = acc * aux.float()
    if epi == EPI_GELU:
        z = acc.to(out_dtype)
        return z, _gelu(z.float()).to(out_dtype)
    if epi == EPI_SWIGLU:  # ([gate | up], silu(gate) * up) with the activation taken from the rounded halves
        gu = acc.to(out_dtype)
        f = gu.shape[-1] // 2
        return gu, (torch.nn.functional.silu(gu[..., :f].float()) * gu[..., f:].float()).to(out_dtype)
    if epi == EPI_SWIGLU_BWD:  # acc = dh [M, F], aux = [gate | up]
        assert aux is not None
        f = acc.shape[-1]
        gate, up = aux[..., :f].float(), aux[..., f:].float()
        sig = torch.sigmoid(gate)
        return torch.cat([acc * up * sig * (1 + gate * (1 - sig)), acc * gate * sig], dim=-1).to(out_dtype)
    if epi == EPI_GELU_GRAD:  # (gelu'(z), gelu(z)) of the rounded pre-activation
        z = acc.to(out_dtype).float()
        return _dgelu(z).to(out_dtype), _gelu(z).to(out_dtype)
    return acc.to(out_dtype)


def _ld(t: torch.Tensor) -> tuple[int, int]:
    """(leading dim, batch stride) in elements of a 2-D/3-D tensor with unit inner stride."""
    if t.stride(-1) != 1:
        raise ValueError("GEMM operands need a unit inner stride")
    if t.dim() == 2:
        return t.stride(0), 0
    if t.dim() == 3:
        return t.stride(1), t.stride(0)
    raise ValueError("GEMM operands must be 2-D or batched 3-D")


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    epi: int = EPI_NONE,
    aux: torch.Tensor | None = None,
    alpha: float = 1.0,
    out: torch.Tensor | None = None,
    out2: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    accumulate: bool = False,
    split_k: bool = True,
    a_sum: torch.Tensor | None = None,
):
    """``out = epilogue(alpha * A·Bᵀ)``; returns ``out``, ``(z, gelu(z))`` for ``EPI_GELU`` or ``(gelu'(z), gelu(z))``
    for ``EPI_GELU_GRAD`` (``EPI_MUL`` with that first output as ``aux`` is then the whole GELU backward).

    ``a``: [M,K] (``a_mn=False``) or [K,M] (``a_mn=True``); ``b``: [N,K] or [K,N]
    likewise; optional leading batch dim on both. ``accumulate`` adds into an fp32
    ``out`` (used for weight gradients accumulated across micro-batches). ``a_sum`` (fp32 [M], only with ``a_mn`` and an
    fp32 ``out``) receives ``+= Σ_k A[m, k]`` from the same launch: the bias gradient of a linear layer comes out of its
    weight-gradient GEMM.
    """
    use_kernel = a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    if not use_kernel:
        res = gemm_reference(
            a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, residual=residual, epi=epi, aux=aux, alpha=alpha,
            out_dtype=out_dtype or (out.dtype if out is not None else None),
        )
        if out is not None:
            if epi in (EPI_GELU, EPI_GELU_GRAD, EPI_SWIGLU):
                out.copy_(res[0])
                if out2 is not None:
                    out2.copy_(res[1])
                    return out, out2
                return out, res[1]
            if accumulate:
                out.add_(res.to(out.dtype))
            else:
                out.copy_(res)
        if a_sum is not None:
            a_sum.add_((a.float().sum(dim=-2) if a_mn else a.float().sum(dim=-1)).to(a_sum.dtype))
        return res if out is None else out

    batched = a.dim() == 3
    M = a.shape[-1] if a_mn else a.shape[-2]
    K = a.shape[-2] if a_mn else a.shape[-1]
    N = b.shape[-1] if b_mn else b.shape[-2]
    Kb = b.shape[-2] if b_mn else b.shape[-1]
    if K != Kb:
        raise ValueError(f"GEMM inner dims differ: {K} vs {Kb}")
    batch = a.shape[0] if batched else 1
    if out is None:
        dt = out_dtype or torch.bfloat16
        n_out = 2 * N if epi == EPI_SWIGLU_BWD else N  # the SwiGLU backward writes both halves of [d_gate | d_up]
        shape = (batch, M, n_out) if batched else (M, n_out)
        out = torch.empty(shape, dtype=dt, device=a.device)
        if accumulate:
            out.zero_()
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("GEMM output must be bf16 or fp32")
    if epi in (EPI_GELU, EPI_GELU_GRAD) and out2 is None:
        out2 = torch.empty_like(out)
    if epi == EPI_SWIGLU and out2 is None:
        out2 = torch.empty((M, N // 2), dtype=out.dtype, device=a.device)

    args = GemmArgsCache.get()
    lda, bsa = _ld(a)
    ldb, bsb = _ld(b)
    ldo, bso = _ld(out)
    args.A, args.B, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.out2 = out2.data_ptr() if out2 is not None else None
    args.bias = bias.data_ptr() if bias is not None else None
    args.residual = residual.data_ptr() if residual is not None else None
    args.aux = aux.data_ptr() if aux is not None else None
    args.M, args.N, args.K, args.batch = M, N, K, batch
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.epi = epi
    args.out_f32 = int(out.dtype == torch.float32)
    args.accumulate = int(accumulate)
    args.allow_split_k = int(split_k)
    args.alpha = alpha
    args.lda, args.ldb, args.ldo = lda, ldb, ldo
    args.bs_a, args.bs_b, args.bs_out = bsa, bsb, bso
    args.ldo2, args.bs_out2 = _ld(out2) if out2 is not None else (0, 0)
    args.ldr, args.bs_res = _ld(residual) if residual is not None else (0, 0)
    args.ldaux, args.bs_aux = _ld(aux) if aux is not None else (0, 0)
    args.bs_bias = bias.stride(0) if (bias is not None and bias.dim() == 2) else 0
    if a_sum is not None and (a_sum.dtype != torch.float32 or not a_sum.is_contiguous() or a_sum.numel() != M):
        raise ValueError("a_sum must be a dense fp32 vector of M elements")
    args.a_sum = a_sum.data_ptr() if a_sum is not None else None
    for t in (bias, residual, aux, out, out2):
        if t is not None and t.data_ptr() % 16:
            raise ValueError("GEMM epilogue tensors must be 16-byte aligned")
    _lib.call("db200_gemm_bf16", ctypes.byref(args), _lib.stream_ptr())
    if epi in (EPI_GELU, EPI_GELU_GRAD, EPI_SWIGLU):
        return out, out2
    return out


class GemmArgsCache:
    """One reusable argument struct per thread (ctypes allocation is not free)."""

    _local = None

    @classmethod
    def get(cls) -> _lib.GemmArgs:
        import threading

        if cls._local is None:
            cls._local = threading.local()
        inst = getattr(cls._local, "args", None)
        if inst is None:
            inst = _lib.GemmArgs()
            cls._local.args = inst
        return inst
