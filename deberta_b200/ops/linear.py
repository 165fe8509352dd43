"""Linear layers and the fused GELU feed-forward block on the tcgen05 GEMM.

On bf16 CUDA tensors every product (forward, data gradient, weight gradient) runs on
``csrc/gemm.cu`` with the bias / residual / GELU / GELU-derivative work folded into the
GEMM epilogues. Weight and bias gradients are accumulated in fp32 directly into
``param.main_grad`` when the engine attached one (so micro-batch accumulation costs no
extra pass); otherwise they are returned to autograd. Everything else (CPU, fp32)
takes the plain PyTorch path, which is also the oracle for the GPU tests.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .gemm import EPI_DGELU, EPI_GELU, EPI_GELU_GRAD, EPI_MUL, EPI_SWIGLU, EPI_SWIGLU_BWD, gemm

__all__ = ["linear", "linear_qkv", "split_qkv", "ffn_gelu", "ffn_swiglu", "use_kernels", "ResidualGradSink"]


def use_kernels(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def weight_grad_into(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, main: torch.Tensor | None) -> torch.Tensor | None:
    """dW[out,in] = dyᵀ·x: added to the fp32 buffer ``main`` when given (returns ``None``), else returned in ``w``'s dtype."""
    if main is not None:
        gemm(dy, x, a_mn=True, b_mn=True, out=main, accumulate=True)
        return None
    return gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32).to(w.dtype)


def _weight_grad(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor | None:
    """dW accumulated into ``w.main_grad`` when the engine attached one."""
    return weight_grad_into(dy, x, w, getattr(w, "main_grad", None))


def colsum_into(dy: torch.Tensor, out: torch.Tensor) -> None:
    """``out[n] += Σ_m dy[m, n]`` (bf16 in, fp32 accumulate) on the column-sum kernel."""
    import ctypes

    from . import _lib

    _lib.call("db200_colsum_bf16", _lib.ptr(dy), ctypes.c_longlong(dy.stride(0)), ctypes.c_int(dy.shape[0]),
              ctypes.c_int(dy.shape[1]), _lib.ptr(out), _lib.stream_ptr())


def bias_grad_into(dy: torch.Tensor, main: torch.Tensor | None, dtype: torch.dtype) -> torch.Tensor | None:
    """Column sums of ``dy``: added to the fp32 buffer ``main`` when given (returns ``None``), else returned as ``dtype``."""
    kernel_ok = dy.is_cuda and dy.dtype == torch.bfloat16 and dy.stride(1) == 1 and dy.stride(0) % 8 == 0 and dy.data_ptr() % 16 == 0
    if main is not None and kernel_ok:
        colsum_into(dy, main)
        return None
    if kernel_ok:
        g = torch.zeros(dy.shape[1], dtype=torch.float32, device=dy.device)
        colsum_into(dy, g)
    else:
        g = dy.sum(dim=0, dtype=torch.float32)
    if main is not None:
        main.add_(g)
        return None
    return g.to(dtype)


def _bias_grad(dy: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor | None:
    if b is None:
        return None
    return bias_grad_into(dy, getattr(b, "main_grad", None), b.dtype)


def param_grads_into(dy, x, w, w_main, b_main, want_w: bool = True, want_b: bool = True, b_dtype=None):
    """(dW, db) of ``y = x·Wᵀ + b`` from ``dy``. With fp32 accumulation buffers for both, ONE launch produces them: the
    weight-gradient GEMM also sums ``dy`` over the tokens on the tensor cores (no separate column-sum pass)."""
    fused = (want_w and want_b and w_main is not None and b_main is not None and dy.is_cuda and dy.dtype == torch.bfloat16
             and x.dtype == torch.bfloat16 and dy.dim() == 2 and b_main.is_contiguous())
    if fused:
        gemm(dy, x, a_mn=True, b_mn=True, out=w_main, accumulate=True, a_sum=b_main)
        return None, None
    dw = weight_grad_into(dy, x, w, w_main) if want_w else None
    db = bias_grad_into(dy, b_main, b_dtype or w.dtype) if want_b else None
    return dw, db


def _param_grads(dy, x, w, b):
    want_b = b is not None and b.requires_grad
    return param_grads_into(dy, x, w, getattr(w, "main_grad", None), getattr(b, "main_grad", None) if want_b else None,
                            w.requires_grad, want_b, b.dtype if b is not None else None)


class ResidualGradSink:
    """Carries the gradient of a residual branch from the projection that closes a block to the projection that opened
    it, when both read the same tensor: ``y = W_o·f(W_qkv·x) + x``. Autograd would add the two gradients of ``x`` with a
    separate kernel; instead the closing projection's backward parks its residual gradient here (and reports none), and
    the opening projection's backward, which autograd necessarily runs later, adds it in the epilogue of its
    data-gradient GEMM. ``armed`` is set by the opening projection once it is certain to collect."""

    __slots__ = ("armed", "grad")

    def __init__(self) -> None:
        self.armed = False
        self.grad = None


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual, sink):
        # Parameters are kept by reference, not through save_for_backward: activation checkpointing hands saved
        # tensors back as detached copies, which have lost the parameter's ``main_grad`` buffer.
        ctx.save_for_backward(x)
        ctx.w_ref = w
        ctx.has_bias = b is not None
        ctx.bias_ref = b
        ctx.has_res = residual is not None
        ctx.sink = sink if (sink is not None and sink.armed and residual is not None) else None
        return gemm(x, w, bias=b, residual=residual)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        w = ctx.w_ref
        # (a column slice of a wider buffer, e.g. one third of the attention backward's dQ | dK | dV, is read in place)
        if dy.stride(1) != 1 or dy.stride(0) % 8 or dy.data_ptr() % 16:
            dy = dy.contiguous()
        dx = gemm(dy, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw, db = _param_grads(dy, x, w, ctx.bias_ref if ctx.has_bias else None)
        dres = dy if ctx.has_res else None
        if ctx.sink is not None and dres is not None:
            ctx.sink.grad, dres = dres, None
        return dx, dw, db, dres, None


def linear(
    x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None, residual: torch.Tensor | None = None,
    residual_sink: ResidualGradSink | None = None,
) -> torch.Tensor:
    """``x @ wᵀ + b (+ residual)`` over the last dim of ``x`` (any leading shape). ``residual_sink``: see
    :class:`ResidualGradSink` (only an armed sink is used)."""
    if not (use_kernels(x) and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0):
        out = F.linear(x, w.to(x.dtype) if w.dtype != x.dtype else w, None if b is None else b.to(x.dtype))
        return out if residual is None else out + residual
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    r2 = None if residual is None else residual.reshape(-1, w.shape[0]).contiguous()
    if torch.compiler.is_compiling():
        from . import library

        # No gradient buffers under a compiler: a buffer is a view at an offset inside the engine's flat fp32 storage, and an
        # op that mutates such a graph input makes the compiler copy "its base" (offset + size elements, read from the
        # view's own address: past the end of the storage). The parameter gradients come back as tensors instead and
        # the engine's post-accumulate hook adds them to the buffers.
        out = library.linear(x2, w, b, r2, None, None)
    else:
        out = _Linear.apply(x2, w, b, r2, residual_sink)
    return out.view(*lead, w.shape[0])


class _FFNGelu(torch.autograd.Function):
    """y = W2·gelu(W1·x + b1) + b2 + residual.

    The first GEMM writes gelu(z) and gelu'(z) (both from one cdf/pdf evaluation) instead of z, so the W2
    data-gradient GEMM only multiplies by a stored factor in its epilogue.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual, residual_is_x):
        if residual_is_x:  # the usual transformer block: y = FFN(x) + x
            residual = x
        g, a = gemm(x, w1, bias=b1, epi=EPI_GELU_GRAD)
        y = gemm(a, w2, bias=b2, residual=residual)
        ctx.save_for_backward(x, g, a)
        ctx.params = (w1, b1, w2, b2)  # by reference (see _Linear)
        ctx.has_res = residual is not None and not residual_is_x
        ctx.res_is_x = bool(residual_is_x)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, g, a = ctx.saved_tensors
        w1, b1, w2, b2 = ctx.params
        dy = dy.contiguous()
        dz = gemm(dy, w2, b_mn=True, epi=EPI_MUL, aux=g)
        dw2, db2 = _param_grads(dy, a, w2, b2)
        # with y = FFN(x) + x the two gradients of x meet in the epilogue of the W1 data-gradient GEMM (no add kernel)
        dx = gemm(dz, w1, b_mn=True, residual=dy if ctx.res_is_x else None) if ctx.needs_input_grad[0] else None
        dw1, db1 = _param_grads(dz, x, w1, b1)
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None), None


def ffn_gelu(x, w1, b1, w2, b2, residual=None):
    """Feed-forward block with exact-erf GELU: ``W2·gelu(W1·x+b1)+b2 (+residual)``."""
    if not (use_kernels(x) and w1.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w1.shape[0] % 8 == 0):
        h = F.gelu(F.linear(x, w1.to(x.dtype), None if b1 is None else b1.to(x.dtype)))
        out = F.linear(h, w2.to(x.dtype), None if b2 is None else b2.to(x.dtype))
        return out if residual is None else out + residual
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    r2 = None if residual is None else residual.reshape(-1, w2.shape[0]).contiguous()
    if torch.compiler.is_compiling():
        from . import library

        out = library.ffn_gelu(x2, w1, b1, w2, b2, r2, None, None, None, None)[0]  # no buffers: see linear()
    else:
        same = residual is x and x.requires_grad
        out = _FFNGelu.apply(x2, w1, b1, w2, b2, None if same else r2, same)
    return out.view(*lead, w2.shape[0])


class _FFNSwiGLU(torch.autograd.Function):
    """``W3·(silu(gate) ⊙ up) + b3`` with ``[gate | up] = W12·x + b12``: the activation and its derivative run in the
    epilogues of the GEMMs next to them (``EPI_SWIGLU`` writes ``[gate | up]`` and the product from one accumulator
    tile; ``EPI_SWIGLU_BWD`` turns ``dh = dy·W3`` into ``[d_gate | d_up]`` before it leaves the SM), so the forward has no
    pass that re-reads the ``[tokens, 2F]`` projection and the backward none that writes and re-reads ``dh``."""

    @staticmethod
    def forward(ctx, x, w12, b12, w3, b3, residual):
        gu, h = gemm(x, w12, bias=b12, epi=EPI_SWIGLU)
        y = gemm(h, w3, bias=b3, residual=residual)
        ctx.save_for_backward(x, gu, h)
        ctx.params = (w12, b12, w3, b3)  # by reference (see _Linear)
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gu, h = ctx.saved_tensors
        w12, b12, w3, b3 = ctx.params
        dy = dy.contiguous()
        dgu = gemm(dy, w3, b_mn=True, epi=EPI_SWIGLU_BWD, aux=gu)
        dw3, db3 = _param_grads(dy, h, w3, b3)
        dx = gemm(dgu, w12, b_mn=True) if ctx.needs_input_grad[0] else None
        dw12, db12 = _param_grads(dgu, x, w12, b12)
        return dx, dw12, db12, dw3, db3, (dy if ctx.has_res else None)


def ffn_swiglu(x, w12, b12, w3, b3, residual=None):
    """SwiGLU feed-forward block ``W3·(silu(gate) ⊙ up) + b3 (+ residual)``, ``[gate | up] = W12·x + b12``
    (the reference's ``modeling/rope_encoder.py:290-343``)."""
    f = w12.shape[0] // 2
    fused = (use_kernels(x) and w12.dtype == torch.bfloat16 and w3.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
             and f % 8 == 0 and w12.shape[0] == 2 * f and f >= 64 and w3.shape[0] % 8 == 0
             and not torch.compiler.is_compiling())
    if not fused:
        from .elementwise import swiglu

        return linear(swiglu(linear(x, w12, b12)), w3, b3, residual)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    r2 = None if residual is None else residual.reshape(-1, w3.shape[0]).contiguous()
    return _FFNSwiGLU.apply(x2, w12, b12, w3, b3, r2).view(*lead, w3.shape[0])


# ---- fused query / key / value projection ------------------------------------------------------------

def _follows(a: torch.Tensor, b: torch.Tensor) -> bool:
    """``b`` starts where ``a`` ends in memory (both dense)."""
    return a.is_contiguous() and b.is_contiguous() and b.data_ptr() == a.data_ptr() + a.numel() * a.element_size()


def _span3(t: torch.Tensor, shape: tuple[int, ...]) -> torch.Tensor:
    """View over ``t`` and the two tensors that follow it in memory."""
    strides = (shape[1], 1) if len(shape) == 2 else (1,)
    return t.detach().as_strided(shape, strides, t.storage_offset())


def _qkv_fusable(x, wq, bq, wk, bk, wv, bv) -> bool:
    if not (use_kernels(x) and wq.dtype == torch.bfloat16 and wq.shape == wk.shape == wv.shape):
        return False
    if wq.shape[0] % 8 or wq.shape[1] % 8 or not (_follows(wq, wk) and _follows(wk, wv)):
        return False
    if (bq is None) != (bk is None) or (bq is None) != (bv is None):
        return False
    if bq is not None and not (_follows(bq, bk) and _follows(bk, bv)):
        return False
    grads = [getattr(t, "main_grad", None) for t in (wq, wk, wv)]
    if any(g is None for g in grads) or not (_follows(grads[0], grads[1]) and _follows(grads[1], grads[2])):
        return False
    if bq is not None:
        bg = [getattr(t, "main_grad", None) for t in (bq, bk, bv)]
        if any(g is None for g in bg) or not (_follows(bg[0], bg[1]) and _follows(bg[1], bg[2])):
            return False
    return all(t.requires_grad for t in (wq, wk, wv))


class _LinearQKV(torch.autograd.Function):
    """``x @ [Wq; Wk; Wv]ᵀ + [bq; bk; bv]`` as one GEMM when the three parameter sets are adjacent in memory."""

    @staticmethod
    def forward(ctx, x, wq, bq, sink):
        n, k = wq.shape
        w_all = _span3(wq, (3 * n, k))
        b_all = None if bq is None else _span3(bq, (3 * n,))
        ctx.save_for_backward(x)
        ctx.wq = wq  # by reference (see _Linear)
        ctx.bq = bq
        ctx.sink = sink
        return gemm(x, w_all, bias=b_all)

    @staticmethod
    def backward(ctx, dqkv):
        (x,) = ctx.saved_tensors
        wq = ctx.wq
        n, k = wq.shape
        if dqkv.stride(1) != 1 or dqkv.stride(0) % 8 or dqkv.data_ptr() % 16:
            dqkv = dqkv.contiguous()
        parked = None
        if ctx.sink is not None:  # the block's residual gradient, parked by the projection that closed the block
            parked, ctx.sink.grad = ctx.sink.grad, None
            if parked is not None and (parked.shape != x.shape or not parked.is_contiguous()):
                parked = parked.reshape(x.shape).contiguous()
        dx = gemm(dqkv, _span3(wq, (3 * n, k)), b_mn=True, residual=parked) if ctx.needs_input_grad[0] else None
        want_b = ctx.bq is not None and ctx.bq.requires_grad
        gemm(dqkv, x, a_mn=True, b_mn=True, out=_span3(wq.main_grad, (3 * n, k)), accumulate=True,
             a_sum=_span3(ctx.bq.main_grad, (3 * n,)) if want_b else None)
        return dx, None, None, None


class _SplitQKV(torch.autograd.Function):
    """[T, 3N] → three [T, N] column views; the backward hands back one [T, 3N] tensor without a copy when the
    three gradients already sit side by side in one buffer (the attention backward writes them that way)."""

    @staticmethod
    def forward(ctx, qkv):
        n = qkv.shape[-1] // 3
        return qkv[:, :n], qkv[:, n : 2 * n], qkv[:, 2 * n :]

    @staticmethod
    def backward(ctx, dq, dk, dv):
        n = dq.shape[-1]
        es = dq.element_size()
        side_by_side = (
            dq.stride() == dk.stride() == dv.stride() == (3 * n, 1)
            and dk.data_ptr() == dq.data_ptr() + n * es and dv.data_ptr() == dk.data_ptr() + n * es
        )
        if side_by_side:
            return dq.as_strided((dq.shape[0], 3 * n), (3 * n, 1), dq.storage_offset())
        return torch.cat([dq, dk, dv], dim=-1)


def split_qkv(qkv: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``[..., 3N]`` → three ``[..., N]`` column views. Unlike three slices, whose backward passes would each zero-fill
    and copy a full ``[..., 3N]`` tensor and then be added up, the backward hands the three gradients back as one tensor
    (without any copy when they already sit side by side, as the attention backward writes them)."""
    lead = qkv.shape[:-1]
    q, k, v = _SplitQKV.apply(qkv.reshape(-1, qkv.shape[-1]))
    if len(lead) == 1:
        return q, k, v
    return tuple(t.unflatten(0, lead) for t in (q, k, v))


def linear_qkv(x, wq, bq, wk, bk, wv, bv, residual_sink: ResidualGradSink | None = None):
    """Query, key and value projections of the same input: ``(q, k, v)`` with ``x``'s leading shape.

    One GEMM with a three times wider output when the engine laid the three weights (and biases, and their fp32
    gradient buffers) out back to back, three GEMMs otherwise. ``residual_sink``: when the fused form runs and ``x``
    needs a gradient, the sink is armed and this projection's backward collects what the block's closing projection
    parks there (:class:`ResidualGradSink`).
    """
    if torch.compiler.is_compiling() or not _qkv_fusable(x, wq, bq, wk, bk, wv, bv):
        # (the fused form compares storage addresses of parameters, which a tracing compiler cannot see)
        return linear(x, wq, bq), linear(x, wk, bk), linear(x, wv, bv)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or x2.stride(0) % 8:
        x2 = x2.contiguous()
    sink = residual_sink if (residual_sink is not None and x.requires_grad and torch.is_grad_enabled()) else None
    if sink is not None:
        sink.armed = True
    q, k, v = _SplitQKV.apply(_LinearQKV.apply(x2, wq, bq, sink))
    if len(lead) == 1:
        return q, k, v
    return tuple(t.unflatten(0, lead) for t in (q, k, v))
