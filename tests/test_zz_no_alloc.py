"""The allocation-free vocabulary cross-entropy entry point vs. the regular one.

Some callers of this library cannot request device memory at the moment they need the fused
cross-entropy / sampling forward: serving loops with a frozen memory plan, hosts whose allocator
the library must not touch. ``db200_vocab_ce_forward_noalloc`` keeps its scratch inside the
library for them. This test prepares the device once (``db200_noalloc_prepare``: the CUDA driver
loads the library's device image, scratch array included, on first use), then calls the entry
point through its exported C symbol, twice in a row with different sizes (the scratch is shared
and keeps old contents, so the second call checks that stale data does not leak), checks that
neither call changed the amount of free device memory, and compares every output with the
regular entry point, which takes caller-allocated scratch. The file name keeps it last in collection order.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(x, w, b, labels, forb, temperature, seed):
    """Reference path: the existing launcher with scratch allocated by the caller."""
    from deberta_b200.ops import _lib
    from deberta_b200.ops.heads_cuda import _ce_gemm

    N, V = x.shape[0], w.shape[0]
    tile_n = int(_lib.lib().db200_gemm_tile_n(ctypes.c_int(V)))
    tiles_n = (V + tile_n - 1) // tile_n
    part = torch.empty((4, tiles_n, N), dtype=torch.float32, device="cuda")
    label_logit = torch.zeros(N, dtype=torch.float32, device="cuda")
    _ce_gemm(x, w, b, labels, epi=_lib.EPI_CE_FWD, forbidden=forb.data_ptr(), inv_temp=1.0 / temperature, seed=seed,
             ce_part=part.data_ptr(), label_logit=label_logit.data_ptr())
    lse = torch.empty(N, dtype=torch.float32, device="cuda")
    loss = torch.empty(N, dtype=torch.float32, device="cuda")
    sampled = torch.empty(N, dtype=torch.int64, device="cuda")
    _lib.call("db200_ce_combine", _lib.ptr(part), _lib.ptr(label_logit), ctypes.c_int(tiles_n), ctypes.c_int(N),
              _lib.ptr(lse), _lib.ptr(loss), _lib.ptr(sampled), _lib.stream_ptr())
    return lse, loss, sampled


def _noalloc(x, w, b, labels, forb, temperature, seed):
    from deberta_b200.ops import _lib

    fn = _lib.lib().db200_vocab_ce_forward_noalloc
    fn.restype = ctypes.c_int
    N, E = x.shape
    lse = torch.empty(N, dtype=torch.float32, device="cuda")
    loss = torch.empty(N, dtype=torch.float32, device="cuda")
    sampled = torch.empty(N, dtype=torch.int64, device="cuda")
    prepare = _lib.lib().db200_noalloc_prepare
    prepare.restype = ctypes.c_int
    assert prepare() == 0  # idempotent: every call of this helper repeats it
    torch.cuda.synchronize()
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    rc = fn(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(b.data_ptr()),
            ctypes.c_void_p(labels.data_ptr()), ctypes.c_void_p(forb.data_ptr()), ctypes.c_int(N),
            ctypes.c_int(w.shape[0]), ctypes.c_int(E), ctypes.c_float(temperature), ctypes.c_ulonglong(seed),
            ctypes.c_void_p(lse.data_ptr()), ctypes.c_void_p(loss.data_ptr()), ctypes.c_void_p(sampled.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    # neither torch's caching allocator nor the driver handed out memory during the call (cudaMemGetInfo also sees a
    # cudaMalloc made behind torch's back)
    assert torch.cuda.memory_allocated() == before and torch.cuda.mem_get_info()[0] >= free_before
    return rc, lse, loss, sampled


def _problem(N, V, E, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = (torch.randn(N, E, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(V, E, device="cuda", generator=g) * 0.2).to(torch.bfloat16)
    b = (torch.randn(V, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    labels = torch.randint(5, V, (N,), device="cuda", generator=g)
    labels[::7] = -100  # rows without a target: their label logit must read as zero, not as stale scratch
    forb = torch.zeros(V, dtype=torch.uint8, device="cuda")
    forb[:5] = 1
    return x, w, b, labels, forb


def test_noalloc_entry_point_matches_regular_entry_point_twice():
    from deberta_b200.ops import _lib

    for call, (N, V, E) in enumerate([(600, 9000, 128), (130, 128100, 768)]):
        prob = _problem(N, V, E, seed=call)
        want = _regular(*prob, 1.0, 1234 + call)
        rc, *got = _noalloc(*prob, 1.0, 1234 + call)
        torch.cuda.synchronize()
        strerror = _lib.lib().db200_noalloc_strerror
        strerror.restype = ctypes.c_char_p
        assert rc == 0, strerror(rc).decode()
        _lib.check_status()
        torch.testing.assert_close(got[0], want[0], atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(got[1], want[1], atol=1e-5, rtol=1e-5)
        assert torch.equal(got[2], want[2])
        # and against plain PyTorch, within the tolerance of the other kernel tests
        logits = prob[0].float() @ prob[1].float().t() + prob[2].float()
        ref_lse = torch.logsumexp(logits, dim=-1)
        assert (got[0] - ref_lse).abs().max().item() / ref_lse.abs().max().item() < 5e-3


def test_noalloc_entry_point_rejects_oversized_problems():
    from deberta_b200.ops import _lib

    lib = _lib.lib()
    lib.db200_noalloc_strerror.restype = ctypes.c_char_p
    x, w, b, labels, forb = _problem(16, 256, 64, seed=9)
    fn = lib.db200_vocab_ce_forward_noalloc
    fn.restype = ctypes.c_int
    out = torch.empty(16, dtype=torch.float32, device="cuda")
    smp = torch.empty(16, dtype=torch.int64, device="cuda")
    args = lambda rows, vocab: (  # noqa: E731
        ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(b.data_ptr()),
        ctypes.c_void_p(labels.data_ptr()), ctypes.c_void_p(forb.data_ptr()), ctypes.c_int(rows), ctypes.c_int(vocab),
        ctypes.c_int(64), ctypes.c_float(1.0), ctypes.c_ulonglong(1), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(smp.data_ptr()), ctypes.c_void_p(0))
    rc = fn(*args(100_000, 256))  # rejected before any launch: the pointers are never dereferenced
    assert rc == -20 and b"exceeds" in lib.db200_noalloc_strerror(rc)
    assert fn(*args(8192, 128_100)) == -20
