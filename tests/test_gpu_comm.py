"""Fused gradient collectives (csrc/comm.cu).

On one GPU the ranks are emulated: each "rank" is a set of local buffers, the flags a peer would
raise are written by the host before the launch, and the ranks' kernels run one after the other
(no kernel ever waits for another kernel). The real multi-GPU path runs as child processes when the
machine has at least two GPUs.
"""

import ctypes
import math
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

FLAG_WORDS = 32          # [4 channels][8 sources]
NORM_WORD0 = 32          # squared-norm share of each source


def _ctx(rank, grads, params, pads, timeout_s=2.0):
    from deberta_b200.parallel.peer import CommCtx

    c = CommCtx()
    c.world, c.rank = len(grads), rank
    for r in range(len(grads)):
        c.grads[r] = grads[r].data_ptr()
        c.params[r] = params[r].data_ptr()
        c.pads[r] = pads[r].data_ptr()
    c.mc_grads = None
    c.mc_params = None
    c.timeout_ns = int(timeout_s * 1e9)
    return c


def test_emulated_ranks_reduce_adamw_match_reference():
    from deberta_b200.ops import _lib
    from deberta_b200.parallel.peer import PAD_WORDS, AdamSegment

    dev = torch.device("cuda")
    world, per = 4, 64 * 1024
    n = world * per
    torch.manual_seed(0)
    grads = [torch.randn(n, device=dev) for _ in range(world)]
    params = [torch.zeros(n, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    pads = [torch.zeros(PAD_WORDS, device=dev, dtype=torch.int32) for _ in range(world)]
    for p in pads:
        p[:FLAG_WORDS] = 1000  # every flag a peer would raise is already up
    want = torch.stack(grads).double().sum(0) / world
    masters = [torch.randn(per, device=dev) for _ in range(world)]
    ref_masters = [m.clone() for m in masters]
    ms = [torch.zeros(per, device=dev) for _ in range(world)]
    vs = [torch.zeros(per, device=dev) for _ in range(world)]
    norm_out = torch.zeros(1, device=dev)
    lr, wd, b1, b2, eps, max_norm = 1e-2, 0.1, 0.9, 0.999, 1e-6, 1.0
    stream = _lib.stream_ptr()
    for r in range(world):
        c = _ctx(r, grads, params, pads)
        _lib.call("db200_comm_reduce", ctypes.byref(c), ctypes.c_longlong(r * per), ctypes.c_longlong(per),
                  ctypes.c_float(1.0 / world), ctypes.c_int(0), ctypes.c_uint(7), None, None, stream)
    torch.cuda.synchronize()
    for r in range(world):
        got = grads[r][r * per:(r + 1) * per].double()
        assert (got - want[r * per:(r + 1) * per]).abs().max() < 1e-5
    shares = torch.stack([p[NORM_WORD0:NORM_WORD0 + world].view(torch.float32) for p in pads])
    assert torch.equal(shares[0], shares[1])  # every pad received the same shares
    want_norm_sq = float(want.pow(2).sum())
    assert abs(float(shares[0].double().sum()) - want_norm_sq) < 1e-4 * want_norm_sq
    seg = (AdamSegment * 1)(AdamSegment(0, per, lr, wd))
    cf = ctypes.c_float
    for r in range(world):
        c = _ctx(r, grads, params, pads)
        _lib.call("db200_comm_adamw", ctypes.byref(c), ctypes.c_longlong(r * per), ctypes.c_longlong(per),
                  _lib.ptr(masters[r]), _lib.ptr(ms[r]), _lib.ptr(vs[r]), seg, ctypes.c_int(1), cf(b1), cf(b2), cf(eps),
                  cf(1.0 / (1 - b1)), cf(1.0 / math.sqrt(1 - b2)), cf(max_norm), ctypes.c_uint(7), _lib.ptr(norm_out), None, None, stream)
    torch.cuda.synchronize()
    _lib.check_status()
    assert abs(float(norm_out) - want_norm_sq) < 1e-4 * want_norm_sq
    coef = min(1.0, max_norm / (math.sqrt(want_norm_sq) + 1e-6))
    for r in range(world):
        g = (want[r * per:(r + 1) * per] * coef).float()
        p = ref_masters[r] * (1 - lr * wd)
        m = g * (1 - b1)
        v = g * g * (1 - b2)
        p = p - lr / (1 - b1) * m / (v.sqrt() / math.sqrt(1 - b2) + eps)
        assert (masters[r] - p).abs().max() < 1e-5
        for q in range(world):  # the bf16 copy landed in every rank's parameter buffer
            assert torch.equal(params[q][r * per:(r + 1) * per], masters[r].to(torch.bfloat16))


def test_emulated_all_reduce_mode_and_vector_sum():
    from deberta_b200.ops import _lib
    from deberta_b200.parallel.peer import PAD_WORDS

    dev = torch.device("cuda")
    world, per = 2, 4096
    n = world * per
    torch.manual_seed(1)
    grads = [torch.randn(n, device=dev) for _ in range(world)]
    params = [torch.zeros(8, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    pads = [torch.zeros(PAD_WORDS, device=dev, dtype=torch.int32) for _ in range(world)]
    for p in pads:
        p[:FLAG_WORDS] = 1000
    want = (grads[0].double() + grads[1].double()) * 0.5
    norm_out = torch.zeros(1, device=dev)
    for r in range(world):
        c = _ctx(r, grads, params, pads)
        _lib.call("db200_comm_reduce", ctypes.byref(c), ctypes.c_longlong(r * per), ctypes.c_longlong(per),
                  ctypes.c_float(0.5), ctypes.c_int(1), ctypes.c_uint(3), None, _lib.ptr(norm_out), _lib.stream_ptr())
    torch.cuda.synchronize()
    for r in range(world):
        assert (grads[r].double() - want).abs().max() < 1e-6
    assert abs(float(norm_out) - float(want.pow(2).sum())) < 1e-3 * float(want.pow(2).sum())
    # vector sum: rank 1 pushed earlier (emulated by running it first), rank 0 then sums both
    for p in pads:
        p[:FLAG_WORDS] = 1000
    vec = [torch.tensor([1.0, 2.0, 3.0], device=dev), torch.tensor([10.0, 20.0, 30.0], device=dev)]
    outs = [torch.zeros(3, device=dev) for _ in range(world)]
    for r in (1, 0):
        c = _ctx(r, grads, params, pads)
        _lib.call("db200_comm_vector_sum", ctypes.byref(c), _lib.ptr(vec[r]), _lib.ptr(outs[r]), ctypes.c_int(3),
                  ctypes.c_uint(4), _lib.stream_ptr())
    torch.cuda.synchronize()
    _lib.check_status()
    assert outs[0].tolist() == [11.0, 22.0, 33.0]


def test_wait_for_absent_peer_times_out_with_status():
    """A flag that nothing raises: the kernel gives up after its time limit and reports through the status word."""
    from deberta_b200.ops import _lib
    from deberta_b200.parallel.peer import PAD_WORDS

    dev = torch.device("cuda")
    grads = [torch.zeros(1024, device=dev) for _ in range(2)]
    params = [torch.zeros(8, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    pads = [torch.zeros(PAD_WORDS, device=dev, dtype=torch.int32) for _ in range(2)]
    _lib.check_status()
    c = _ctx(0, grads, params, pads, timeout_s=0.2)
    out = torch.zeros(4, device=dev)
    _lib.call("db200_comm_vector_sum", ctypes.byref(c), _lib.ptr(grads[0]), _lib.ptr(out), ctypes.c_int(4),
              ctypes.c_uint(1), _lib.stream_ptr())
    torch.cuda.synchronize()  # the context is still usable
    with pytest.raises(_lib.KernelError):
        _lib.check_status()
    _lib.check_status()  # cleared by the read
    assert float(torch.ones(4, device=dev).sum()) == 4.0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("multicast", [False, True])
def test_two_gpu_selftest_matches_nccl(multicast):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533" if multicast else "29534", "-m", "deberta_b200.parallel.comm_selftest",
           "--elems", str(1 << 20)] + ([] if multicast else ["--no-multicast"])
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_full_shard_matches_sharded_optimizer():
    """Parameters gathered layer by layer from the peer's slabs: same losses and masters as with replicated parameters."""
    import json

    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29535", "-m", "deberta_b200.parallel.fsdp_selftest", "--steps", "5"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    row = json.loads([ln for ln in res.stdout.splitlines() if ln.startswith("{")][-1])
    assert row["ok"] and row["fused_collectives"] and row["bytes_from_peers"] > 0
