"""Multi-GPU check of the fused collectives against NCCL.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m deberta_b200.parallel.comm_selftest [--elems N] [--no-multicast] [--bench]

Every rank fills its gradient buffer with its own pseudo-random values, runs the slab reduction in both
modes, the slab AdamW and the vector sum, and compares with ``torch.distributed`` collectives and a plain
PyTorch AdamW on the same numbers. ``--bench`` also times the launches with CUDA events (max over ranks).
Exit status 0 means every comparison passed on every rank.
"""

from __future__ import annotations

import argparse
import json
import math
import sys

import torch
import torch.distributed as dist

from ..ops import _lib
from .dist import init_distributed
from .peer import PeerComm


def _time_ms(fn, iters: int = 10) -> float:
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(stop) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--elems", type=int, default=1 << 22)
    ap.add_argument("--no-multicast", action="store_true")
    ap.add_argument("--bench", action="store_true")
    args = ap.parse_args(argv)
    ctx = init_distributed()
    if ctx.world_size < 2 or ctx.device.type != "cuda":
        print("comm_selftest needs at least two GPUs", file=sys.stderr)
        return 2
    world, rank, dev = ctx.world_size, ctx.rank, ctx.device
    n = args.elems // (64 * world) * (64 * world)
    per = n // world
    comm = PeerComm(n, rank=rank, world_size=world, device=dev, use_multicast=not args.no_multicast, timeout_s=5.0)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    src = torch.randn(n, device=dev, generator=gen)
    failures: list[str] = []

    def close(name: str, got: torch.Tensor, want: torch.Tensor, tol: float) -> None:
        err = float((got.double() - want.double()).abs().max())
        ref = float(want.double().abs().max()) + 1e-12
        if not (err <= tol * ref):
            failures.append(f"{name}: max err {err:.3e} vs scale {ref:.3e}")

    want = src.clone()
    dist.all_reduce(want)
    want /= world
    want_norm = want.double().pow(2).sum()

    # ---- reduce-scatter + norm share, then AdamW + parameter all-gather ---------------------------
    comm.grads.copy_(src)
    master = torch.randn(per, device=dev, generator=gen)
    m0, v0 = torch.zeros(per, device=dev), torch.zeros(per, device=dev)
    ref_p, ref_m, ref_v = master.clone(), m0.clone(), v0.clone()
    norm_out = torch.zeros(1, device=dev)
    dist.barrier()
    e = comm.reduce(rank * per, per, scale=1.0 / world, to_all=False, extra_share=None, norm_sq_out=None)
    lr, wd, b1, b2, eps, max_norm = 1e-2, 0.1, 0.9, 0.999, 1e-6, 1.0
    half = per // 2 // 8 * 8
    comm.adamw(rank * per, per, master=master, exp_avg=m0, exp_avg_sq=v0,
               segments=[(0, half, lr, wd), (half, per, lr, 0.0)], betas=(b1, b2), eps=eps, inv_bc1=1.0 / (1 - b1),
               inv_sqrt_bc2=1.0 / math.sqrt(1 - b2), max_norm=max_norm, epoch=e, norm_sq_out=norm_out)
    torch.cuda.synchronize()
    close("reduce_scatter", comm.grads[rank * per:(rank + 1) * per], want[rank * per:(rank + 1) * per], 1e-5)
    close("norm", norm_out.double(), want_norm.reshape(1), 1e-4)
    coef = min(1.0, max_norm / (float(want_norm.sqrt()) + 1e-6))
    g = want[rank * per:(rank + 1) * per] * coef
    decay = torch.ones(per, device=dev)
    decay[:half] = 1 - lr * wd
    ref_p *= decay
    ref_m.lerp_(g, 1 - b1)
    ref_v.mul_(b2).addcmul_(g, g, value=1 - b2)
    ref_p -= lr / (1 - b1) * ref_m / (ref_v.sqrt() / math.sqrt(1 - b2) + eps)
    close("adamw_master", master, ref_p, 1e-5)
    gathered = [torch.empty(per, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    dist.all_gather(gathered, ref_p.to(torch.bfloat16))
    close("param_all_gather", comm.params.float(), torch.cat(gathered).float(), 1e-2)

    # ---- all-reduce mode ---------------------------------------------------------------------------
    comm.grads.copy_(src)
    dist.barrier()
    comm.reduce(rank * per, per, scale=1.0 / world, to_all=True, extra_share=None, norm_sq_out=norm_out)
    torch.cuda.synchronize()
    close("all_reduce", comm.grads, want, 1e-5)
    close("all_reduce_norm", norm_out.double(), want_norm.reshape(1), 1e-4)

    # ---- non-finite share makes every rank skip ----------------------------------------------------
    comm.grads.copy_(src)
    before = master.clone()
    pen = torch.tensor([float("inf") if rank == world - 1 else 0.0], device=dev)
    dist.barrier()
    e = comm.reduce(rank * per, per, scale=1.0 / world, to_all=False, extra_share=pen, norm_sq_out=None)
    comm.adamw(rank * per, per, master=master, exp_avg=m0, exp_avg_sq=v0, segments=[(0, per, lr, wd)], betas=(b1, b2),
               eps=eps, inv_bc1=1.0, inv_sqrt_bc2=1.0, max_norm=max_norm, epoch=e, norm_sq_out=norm_out)
    torch.cuda.synchronize()
    if not torch.equal(before, master) or math.isfinite(float(norm_out)):
        failures.append("non-finite share did not skip the update")

    # ---- vector sum --------------------------------------------------------------------------------
    vec = torch.arange(7, device=dev, dtype=torch.float32) * (rank + 1)
    for _ in range(3):
        got = comm.vector_sum(vec)
    wantv = vec.clone()
    dist.all_reduce(wantv)
    close("vector_sum", got, wantv, 1e-6)

    _lib.check_status()
    report = {"rank": rank, "world": world, "elems": n, "multicast": comm.multicast, "failures": failures}
    if args.bench:
        def fused():
            ee = comm.reduce(rank * per, per, scale=1.0 / world, to_all=False, extra_share=None, norm_sq_out=None)
            comm.adamw(rank * per, per, master=master, exp_avg=m0, exp_avg_sq=v0, segments=[(0, per, lr, wd)],
                       betas=(b1, b2), eps=eps, inv_bc1=1.0, inv_sqrt_bc2=1.0, max_norm=0.0, epoch=ee, norm_sq_out=norm_out)

        shard = torch.empty(per, device=dev)
        full_bf16 = torch.empty(n, device=dev, dtype=torch.bfloat16)
        scratch = torch.zeros(1, device=dev)

        def nccl():
            dist.reduce_scatter_tensor(shard, comm.grads, op=dist.ReduceOp.AVG)
            scratch.zero_()
            _lib.call("db200_sumsq", _lib.ptr(shard), __import__("ctypes").c_longlong(per), _lib.ptr(scratch), _lib.stream_ptr())
            dist.all_reduce(scratch)
            master.mul_(1.0)  # stands in for the AdamW pass (same bytes moved)
            dist.all_gather_into_tensor(full_bf16, full_bf16[rank * per:(rank + 1) * per])

        report["fused_ms"] = _time_ms(fused)
        report["nccl_ms"] = _time_ms(nccl)
        report["all_reduce_fused_ms"] = _time_ms(
            lambda: comm.reduce(rank * per, per, scale=1.0, to_all=True, extra_share=None, norm_sq_out=norm_out))
        report["all_reduce_nccl_ms"] = _time_ms(lambda: dist.all_reduce(comm.grads))
        report["vector_sum_ms"] = _time_ms(lambda: comm.vector_sum(vec), iters=50)
        report["nccl_small_all_reduce_ms"] = _time_ms(lambda: dist.all_reduce(wantv), iters=50)
        _lib.check_status()
    bad = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(bad)
    if rank == 0 or failures:
        print(json.dumps(report), flush=True)
    dist.barrier()
    ctx.shutdown()
    return 0 if int(bad) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
