"""Roofline check of the fused GEMM + tensor-parallel all-reduce kernel (run with torchrun).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m terapipe_b200.ops.bench_comm --hidden 5120 --tokens 1024

For the two row-parallel products of a layer (attention output projection and FFN down
projection) it times, with CUDA events and the maximum over ranks,
  (a) the fused kernel (``tp_gemm_ar``: partial tiles pushed to their owner over NVLink,
      reduced, result pushed to every rank), and
  (b) the unfused pair: the same tcgen05 GEMM followed by an NCCL all-reduce,
and prints the achieved fraction of the roofline
``max(FLOPs / measured GEMM peak, NVLink bytes per GPU / 770 GB/s)``.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..parallel.symm import FusedAllReduceContext
from . import functional as F
from .lib import check, cuda_lib

PEAK_TFLOPS = 1638.7      # measured cuBLAS bf16/fp16 burst on this pool (MEASURED_PEAKS.json)
LINK_GBS = 770.0          # measured peer copy bandwidth per direction


def _max_ms(fn, world, n=20, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / n], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--tokens", type=int, default=1024)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    lib, dt, H, T, tp = cuda_lib(), torch.float16, a.hidden, a.tokens, world
    ctx = FusedAllReduceContext(dist.group.WORLD, T, H, pool_bytes=T * H * 2 + 4096)
    out_sym, off = ctx.alloc((T, H), dt)
    epoch_base = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = F.status_word()
    results = []
    for name, K in (("out_proj", H // tp), ("fc2", 4 * H // tp)):
        x = torch.randn(T, K, device="cuda", dtype=dt)
        w = torch.randn(H, K, device="cuda", dtype=dt) * 0.02
        bias = torch.zeros(H, device="cuda", dtype=dt)
        res = torch.randn(T, H, device="cuda", dtype=dt)
        out = torch.empty(T, H, device="cuda", dtype=dt)
        calls = [0]

        def fused():
            calls[0] += 1
            st = lib.tp_gemm_ar(0, 0, x.data_ptr(), K, w.data_ptr(), K, H, T, H, K, bias.data_ptr(),
                                res.data_ptr(), H, tp, rank, calls[0], epoch_base.data_ptr(),
                                ctx.max_tiles, ctx.stage_ptrs, ctx.flag_a_ptrs, ctx.flag_b_ptrs,
                                ctx.out_ptrs(off), status.data_ptr(),
                                torch.cuda.current_stream().cuda_stream)
            check(st, "tp_gemm_ar")

        def unfused():
            F.gemm(x, w, out, bias=bias if rank == 0 else None, residual=res if rank == 0 else None)
            dist.all_reduce(out)

        # correctness of the fused result against the unfused one, then timing
        fused()
        unfused()
        torch.cuda.synchronize()
        err = ((out_sym.float() - out.float()).norm() / out.float().norm()).item()
        ms_f = _max_ms(fused, world)
        epoch_base += 0  # keep tensor alive; epochs keep growing through `calls`
        ms_u = _max_ms(unfused, world)
        flops = 2.0 * T * H * K
        wire = 2.0 * (tp - 1) / tp * T * H * 2            # partials out + results out, bytes per GPU
        roof_ms = max(flops / (PEAK_TFLOPS * 1e12), wire / (LINK_GBS * 1e9)) * 1e3
        results.append({"gemm": name, "M": T, "N": H, "K": K, "tp": tp, "fused_us": ms_f * 1e3,
                        "gemm_plus_nccl_us": ms_u * 1e3, "roofline_us": roof_ms * 1e3,
                        "fraction_of_roofline": roof_ms / ms_f, "rel_err_vs_unfused": err,
                        "compute_bound": flops / (PEAK_TFLOPS * 1e12) > wire / (LINK_GBS * 1e9)})
    F.check_device_status()
    if rank == 0:
        for r in results:
            print(json.dumps(r))
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
