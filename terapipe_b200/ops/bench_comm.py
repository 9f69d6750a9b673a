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

LINK_GBS = 770.0          # measured peer copy bandwidth per direction


def _measured_peak_tflops(default=1638.7):
    """cuBLAS bf16/fp16 burst throughput measured on this machine pool: read from
    ``MEASURED_PEAKS.json`` at the repository root when present, else the recorded value."""
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"])
    except (OSError, KeyError, ValueError):
        return default


PEAK_TFLOPS = _measured_peak_tflops()


def _max_ms(fn, world, n=20, warm=5):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(6_000_000)  # lets the host run ahead: device time, not launch overhead
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / n], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def link_probe(lib, rank, world, nbytes=148 * 16384 * 64):
    """Every rank stores `nbytes` into the buffer of the next rank (all at once, so both
    directions of every link are busy) and into its own memory, with each store pattern."""
    from ..parallel.symm import SymmetricBuffer
    buf = SymmetricBuffer(nbytes, dist.group.WORLD)
    stream = torch.cuda.current_stream().cuda_stream
    names = {0: "16-byte stores", 1: "16-byte stores + system fence per 32 KB", 2: "16 KB bulk copies from shared memory"}
    for target, tname in ((buf.ptrs[(rank + 1) % world], "next rank"), (buf.ptrs[rank], "own memory")):
        for mode in (0, 1, 2):
            def run():
                check(lib.tp_link_probe(target, nbytes, mode, stream), "tp_link_probe")
            ms = _max_ms(run, world, n=5, warm=2)
            if rank == 0:
                print(json.dumps({"link_probe": names[mode], "target": tname, "MiB": nbytes >> 20,
                                  "us": ms * 1e3, "GB_per_s": nbytes / ms / 1e6}), flush=True)
    buf.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--exchange", action="store_true", help="one-hop exchange instead of reduce-scatter + all-gather")
    ap.add_argument("--probe", action="store_true", help="print in-kernel phase times of the fused kernel")
    ap.add_argument("--link", action="store_true",
                    help="only measure how fast SM-issued stores fill the next rank's memory")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    lib, dt, H, T, tp = cuda_lib(), torch.float16, a.hidden, a.tokens, world
    if a.link:
        link_probe(lib, rank, world)
        dist.destroy_process_group()
        return
    ctx = FusedAllReduceContext(dist.group.WORLD, T, H, pool_bytes=T * H * 2 + 4096)
    out_sym, off = ctx.alloc((T, H), dt)
    epoch_base = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = F.status_word()
    lib.tp_gemm_ar_set_exchange(int(a.exchange))
    probe = torch.zeros(296, 8, dtype=torch.int64, device="cuda") if a.probe else None
    results = []
    calls = [0]  # epochs grow over the whole run: the flags are never cleared
    for name, K in (("out_proj", H // tp), ("fc2", 4 * H // tp)):
        torch.manual_seed(100 + rank)            # every rank its own K shard of x and w
        x = torch.randn(T, K, device="cuda", dtype=dt)
        w = torch.randn(H, K, device="cuda", dtype=dt) * 0.02
        torch.manual_seed(7)                     # bias and residual are replicated
        bias = torch.randn(H, device="cuda", dtype=dt)
        res = torch.randn(T, H, device="cuda", dtype=dt)
        out = torch.empty(T, H, device="cuda", dtype=dt)
        out_ptrs = ctx.out_ptrs(off)

        def fused():
            calls[0] += 1
            st = lib.tp_gemm_ar(0, 0, x.data_ptr(), K, w.data_ptr(), K, H, T, H, K, bias.data_ptr(),
                                res.data_ptr(), H, tp, rank, calls[0], epoch_base.data_ptr(),
                                ctx.max_tiles, ctx.stage_ptrs, ctx.flag_a_ptrs, ctx.flag_b_ptrs,
                                out_ptrs, status.data_ptr(),
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
        phases = None
        if probe is not None:
            lib.tp_gemm_ar_set_debug(probe.data_ptr())
            dist.barrier()
            torch.cuda._sleep(2_000_000)
            for _ in range(3):
                fused()
            torch.cuda.synchronize()
            lib.tp_gemm_ar_set_debug(None)
            t = probe.cpu().double()
            t = t[t[:, 0] > 0]
            t0 = t[:, 0].min()
            lead = t[t[:, 7] > 0]
            phases = {"ctas": int(t.shape[0]),
                      "entry_spread_us": float(t[:, 0].max() - t0) / 1e3,
                      "last_mma_issued_us": float((lead[:, 7] - t0).max()) / 1e3,
                      "own_tiles_published_us": [float((t[:, 1] - t0).median()) / 1e3, float((t[:, 1] - t0).max()) / 1e3],
                      "reductions_done_us": [float((t[:, 2] - t0).median()) / 1e3, float((t[:, 2] - t0).max()) / 1e3],
                      "exit_us": [float((t[:, 3] - t0).median()) / 1e3, float((t[:, 3] - t0).max()) / 1e3],
                      "early_reductions_per_cta": float(t[:, 4].mean()),
                      "publish_stall_us_per_cta": float(t[:, 5].mean()) / 1e3}
        flops = 2.0 * T * H * K
        wire = 2.0 * (tp - 1) / tp * T * H * 2            # partials out + results out, bytes per GPU
        roof_ms = max(flops / (PEAK_TFLOPS * 1e12), wire / (LINK_GBS * 1e9)) * 1e3
        results.append({"gemm": name, "M": T, "N": H, "K": K, "tp": tp, "fused_us": ms_f * 1e3,
                        "gemm_plus_nccl_us": ms_u * 1e3, "roofline_us": roof_ms * 1e3,
                        "fraction_of_roofline": roof_ms / ms_f,
                        "unfused_fraction_of_roofline": roof_ms / ms_u, "rel_err_vs_unfused": err,
                        "compute_bound": flops / (PEAK_TFLOPS * 1e12) > wire / (LINK_GBS * 1e9),
                        "phases": phases})
    F.check_device_status()
    if rank == 0:
        for r in results:
            print(json.dumps(r))
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
