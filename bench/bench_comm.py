"""Roofline check of the fused GEMM + tensor-parallel collective kernels (run with torchrun).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \\
        bench/bench_comm.py --hidden 5120 --tokens 1024 [--peak-tflops 1638.7]

For the two row-parallel products of a layer (attention output projection and FFN down
projection) it times, with CUDA events and the maximum over ranks,
  (a) ``tp_gemm_rs``: GEMM -> reduce-scatter in one kernel (partial tiles pushed to the rank
      that owns the rows, summed there inside the epilogue),
  (b) ``tp_gemm_ar``: GEMM + all-reduce in one kernel (reduce-scatter, then the result pushed to
      every rank),
  (c) the unfused pairs: the same tcgen05 GEMM followed by NCCL reduce-scatter / all-reduce,
and for the column-parallel products (QKV and FFN up projection)
  (d) ``tp_layernorm_fwd_push`` + ``tp_gemm_ag``: the LayerNorm of the local token shard pushed to
      every rank, and the GEMM that waits for the peers' rows inside its producer warp,
  (e) LayerNorm of the shard + NCCL all-gather + the plain GEMM,
and prints the achieved fraction of the roofline
``max(FLOPs / GEMM peak, NVLink bytes per GPU / link bandwidth)``.  ``--peak-tflops`` is the
measured dense 16-bit GEMM throughput of the machine (default: the value measured on a B200 of
this pool); ``--link-gbs`` the measured peer-copy bandwidth per direction.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from terapipe_b200.ops import functional as F                    # noqa: E402
from terapipe_b200.ops.lib import check, cuda_lib                # noqa: E402
from terapipe_b200.parallel.symm import FusedAllReduceContext    # noqa: E402


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
    from terapipe_b200.parallel.symm import SymmetricBuffer
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


class Ctx:
    """Buffers and flags shared by the measured calls (one tensor-parallel group = the world)."""

    def __init__(self, T, H, args):
        self.rank, self.tp = dist.get_rank(), dist.get_world_size()
        self.T, self.H, self.dt = T, H, torch.float16
        self.lib = cuda_lib()
        pool = 3 * (T * H * 2 + 256) + 65536
        self.ar = FusedAllReduceContext(dist.group.WORLD, T, H, pool_bytes=pool)
        self.out_sym, self.out_off = self.ar.alloc((T, H), self.dt)       # all-reduce result
        self.ln_sym, self.ln_off = self.ar.alloc((T, H), self.dt)         # all-gathered LayerNorm output
        self.ag_flags, self.ag_flags_off = self.ar.alloc((16,), torch.int32)
        self.ag_flag_ptrs = self.ar.out_ptrs(self.ag_flags_off)
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.status = F.status_word()
        self.calls = 0      # epochs grow over the whole run: the flags are never cleared
        self.ag_calls = 0
        self.peak, self.link = args.peak_tflops, args.link_gbs

    def stream(self):
        return torch.cuda.current_stream().cuda_stream

    def roof_ms(self, flops, wire_bytes):
        return max(flops / (self.peak * 1e12), wire_bytes / (self.link * 1e9)) * 1e3


def bench_row_parallel(c: Ctx, name, K, probe=None):
    """out = sum over ranks of x_r @ w_r^T (+ bias + residual): reduce-scatter and all-reduce forms."""
    lib, T, H, tp, rank, dt = c.lib, c.T, c.H, c.tp, c.rank, c.dt
    torch.manual_seed(100 + rank)            # every rank its own K shard of x and w
    x = torch.randn(T, K, device="cuda", dtype=dt)
    w = torch.randn(H, K, device="cuda", dtype=dt) * 0.02
    torch.manual_seed(7)                     # bias and residual are replicated
    bias = torch.randn(H, device="cuda", dtype=dt)
    res = torch.randn(T, H, device="cuda", dtype=dt)
    out = torch.empty(T, H, device="cuda", dtype=dt)
    out_rs = torch.zeros(T, H, device="cuda", dtype=dt)
    rpr = T // tp
    shard = torch.empty(rpr, H, device="cuda", dtype=dt)
    out_ptrs = c.ar.out_ptrs(c.out_off)

    def fused_ar():
        c.calls += 1
        check(lib.tp_gemm_ar(0, 0, x.data_ptr(), K, w.data_ptr(), K, H, T, H, K, bias.data_ptr(),
                             res.data_ptr(), H, tp, rank, c.calls, c.epoch_base.data_ptr(),
                             c.ar.max_tiles, c.ar.stage_ptrs, c.ar.flag_a_ptrs, c.ar.flag_b_ptrs,
                             out_ptrs, c.status.data_ptr(), c.stream()), "tp_gemm_ar")

    def fused_rs():
        c.calls += 1
        check(lib.tp_gemm_rs(0, 0, x.data_ptr(), K, w.data_ptr(), K, out_rs.data_ptr(), H, T, H, K,
                             bias.data_ptr(), res.data_ptr(), H, tp, rank, rpr, c.calls,
                             c.epoch_base.data_ptr(), c.ar.max_tiles, c.ar.stage_ptrs,
                             c.ar.flag_a_ptrs, c.status.data_ptr(), c.stream()), "tp_gemm_rs")

    def unfused_ar():
        F.gemm(x, w, out, bias=bias if rank == 0 else None, residual=res if rank == 0 else None)
        dist.all_reduce(out)

    def unfused_rs():
        F.gemm(x, w, out, bias=bias if rank == 0 else None, residual=res if rank == 0 else None)
        dist.reduce_scatter_tensor(shard, out)

    def gemm_only():
        F.gemm(x, w, out, bias=bias, residual=res)

    fused_ar()
    fused_rs()
    unfused_ar()
    torch.cuda.synchronize()
    ref = out.float()
    err_ar = ((c.out_sym.float() - ref).norm() / ref.norm()).item()
    mine = slice(rank * rpr, (rank + 1) * rpr)
    err_rs = ((out_rs[mine].float() - ref[mine]).norm() / ref[mine].norm()).item()
    ms = {"rs": _max_ms(fused_rs, tp), "ar": _max_ms(fused_ar, tp), "gemm": _max_ms(gemm_only, tp),
          "gemm_nccl_rs": _max_ms(unfused_rs, tp), "gemm_nccl_ar": _max_ms(unfused_ar, tp)}
    flops = 2.0 * T * H * K
    wire_rs = (tp - 1) / tp * T * H * 2              # partials out, bytes per GPU
    wire_ar = 2.0 * wire_rs                          # + results out
    roof_rs, roof_ar = c.roof_ms(flops, wire_rs), c.roof_ms(flops, wire_ar)
    return {"gemm": name, "M": T, "N": H, "K": K, "tp": tp,
            "roofline_us": {"rs": roof_rs * 1e3, "ar": roof_ar * 1e3},
            "us": {k: v * 1e3 for k, v in ms.items()},
            "fraction_of_roofline": {"rs": roof_rs / ms["rs"], "ar": roof_ar / ms["ar"],
                                     "gemm_alone_vs_compute": flops / (c.peak * 1e12) * 1e3 / ms["gemm"],
                                     "gemm_nccl_rs": roof_rs / ms["gemm_nccl_rs"],
                                     "gemm_nccl_ar": roof_ar / ms["gemm_nccl_ar"]},
            "rel_err_vs_unfused": {"rs": err_rs, "ar": err_ar}}


def bench_column_parallel(c: Ctx, name, N):
    """y = LayerNorm(x) over all T rows (each rank normalises T / tp of them), then y @ w^T + b:
    push + waiting GEMM against NCCL all-gather + GEMM."""
    lib, T, H, tp, rank, dt = c.lib, c.T, c.H, c.tp, c.rank, c.dt
    rpr = T // tp
    torch.manual_seed(3)
    x = torch.randn(T, H, device="cuda", dtype=dt)                # the full residual stream
    gamma = (1 + 0.1 * torch.randn(H, device="cuda")).to(dt)
    beta = (0.1 * torch.randn(H, device="cuda")).to(dt)
    torch.manual_seed(200 + rank)
    w = torch.randn(N, H, device="cuda", dtype=dt) * 0.02          # this rank's output columns
    b = torch.randn(N, device="cuda", dtype=dt)
    y = torch.empty(T, N, device="cuda", dtype=dt)
    y_ref = torch.empty(T, N, device="cuda", dtype=dt)
    mean = torch.empty(T, device="cuda")
    rstd = torch.empty(T, device="cuda")
    ln_shard = torch.empty(rpr, H, device="cuda", dtype=dt)
    ln_full = torch.empty(T, H, device="cuda", dtype=dt)
    m0 = rank * rpr
    dst_ptrs = c.ar.out_ptrs(c.ln_off + m0 * H * 2)

    def pushed():
        c.ag_calls += 1
        check(lib.tp_layernorm_fwd_push(0, x[m0:].data_ptr(), gamma.data_ptr(), beta.data_ptr(), dst_ptrs,
                                        mean[m0:].data_ptr(), rstd[m0:].data_ptr(), rpr, H, 1e-5, tp, rank,
                                        c.ag_flag_ptrs, c.ag_calls, None, c.counter.data_ptr(), c.stream()),
              "tp_layernorm_fwd_push")
        check(lib.tp_gemm_ag(0, 0, c.ln_sym.data_ptr(), H, w.data_ptr(), H, y.data_ptr(), N, T, N, H,
                             b.data_ptr(), 0, None, 0, None, 0, c.ag_flags.data_ptr(), None, c.ag_calls,
                             rpr, rank, c.status.data_ptr(), c.stream()), "tp_gemm_ag")

    side = torch.cuda.Stream()
    local_dst = c.ln_sym[m0:m0 + rpr]

    def copied():
        # LayerNorm writes its shard locally; copy engines carry it to the peers on a side stream
        # while the GEMM already works on this rank's own row blocks
        c.ag_calls += 1
        F.layernorm_fwd(x[m0:m0 + rpr], gamma, beta, local_dst, mean[m0:m0 + rpr], rstd[m0:m0 + rpr])
        side.wait_stream(torch.cuda.current_stream())
        check(lib.tp_ag_copy(local_dst.data_ptr(), rpr * H * 2, dst_ptrs, c.ag_flag_ptrs, tp, rank,
                             c.ag_calls, None, side.cuda_stream), "tp_ag_copy")
        check(lib.tp_gemm_ag(0, 0, c.ln_sym.data_ptr(), H, w.data_ptr(), H, y.data_ptr(), N, T, N, H,
                             b.data_ptr(), 0, None, 0, None, 0, c.ag_flags.data_ptr(), None, c.ag_calls,
                             rpr, rank, c.status.data_ptr(), c.stream()), "tp_gemm_ag")
        torch.cuda.current_stream().wait_stream(side)

    def gathered():
        F.layernorm_fwd(x[m0:m0 + rpr], gamma, beta, ln_shard, mean[m0:m0 + rpr], rstd[m0:m0 + rpr])
        dist.all_gather_into_tensor(ln_full, ln_shard)
        F.gemm(ln_full, w, y_ref, bias=b)

    def local_only():
        F.layernorm_fwd(x[m0:m0 + rpr], gamma, beta, ln_shard, mean[m0:m0 + rpr], rstd[m0:m0 + rpr])
        F.gemm(ln_full, w, y_ref, bias=b)

    pushed()
    gathered()
    torch.cuda.synchronize()
    err = ((y.float() - y_ref.float()).norm() / y_ref.float().norm()).item()
    y.zero_()
    copied()
    torch.cuda.synchronize()
    err_copy = ((y.float() - y_ref.float()).norm() / y_ref.float().norm()).item()
    err = max(err, err_copy)
    ms = {"copy_ag_gemm": _max_ms(copied, tp), "push_ag_gemm": _max_ms(pushed, tp),
          "ln_gemm_no_comm": _max_ms(local_only, tp),
          "ln_nccl_ag_gemm": _max_ms(gathered, tp)}
    flops = 2.0 * T * N * H
    wire = (tp - 1) * rpr * H * 2                  # this rank's shard to every peer
    roof = c.roof_ms(flops, wire)
    return {"gemm": name, "M": T, "N": N, "K": H, "tp": tp, "roofline_us": roof * 1e3,
            "us": {k: v * 1e3 for k, v in ms.items()},
            "fraction_of_roofline": {k: roof / v for k, v in ms.items()}, "rel_err_vs_unfused": err}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--peak-tflops", type=float, default=1638.7,
                    help="measured dense 16-bit GEMM throughput of the machine")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="measured peer copy bandwidth per direction")
    ap.add_argument("--exchange", action="store_true", help="all-reduce kernel: one-hop exchange form")
    ap.add_argument("--link", action="store_true",
                    help="only measure how fast SM-issued stores fill the next rank's memory")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    lib = cuda_lib()
    if a.link:
        link_probe(lib, rank, world)
        dist.destroy_process_group()
        return
    H, T, tp = a.hidden, a.tokens, world
    lib.tp_gemm_ar_set_exchange(int(a.exchange))
    c = Ctx(T, H, a)
    results = [bench_row_parallel(c, "out_proj", H // tp), bench_row_parallel(c, "fc2", 4 * H // tp),
               bench_column_parallel(c, "qkv", 3 * H // tp), bench_column_parallel(c, "fc1", 4 * H // tp)]
    F.check_device_status()
    if rank == 0:
        for r in results:
            print(json.dumps(r), flush=True)
    dist.barrier()
    c.ar.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
