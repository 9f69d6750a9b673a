"""Micro-benchmarks of the sm_100a kernels at the GPT-3 layer shapes (CUDA-event timing).

    python bench/bench_ops.py --case gemm  [--hidden 2048] [--tokens 1024]
    python bench/bench_ops.py --case attn  [--ctx 1920] [--slice 128]
    python bench/bench_ops.py --case norm
    python bench/bench_ops.py --case adam

``--once`` runs each kernel a few times without timing (a small, self-terminating workload
for profiler captures).  Between timed kernels a 256 MB buffer is rewritten to flush the L2
when ``--flush`` is given; otherwise launches run back to back (warm L2).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from terapipe_b200.ops import functional as F  # noqa: E402


def _timeit(fn, n=20, warm=3, flush=None):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if flush is None:
        torch.cuda._sleep(3_000_000)  # lets the host run ahead so launch overhead is not timed
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3
    for _ in range(n):
        flush.zero_()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / n * 1e3


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def case_gemm(a):
    """Layer GEMMs of one token slice.  ``--tile`` takes a comma list of tile codes to force
    (0 = automatic choice, 64/128/256 = one CTA with a 128 x BN tile, 512 = one CTA 256 x 256,
    1128/1256 = CTA pair with a 256 x 128 / 256 x 256 tile); every forced run is also checked
    against torch."""
    dt, dev, H, T = a.dtype, "cuda", a.hidden, a.tokens
    tiles = [int(t) for t in a.tile.split(",")]
    shapes = {"qkv": (T, 3 * H, H), "out": (T, H, H), "fc1": (T, 4 * H, H), "fc2": (T, H, 4 * H)}
    for name, (M, N, K) in shapes.items():
        x = torch.randn(M, K, device=dev, dtype=dt)
        w = torch.randn(N, K, device=dev, dtype=dt) * 0.02
        bias = torch.zeros(N, device=dev, dtype=dt)
        out = torch.empty(M, N, device=dev, dtype=dt)
        dy = torch.randn(M, N, device=dev, dtype=dt)
        dx = torch.empty(M, K, device=dev, dtype=dt)
        if a.once:
            for _ in range(3):
                F.gemm(x, w, out, bias=bias, force_bn=tiles[0])
            continue
        ref = _timeit(lambda: torch.nn.functional.linear(x, w, bias), flush=a.flush_buf)
        y_ref = torch.nn.functional.linear(x, w, bias)
        dx_ref = dy @ w
        for tile in tiles:
            out.fill_(float("nan"))
            us = _timeit(lambda: F.gemm(x, w, out, bias=bias, force_bn=tile), flush=a.flush_buf)
            err = _rel(out, y_ref)
            print(f"gemm {name:4s} M{M} N{N} K{K} tile {tile:4d}: {us:7.1f} us "
                  f"{2 * M * N * K / us / 1e6:7.1f} TFLOP/s  rel.err {err:.1e}   (torch/cuBLAS {ref:7.1f} us)")
            dx.fill_(float("nan"))
            us = _timeit(lambda: F.gemm(dy, w, dx, b_mn=True, force_bn=tile), flush=a.flush_buf)
            err = _rel(dx, dx_ref)
            print(f"  dgrad                     tile {tile:4d}: {us:7.1f} us "
                  f"{2 * M * N * K / us / 1e6:7.1f} TFLOP/s  rel.err {err:.1e}")
        F.check_device_status()
    if not a.once:
        R = 16 * T
        dy = torch.randn(R, 4 * H, device=dev, dtype=dt)
        x = torch.randn(R, H, device=dev, dtype=dt)
        dw = torch.zeros(4 * H, H, device=dev)
        for tile in tiles:
            us = _timeit(lambda: F.gemm(dy, x, dw, a_mn=True, b_mn=True, accumulate=True, force_bn=tile), n=5)
            dw.zero_()
            F.gemm(dy, x, dw, a_mn=True, b_mn=True, accumulate=True, force_bn=tile)
            err = _rel(dw, dy.float().t() @ x.float())
            print(f"wgrad fc1 over {R} rows tile {tile:4d}: {us:7.1f} us "
                  f"{2 * R * 4 * H * H / us / 1e6:7.1f} TFLOP/s  rel.err {err:.1e}")
        F.check_device_status()


def case_gemm_trace(a):
    """Where the cycles of the CTA-pair GEMM go: per-phase medians over CTAs."""
    dt, dev, H, T = torch.float16, "cuda", a.hidden, a.tokens
    shapes = {"qkv": (T, 3 * H, H), "out": (T, H, H), "fc1": (T, 4 * H, H), "fc2": (T, H, 4 * H)}
    for name, (M, N, K) in shapes.items():
        x = torch.randn(M, K, device=dev, dtype=dt)
        w = torch.randn(N, K, device=dev, dtype=dt) * 0.02
        out = torch.empty(M, N, device=dev, dtype=dt)
        for bn in (128, 256):
            for _ in range(3):
                tr = F.gemm_pair_trace(x, w, out, bn)
            if a.flush_buf is not None:
                a.flush_buf.zero_()
                tr = F.gemm_pair_trace(x, w, out, bn)
            torch.cuda.synchronize()
            tr = tr.cpu().double()
            lead = tr[0::2]
            t0 = tr[:, 0:1]
            rel = tr - t0
            med = lambda v: float(v.median())  # noqa: E731
            mx = lambda v: float(v.max())  # noqa: E731
            tiles = lead[:, 8]
            ideal = (K // 16) * (bn // 2)      # MMA cycles of one tile at the full rate
            print(f"trace {name} M{M} N{N} K{K} pair tile 256x{bn}: CTAs {tr.shape[0]}, tiles/pair "
                  f"{int(tiles.min())}-{int(tiles.max())}, MMA cycles per tile at full rate {ideal}")
            print(f"  set-up done            median {med(rel[:, 1]):8.0f}  max {mx(rel[:, 1]):8.0f}")
            print(f"  first operands arrived median {med(lead[:, 4] - lead[:, 0]):8.0f}  max {mx(lead[:, 4] - lead[:, 0]):8.0f}")
            print(f"  last MMA issued        median {med(lead[:, 7] - lead[:, 0]):8.0f}  max {mx(lead[:, 7] - lead[:, 0]):8.0f}")
            print(f"    of which waiting for operands {med(lead[:, 5]):8.0f} (max {mx(lead[:, 5]):8.0f}), "
                  f"for a free accumulator {med(lead[:, 6]):8.0f} (max {mx(lead[:, 6]):8.0f})")
            print(f"  producer waited for ring slots  median {med(tr[:, 2]):8.0f}; last load issued at {med(rel[:, 3]):8.0f}")
            print(f"  last accumulator ready median {med(rel[:, 10]):8.0f}  max {mx(rel[:, 10]):8.0f}")
            print(f"  last store issued      median {med(rel[:, 12]):8.0f}  max {mx(rel[:, 12]):8.0f}")
            print(f"  kernel exit            median {med(rel[:, 13]):8.0f}  max {mx(rel[:, 13]):8.0f}")
            print(f"  epilogue warp: TMEM loads {med(tr[:, 14]):8.0f}, math + stores {med(tr[:, 15]):8.0f}, "
                  f"waiting for accumulators {med(tr[:, 11]):8.0f}")
            print(f"    math + stores = buffer wait {med(tr[:, 16]):8.0f} + math/smem {med(tr[:, 17]):8.0f} "
                  f"+ fence/issue {med(tr[:, 18]):8.0f}; first TMEM load of each tile: wait returns after "
                  f"{med(tr[:, 19]):6.0f}, register readable after {med(tr[:, 20]):6.0f} more")
        F.check_device_status()


def case_attn(a):
    dt, dev, H = a.dtype, "cuda", a.hidden
    D, b, L, t = 128, a.batch, a.seq, a.slice
    h = H // D
    qkv = torch.randn(L, b, h * 3 * D, device=dev, dtype=dt)
    o = torch.zeros(L * b, h * D, device=dev, dtype=dt)
    lse = torch.zeros(b * h, L, device=dev)
    delta = torch.zeros(b * h, L, device=dev)
    dof = torch.randn(L * b, h * D, device=dev, dtype=dt)
    dqkv = torch.zeros(t * b, h * 3 * D, device=dev, dtype=dt)
    for c in ([a.ctx] if a.ctx is not None else [0, L // 2 - t, L - t]):
        osl = o[c * b:(c + t) * b]
        fwd = lambda: F.attn_fwd(qkv, b, h, D, t, c, osl, lse)  # noqa: E731
        bwd = lambda: F.attn_bwd(qkv, b, h, D, t, c, L, osl, dof, lse, delta, dqkv)  # noqa: E731
        if a.once:
            for _ in range(2):
                fwd()
                bwd()
            continue
        fl = 4.0 * b * h * t * (c + t) * D
        us = _timeit(fwd, flush=a.flush_buf)
        print(f"attn fwd ctx={c:5d} slice={t}: {us:7.1f} us {fl / us / 1e6:7.1f} TFLOP/s")
        us = _timeit(bwd, flush=a.flush_buf)
        print(f"attn bwd ctx={c:5d} (dK/dV over {L - c} queries, dQ over {c + t} keys): {us:7.1f} us")


def case_norm(a):
    dt, dev, H, T = a.dtype, "cuda", a.hidden, a.tokens
    x = torch.randn(T, H, device=dev, dtype=dt)
    g = torch.ones(H, device=dev, dtype=dt)
    bb = torch.zeros(H, device=dev, dtype=dt)
    y = torch.empty_like(x)
    mean, rstd = torch.empty(T, device=dev), torch.empty(T, device=dev)
    dg, db = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
    sc = torch.empty(F.layernorm_bwd_scratch_floats(T, H), device=dev)
    dx = torch.empty_like(x)
    fwd = lambda: F.layernorm_fwd(x, g, bb, y, mean, rstd)  # noqa: E731
    bwd = lambda: F.layernorm_bwd(y, x, mean, rstd, g, dx, dg, db, sc, dres=x)  # noqa: E731
    if a.once:
        for _ in range(3):
            fwd()
            bwd()
        return
    print(f"layernorm fwd [{T},{H}]: {_timeit(fwd, flush=a.flush_buf):6.1f} us")
    print(f"layernorm bwd [{T},{H}]: {_timeit(bwd, flush=a.flush_buf):6.1f} us")


def case_adam(a):
    n = a.params // 4 * 4
    dev = "cuda"
    p, m, v, g = (torch.zeros(n, device=dev) for _ in range(4))
    model = torch.zeros(n, device=dev, dtype=a.dtype)
    st = torch.ones(3, device=dev)
    run = lambda: F.fused_adam(g, p, m, v, model, st, lr=1e-3)  # noqa: E731
    if a.once:
        run()
        return
    us = _timeit(run, n=5)
    print(f"fused adam {n / 1e6:.0f}M params: {us:8.1f} us {n * 34 / us / 1e3:7.0f} GB/s")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["gemm", "gemm-trace", "attn", "norm", "adam"])
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--slice", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--params", type=int, default=302_000_000)
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--tile", default="0", help="gemm: comma list of tile codes to force")
    ap.add_argument("--prefetch", type=int, default=None,
                    help="gemm: L2 prefetch distance of the CTA-pair kernel in k-steps (0 = off)")
    ap.add_argument("--once", action="store_true")
    ap.add_argument("--flush", action="store_true")
    a = ap.parse_args()
    a.dtype = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    if a.prefetch is not None:
        from .lib import cuda_lib
        cuda_lib().tp_gemm_set_prefetch(a.prefetch)
    a.flush_buf = torch.empty(256 * 1024 * 1024, device="cuda", dtype=torch.uint8) if a.flush else None
    {"gemm": case_gemm, "gemm-trace": case_gemm_trace, "attn": case_attn, "norm": case_norm, "adam": case_adam}[a.case](a)
    torch.cuda.synchronize()
    F.check_device_status()


if __name__ == "__main__":
    main()
