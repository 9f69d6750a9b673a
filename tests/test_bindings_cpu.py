"""The ctypes signature table must match the `extern "C"` definitions of the kernel sources:
a drifted argument list corrupts a launch silently."""
import re
from pathlib import Path

from terapipe_b200.ops import lib

CSRC = Path(lib.__file__).resolve().parent / "csrc"
# declared by hand next to their only caller (pointer-returning or byte-buffer arguments)
DECLARED_ELSEWHERE = {"tp_symm_alloc", "tp_symm_free", "tp_ipc_export", "tp_ipc_import", "tp_ipc_close",
                      "tp_layernorm_bwd_noalloc", "tp_layernorm_bwd_noalloc_capacity"}


def _c_entry_points():
    out = {}
    pat = re.compile(r'extern\s+"C"\s+([\w\s\*]+?)\s*\b(tp_\w+)\s*\(([^)]*)\)\s*\{', re.S)
    for src in sorted(CSRC.glob("*.cu")):
        for ret, name, params in pat.findall(src.read_text()):
            params = " ".join(params.split())
            args = [] if params in ("", "void") else [a.strip() for a in params.split(",")]
            out[name] = (ret.strip(), args, src.name)
    return out


def _code(c_param: str) -> str:
    if "*" in c_param:
        return "P"
    if "long long" in c_param:
        return "L"
    if re.match(r"(const\s+)?float\b", c_param):
        return "F"
    if re.match(r"(const\s+)?int\b", c_param):
        return "I"
    raise AssertionError(f"unexpected parameter type: {c_param!r}")


def test_every_entry_point_is_declared_with_the_right_arguments():
    names = {lib.P: "P", lib.I: "I", lib.L: "L", lib.F: "F"}
    entries = _c_entry_points()
    assert len(entries) >= 20
    for name, (ret, args, src) in entries.items():
        if name in DECLARED_ELSEWHERE:
            continue
        assert name in lib.SIGNATURES, f"{name} ({src}) has no ctypes signature"
        want = "".join(_code(a) for a in args)
        have = "".join(names[t] for t in lib.SIGNATURES[name])
        assert have == want, f"{name} ({src}): table {have}, source {want}"
    for name in lib.SIGNATURES:
        assert name in entries, f"{name} is in the table but not defined in csrc/*.cu"


def test_regular_and_checked_builds_export_the_same_entry_points():
    """The checked library (-DTP_CHECKED) is the regular one plus index checks: both load without
    a GPU, say which build they are, and export every entry point of the signature table."""
    import ctypes

    from terapipe_b200.ops import build
    from terapipe_b200.ops.lib import SIGNATURES
    build.build_cuda()
    build.build_cuda(checked=True)
    regular, checked = ctypes.CDLL(str(build.CUDA_LIB)), ctypes.CDLL(str(build.CUDA_LIB_CHECKED))
    assert regular.tp_checked_build() == 0 and checked.tp_checked_build() == 1
    for name in SIGNATURES:
        assert hasattr(regular, name) and hasattr(checked, name), name


def _walk(kind, M, N, K, rank, rpr, pairs=74, tile_rows=256, tile_cols=128):
    import ctypes

    from terapipe_b200.ops.lib import host_lib
    num_m, num_n = -(-M // tile_rows), -(-N // tile_cols)
    order = (ctypes.c_int * 8)()
    coords = (ctypes.c_int * (2 * num_m * num_n))()
    n = host_lib().tp_tile_order_walk(kind, M, N, K, tile_rows, tile_cols, rank, rpr, pairs, order, coords)
    assert n == num_m * num_n, (kind, M, N, K, rank, rpr, n)      # a bijection onto the tile grid
    tiles = [(coords[2 * i], coords[2 * i + 1]) for i in range(n)]
    names = ("num_m_tiles", "num_n_tiles", "m_major", "m_first", "order_split", "order_group",
             "order_first_only", "order_pipelined")
    return tiles, dict(zip(names, order))


def test_gemm_tile_orders_cover_the_grid_and_respect_ownership():
    """The tile orders the kernels run (csrc/tile_order.h, compiled here for the host): every
    order visits every output tile exactly once; all-gather -> GEMM starts with row blocks whose
    operand rows are local; GEMM -> reduce-scatter produces the other ranks' row blocks of a
    column before this rank's own, in one group all of them before any of its own."""
    for M, N, K in [(1024, 5120, 2560), (1024, 5120, 10240), (2048, 7680, 5120), (512, 12288, 6144),
                    (768, 2560, 5120), (1536, 6144, 24576), (256, 5120, 2560), (4096, 1536, 12288)]:
        tiles, o = _walk(0, M, N, K, 0, M)
        assert not o["m_major"] and tiles[1] == ((1, 0) if o["num_m_tiles"] > 1 else (0, 1))
        for tp in (2, 4, 8):
            rpr = -(-M // tp)
            rpr = -(-rpr // 32) * 32
            for rank in range(tp):
                lo, hi = rank * rpr, min((rank + 1) * rpr, M)
                own = {m for m in range(-(-M // 256)) if lo < hi and m * 256 < hi and (m + 1) * 256 > lo}
                # all-gather -> GEMM
                tiles, o = _walk(1, M, N, K, rank, rpr)
                if o["m_major"]:
                    first_wave = tiles[:o["order_split"] * min(o["order_group"], o["num_n_tiles"])]
                    assert all(m in own for m, _ in first_wave), (M, N, tp, rank)
                # GEMM -> reduce-scatter
                tiles, o = _walk(2, M, N, K, rank, rpr)
                if not o["m_major"]:
                    continue
                pos = {t: i for i, t in enumerate(tiles)}
                for n in range(o["num_n_tiles"]):
                    others = [pos[(m, n)] for m in range(o["num_m_tiles"]) if m not in own]
                    mine = [pos[(m, n)] for m in own]
                    assert max(others) < min(mine), (M, N, K, tp, rank, n)
                if not o["order_pipelined"]:
                    assert max(pos[t] for t in tiles if t[0] not in own) < \
                        min(pos[t] for t in tiles if t[0] in own)
                else:
                    # a column's own blocks follow its group's first phase by one more first phase
                    assert o["order_group"] < o["num_n_tiles"]
