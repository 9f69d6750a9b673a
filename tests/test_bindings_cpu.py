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
