"""The allocation-free LayerNorm backward, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory at the point where they call it
(a host application that owns the whole GPU through its own pool, or code in a loop where
cudaMalloc's implicit synchronisation is not acceptable).  ``tp_layernorm_bwd_noalloc`` keeps
the kernel's partial-sum scratch in a fixed array inside the library, so the call needs only the
caller's inputs and outputs.  Here it must reproduce the regular entry point, twice in a row
(the array is shared between calls and keeps the previous call's contents).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    # cuda_lib() builds the library on first use, so this file also runs alone on a fresh tree;
    # the entry point itself is fetched by its exported C name from the loaded library
    from terapipe_b200.ops.lib import cuda_lib
    lib = cuda_lib()
    fn = lib.tp_layernorm_bwd_noalloc
    fn.restype = ctypes.c_int
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [I, P, P, P, P, P, P, P, P, P, I, I, P]
    cap = lib.tp_layernorm_bwd_noalloc_capacity
    cap.restype = ctypes.c_longlong
    return fn, cap


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_layernorm_backward_matches_regular_entry_point():
    from terapipe_b200.ops import functional as F
    fn, cap = _symbol()
    assert cap() == 160 * 2 * 4096
    torch.manual_seed(11)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, H) in enumerate([(520, 2048), (1024, 256), (96, 4096)]):  # 4096: widest accepted
        dtype = torch.float16
        x = torch.randn(rows, H, device="cuda", dtype=dtype)
        g = (1 + 0.1 * torch.randn(H, device="cuda")).to(dtype)
        b = torch.zeros(H, device="cuda", dtype=dtype)
        y = torch.empty_like(x)
        mean = torch.empty(rows, device="cuda")
        rstd = torch.empty(rows, device="cuda")
        F.layernorm_fwd(x, g, b, y, mean, rstd)
        dy = torch.randn(rows, H, device="cuda", dtype=dtype)
        dres = torch.randn(rows, H, device="cuda", dtype=dtype)
        # regular entry point with a caller-provided scratch buffer
        dx_ref = torch.empty_like(x)
        dg_ref, db_ref = torch.ones(H, device="cuda"), torch.ones(H, device="cuda")
        scratch = torch.empty(F.layernorm_bwd_scratch_floats(rows, H), device="cuda")
        F.layernorm_bwd(dy, x, mean, rstd, g, dx_ref, dg_ref, db_ref, scratch, dres=dres)
        # allocation-free entry point: outputs allocated up front, nothing allocated by the call
        dx = torch.empty_like(x)
        dg, db = torch.ones(H, device="cuda"), torch.ones(H, device="cuda")
        args = (0, dy.data_ptr(), x.data_ptr(), mean.data_ptr(), rstd.data_ptr(), g.data_ptr(),
                dres.data_ptr(), dx.data_ptr(), dg.data_ptr(), db.data_ptr(), rows, H, stream)
        for repeat in range(2):      # two calls in a row share the built-in array
            dg.fill_(1.0)
            db.fill_(1.0)
            dx.zero_()
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            free_before = torch.cuda.mem_get_info()[0]
            st = fn(*args)
            torch.cuda.synchronize()
            assert st == 0, (call, repeat, st)
            assert torch.cuda.memory_allocated() == before
            if repeat == 1:
                # the kernels are loaded and the array's address is resolved by now: the device's
                # free memory must not move, i.e. no cudaMalloc inside the library either
                assert torch.cuda.mem_get_info()[0] == free_before
            assert _rel(dx, dx_ref) < 3e-3
            assert _rel(dg, dg_ref) < 2e-3 and _rel(db, db_ref) < 2e-3


def test_noalloc_rejects_rows_wider_than_the_built_in_array():
    fn, _ = _symbol()
    dummy = torch.zeros(16, device="cuda")
    p = dummy.data_ptr()
    st = fn(0, p, p, p, p, p, None, p, p, p, 8, 8192, torch.cuda.current_stream().cuda_stream)
    assert st == -4
