"""Python entry points of the sm_100a kernels (torch tensors in, raw pointers out).

Every function enqueues on the current torch CUDA stream, allocates nothing unless the
caller omits an output/workspace tensor, and raises :class:`KernelError` when the native
call rejects its arguments.  Device-side wait time-outs are reported through a per-device
status word: call :func:`check_device_status` after a synchronisation point.
"""
from __future__ import annotations

from typing import Optional

import torch

from .lib import CHECK_CODES, _ERRORS, CheckFailed, CommTimeout, KernelError, check, cuda_lib

_ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2}
_status = {}


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"unsupported dtype {t.dtype}; kernels take float16 or bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device=None) -> torch.Tensor:
    """int32[1] on the device; kernels CAS their first time-out code into it."""
    idx = None if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def check_device_status(device=None, reset=True) -> None:
    """Synchronising read of the status word; raises :class:`CommTimeout` if a wait ran out and
    :class:`CheckFailed` if an index check of the checked build failed."""
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        if reset:
            word.zero_()
        if code in CHECK_CODES:
            raise CheckFailed(f"{_ERRORS.get(code, 'checked build: index check failed')} (code {code})")
        raise CommTimeout(f"a device-side wait timed out (code {code})")


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, a_mn=False, b_mn=False,
         alpha: float = 1.0, bias=None, residual=None, act=None, aux_out=None, dact=None,
         aux_in=None, accumulate=False, force_bn: int = 0) -> torch.Tensor:
    """``out[m, n] = epilogue(alpha * sum_k A(m, k) B(n, k))`` on tcgen05 tensor cores.

    ``a`` is ``[M, K]`` (or ``[K, M]`` when ``a_mn``), ``b`` is ``[N, K]`` (or ``[K, N]``
    when ``b_mn``); rows may be strided (last dim contiguous).  Epilogue options: ``bias``
    ``[N]``; ``act`` in {"relu", "gelu"} (``aux_out`` receives the pre-activation for
    gelu); ``residual`` ``[M, N]``; ``dact`` in {"relu", "gelu"} multiplies by the
    activation derivative evaluated on ``aux_in`` (post-activation for relu,
    pre-activation for gelu); ``out`` may be fp32 and may ``accumulate``."""
    M, N = out.shape
    K = a.shape[0] if a_mn else a.shape[1]
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    assert (a.shape[1] if a_mn else a.shape[0]) == M, "A does not match out rows"
    assert (b.shape[1] if b_mn else b.shape[0]) == N and (b.shape[0] if b_mn else b.shape[1]) == K
    out_f32 = out.dtype == torch.float32
    aux = aux_out if aux_out is not None else aux_in
    st = cuda_lib().tp_gemm(
        _dt(a), int(a_mn), int(b_mn), a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
        out.data_ptr(), out.stride(0), int(out_f32), int(accumulate), M, N, K, float(alpha),
        _ptr(bias), _ptr(residual), residual.stride(0) if residual is not None else 0,
        _ACT[act], _ptr(aux_out), _ACT[dact], _ptr(aux_in), aux.stride(0) if aux is not None else 0,
        int(force_bn), status_word(a.device).data_ptr(), _stream())
    check(st, "tp_gemm")
    return out


GEMM_TRACE_SLOTS = 24


def gemm_pair_trace(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, bn: int = 256) -> torch.Tensor:
    """Run the CTA-pair GEMM (fp16, ``out = a @ b.T``) in its tracing build and return the
    per-CTA phase stamps, an int64 tensor ``[n_ctas, 24]`` of SM clock cycles (slot meanings
    are listed at ``tp_gemm_trace`` in ``csrc/gemm_sm100.cu``)."""
    M, N = out.shape
    K = a.shape[1]
    assert a.dtype == torch.float16 and b.dtype == torch.float16 and out.dtype == torch.float16
    tiles = ((M + 255) // 256) * ((N + bn - 1) // bn)
    sms = torch.cuda.get_device_properties(a.device).multi_processor_count
    n_ctas = 2 * min(tiles, sms // 2)
    trace = torch.zeros(n_ctas, GEMM_TRACE_SLOTS, dtype=torch.int64, device=a.device)
    st = cuda_lib().tp_gemm_trace(int(bn), a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                                  out.data_ptr(), out.stride(0), M, N, K, trace.data_ptr(),
                                  status_word(a.device).data_ptr(), _stream())
    check(st, "tp_gemm_trace")
    return trace


def layernorm_fwd(x, gamma, beta, y, mean, rstd, eps=1e-5):
    rows, H = x.shape
    st = cuda_lib().tp_layernorm_fwd(_dt(x), x.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                     y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows, H,
                                     float(eps), _stream())
    check(st, "tp_layernorm_fwd")
    return y


def layernorm_bwd_scratch_floats(rows: int, H: int) -> int:
    return cuda_lib().tp_layernorm_bwd_parts(int(rows)) * 2 * H


def layernorm_bwd(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, scratch, dres=None):
    """``dx = LN'(dy) (+ dres)``; ``dgamma``/``dbeta`` (fp32) are accumulated into.
    ``scratch`` is an fp32 workspace of :func:`layernorm_bwd_scratch_floats` elements."""
    rows, H = x.shape
    assert scratch.numel() >= layernorm_bwd_scratch_floats(rows, H)
    st = cuda_lib().tp_layernorm_bwd(_dt(x), dy.data_ptr(), x.data_ptr(), mean.data_ptr(),
                                     rstd.data_ptr(), gamma.data_ptr(), _ptr(dres), dx.data_ptr(),
                                     dgamma.data_ptr(), dbeta.data_ptr(), scratch.data_ptr(),
                                     rows, H, _stream())
    check(st, "tp_layernorm_bwd")
    return dx


def colsum(dy, db):
    """``db[n] += sum_rows dy[row, n]`` (bias gradient), fp32 accumulation."""
    rows, N = dy.shape
    st = cuda_lib().tp_colsum(_dt(dy), dy.data_ptr(), dy.stride(0), rows, N, db.data_ptr(), _stream())
    check(st, "tp_colsum")
    return db


def adam_tick(state, beta1=0.9, beta2=0.999):
    check(cuda_lib().tp_adam_tick(state.data_ptr(), beta1, beta2, _stream()), "tp_adam_tick")


def fused_adam(grad, master, m, v, model, state, lr, beta1=0.9, beta2=0.999, eps=1e-8,
               weight_decay=0.0, grad_scale=1.0):
    """One pass over flat buffers: unscale the fp32 gradient, update fp32 ``master``/``m``/``v``,
    rewrite the 16-bit ``model`` copy and zero ``grad``.  ``state`` is float32[3] =
    (step, 1-beta1^t, 1-beta2^t), advanced on the device by :func:`adam_tick`."""
    n = grad.numel()
    st = cuda_lib().tp_fused_adam(_dt(model), grad.data_ptr(), master.data_ptr(), m.data_ptr(),
                                  v.data_ptr(), model.data_ptr(), n, state.data_ptr(), lr, beta1,
                                  beta2, eps, weight_decay, grad_scale, _stream())
    check(st, "tp_fused_adam")


def fill(t, value: float):
    check(cuda_lib().tp_fill(_dt(t), t.data_ptr(), t.numel(), float(value), _stream()), "tp_fill")
    return t


def attn_fwd(qkv, b: int, h: int, D: int, t: int, c: int, o, lse2, scale: float = 0.0):
    """Slice-causal attention forward.

    ``qkv``: full-length projection buffer ``[L, b, h*3*D]`` (per head q,k,v interleaved);
    rows ``[0, c+t)`` are read, the slice's queries are rows ``[c, c+t)``.
    ``o``: ``[t*b, h*D]`` output of the slice (row = position*b + batch).
    ``lse2``: fp32 ``[b*h, L]`` base-2 log-sum-exp, written at positions ``[c, c+t)``.
    ``scale``: multiplier of q.k (0 = ``D ** -0.5``); heads narrower than ``D`` whose extra
    columns are zero pass the scale of their real width."""
    st = cuda_lib().tp_attn_fwd_scaled(_dt(qkv), D, float(scale), qkv.data_ptr(), b, h, t, c,
                                       o.data_ptr(), o.stride(0), lse2.data_ptr(), lse2.stride(0),
                                       status_word(qkv.device).data_ptr(), _stream())
    check(st, "tp_attn_fwd_scaled")
    return o


def attn_bwd(qkv, b: int, h: int, D: int, t: int, c: int, q_end: int, o, do_full, lse2, delta,
             dqkv, scale: float = 0.0):
    """Slice-causal attention backward for the slice ``[c, c+t)``.

    Slices are processed last to first.  ``do_full`` is the full-length gradient of the
    attention output ``[L*b, h*D]``: rows of the slices after this one (up to position
    ``q_end``) were written by their own backward, rows ``[c*b, (c+t)*b)`` by the caller just
    before this call.  ``o`` is this slice's forward output ``[t*b, h*D]``; ``lse2`` and
    ``delta`` are fp32 ``[b*h, L]`` (``delta`` rows of this slice are written here).
    Writes the slice's complete ``d(qkv)`` ``[t*b, h*3*D]``."""
    st = cuda_lib().tp_attn_bwd_scaled(_dt(qkv), D, float(scale), qkv.data_ptr(), b, h, t, c, q_end,
                                       o.data_ptr(), o.stride(0), do_full.data_ptr(),
                                       do_full.stride(0), lse2.data_ptr(), lse2.stride(0),
                                       delta.data_ptr(), dqkv.data_ptr(), dqkv.stride(0),
                                       status_word(qkv.device).data_ptr(), _stream())
    check(st, "tp_attn_bwd_scaled")
    return dqkv
