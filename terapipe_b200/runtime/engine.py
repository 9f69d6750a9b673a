"""The sm_100a training engine: one pipeline stage per GPU, explicit forward/backward.

What one rank owns
------------------
* Flat parameter state for its layers: a 16-bit model copy, fp32 master weights, Adam
  moments and an fp32 main-gradient buffer.  One fused Adam launch updates the whole
  stage; weight-gradient GEMMs accumulate straight into the main-gradient buffer.
* Full-length activation buffers ``[L*B, width]`` per layer.  A token slice is a contiguous
  row range, so the "KV cache" is simply the QKV projection buffer: slice *j* writes rows
  ``[c, c+t)`` and attends over rows ``[0, c+t)`` in place.
* Full-length gradient buffers per layer (``d`` of the layer output, of the post-attention
  stream, of the FFN pre-activation, of QKV and of the attention output).  They serve two
  purposes.  (1) The backward pass walks the slices in reverse, so when slice *j* runs, the
  attention-output gradients of all later slices are still there and ``dK/dV`` of slice
  *j*'s keys are computed in one pass over those later queries: no accumulator crosses
  slices.  (2) Weight gradients are not computed per slice but once per layer over all
  ``L*B`` rows after the last slice (one long-K GEMM per weight instead of one short
  read-modify-write GEMM per slice); in a pipeline this also takes the weight-gradient work
  off the inter-stage critical path.

Schedule (same as the reference, test_transformer_terapipe.py:107-175,270-287): for each
batch slice all token slices forward in order; backward visits batch slices and token
slices in reverse; data-parallel gradient reduction; optimizer.  There is no autograd graph:
every kernel of the forward and backward pass is launched explicitly, which lets the whole
iteration be captured in one CUDA graph when the stage does not communicate.

Tensor parallelism keeps activations replicated inside the TP group (as the reference
does); the partial products of row-parallel layers and the data gradients of
column-parallel layers are summed either by NCCL all-reduce or by the fused
GEMM + all-reduce kernel over NVLink peer memory (``tp_comm="fused"``).
"""
from __future__ import annotations

import os

import math
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..models import TransformerConfig
from ..ops import functional as F
from ..ops.lib import KernelError, cuda_lib

LOSS_SCALE_FACTOR = 128.0
_ACT = {"none": 0, "relu": 1, "gelu": 2}

# parameter order inside a layer (names match the portable layer's state dict)
PARAM_ORDER = ("attn_ln.weight", "attn_ln.bias", "attn.in_proj.weight", "attn.in_proj.bias",
               "attn.out_proj.weight", "attn.out_proj.bias", "fc_ln.weight", "fc_ln.bias",
               "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias")


def _align(n: int, a: int = 8) -> int:
    return (n + a - 1) // a * a


class _Layout:
    """Offsets (in elements) of every parameter of the stage inside the flat buffers."""

    def __init__(self, n_layers: int, H: int, F_: int, tp: int, hl: Optional[int] = None):
        # hl: local width of the attention projections as the kernels see it (heads padded to the
        # kernels' head width); defaults to the model's own H / tp
        hl, fl = (H // tp if hl is None else hl), F_ // tp
        self.shapes = {
            "attn_ln.weight": (H,), "attn_ln.bias": (H,),
            "attn.in_proj.weight": (3 * hl, H), "attn.in_proj.bias": (3 * hl,),
            "attn.out_proj.weight": (H, hl), "attn.out_proj.bias": (H,),
            "fc_ln.weight": (H,), "fc_ln.bias": (H,),
            "fc1.weight": (fl, H), "fc1.bias": (fl,),
            "fc2.weight": (H, fl), "fc2.bias": (H,),
        }
        self.offsets: List[Dict[str, int]] = []
        off = 0
        for _ in range(n_layers):
            entry = {}
            for name in PARAM_ORDER:
                entry[name] = off
                off += _align(math.prod(self.shapes[name]))
            self.offsets.append(entry)
        self.total = _align(off, 8)


class StageEngine:
    # Tensor-parallel communication: "nccl" = all-reduce after the GEMM (activations replicated),
    # "fused" = GEMM + all-reduce in one kernel over peer memory (activations replicated),
    # "sp" = sequence parallel: LayerNorm, residual stream and pipeline links on a token shard
    # per rank, GEMM -> reduce-scatter and all-gather -> GEMM fused over peer memory.
    TP_COMM_MODES = ("nccl", "fused", "sp")

    def __init__(self, config: TransformerConfig, batch_slices: Sequence[int],
                 seq_slices: Sequence[int], dtype=torch.float16, loss_scale=LOSS_SCALE_FACTOR,
                 lr=1e-10, seed=0, init="device", use_graph: Optional[bool] = None,
                 tp_comm="nccl", dp_comm="nccl", device=None, launch_plan: Optional[bool] = None,
                 segment_graphs: Optional[bool] = None):
        assert torch.cuda.is_available(), "StageEngine needs a CUDA device (sm_100a)"
        self.cfg = config
        self.batch_slices, self.seq_slices = list(batch_slices), list(seq_slices)
        assert sum(self.batch_slices) == config.batch_size and sum(self.seq_slices) == config.seq_len
        self.dtype, self.dt = dtype, (0 if dtype == torch.float16 else 1)
        self.loss_scale, self.lr, self.seed = float(loss_scale), lr, seed
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.lib = cuda_lib()
        self.topo = mpu.get_topology()
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.dp_idx, self.pp_idx, self.tp_idx = self.topo.coords(self.rank)
        self.tp, self.pp, self.dp = self.topo.tp, self.topo.pp, self.topo.dp
        self.is_first, self.is_last = self.pp_idx == 0, self.pp_idx == self.pp - 1
        self.layer_ids = self.topo.layers_of_stage(config.n_layers, self.pp_idx)
        self.n_layers = len(self.layer_ids)
        if tp_comm not in self.TP_COMM_MODES:
            raise ValueError(f"tp_comm must be one of {self.TP_COMM_MODES}")
        self.tp_comm = tp_comm if self.tp > 1 else "none"
        self.dp_comm = dp_comm if self.dp > 1 else "none"
        self.sp = self.tp_comm == "sp"
        # overlap the data-parallel reduction with the weight-gradient products (TERAPIPE_DP_OVERLAP=0
        # runs it after them, for comparison)
        self.dp_overlap = os.environ.get("TERAPIPE_DP_OVERLAP", "1") != "0"
        self._dp_overlap, self._dp_works = False, None
        if self.sp:
            bad = [t * b for b in self.batch_slices for t in self.seq_slices if (t * b) % (32 * self.tp)]
            if bad:
                raise ValueError(f"tp_comm='sp' shards every token slice over {self.tp} ranks in "
                                 f"blocks of 32 rows; slices of {bad} rows do not divide")

        H, Fw = config.embedding_dim, config.ffn_embedding_dim
        heads = config.num_attention_heads
        assert heads % self.tp == 0 and Fw % self.tp == 0
        self.H, self.D = H, H // heads
        self.h = heads // self.tp
        # The attention kernels exist for 64- and 128-wide heads.  Any other width (80: gpt3-2b,
        # 96: megatron-*, gpt3-7hm) runs as the next of the two: the rows of the query/key/value
        # projection and the columns of the output projection that belong to the extra head
        # columns are zero, so q.k, the attention output and every gradient of the real columns
        # are unchanged, the gradients of the padding are exactly zero (Adam leaves it at zero),
        # and only the softmax scale has to be told the real width.
        if self.D > 128 or self.D % 8:
            raise ValueError(f"head dim {self.D} is not supported (a multiple of 8 up to 128)")
        self.Dk = self.D if self.D in (64, 128) else (64 if self.D < 64 else 128)
        self.attn_scale = float(self.D) ** -0.5
        self.Hl, self.Fl = self.h * self.Dk, Fw // self.tp
        self.L, self.B = config.seq_len, config.batch_size
        self.rows = self.L * self.B
        self.act = config.activation
        self.es = 2  # bytes per 16-bit element

        self.layout = _Layout(self.n_layers, H, Fw, self.tp, self.Hl)
        n = self.layout.total
        dev = self.device
        self.dp_sym = None
        if self.dp_comm == "fused":
            # gradients and the 16-bit parameters must be peer-mapped inside the DP group: the
            # fused reduction reads every replica's gradients and writes every replica's model
            from ..parallel.symm import SymmetricBuffer
            model_bytes = (n * 2 + 255) // 256 * 256
            self.dp_sym = SymmetricBuffer(1024 + model_bytes + n * 4, mpu.get_data_parallel_group())
            self._dp_off_model, self._dp_off_grad = 1024, 1024 + model_bytes
            self.model = self.dp_sym.view(self._dp_off_model, (n,), dtype)
            self.grad = self.dp_sym.view(self._dp_off_grad, (n,), torch.float32)
            self.dp_epoch_base = torch.zeros(1, dtype=torch.int32, device=dev)
            # Ownership of the fused reduction + sharded Adam: within the flat range of every
            # layer, replica r owns the r-th chunk.  (lo, hi, begin, end) per layer.
            self._dp_ranges = []
            for l in range(self.n_layers):
                lo = self.layout.offsets[l][PARAM_ORDER[0]]
                hi = self.layout.offsets[l + 1][PARAM_ORDER[0]] if l + 1 < self.n_layers else n
                chunk = ((hi - lo + self.dp - 1) // self.dp + 3) // 4 * 4
                b = min(hi, lo + self.dp_idx * chunk)
                self._dp_ranges.append((lo, hi, b, min(hi, b + chunk)))
            self._dp_ptrs = (self.dp_sym.ptr_array(self._dp_off_grad),
                             self.dp_sym.ptr_array(self._dp_off_model), self.dp_sym.ptr_array(0))
            self._dp_calls = 0
            self._dp_stream = None
        else:
            self.model = torch.zeros(n, dtype=dtype, device=dev)
            self.grad = torch.zeros(n, dtype=torch.float32, device=dev)
        self.master = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.adam_state = torch.zeros(3, dtype=torch.float32, device=dev)
        self._init_weights(init)
        self._alloc_activations()
        self.status = F.status_word(dev)
        self.loss_buf = torch.zeros(1, dtype=torch.float32, device=dev)
        # A CUDA graph may hold this library's kernels only: captured NCCL point-to-point or
        # collective calls deadlocked on replay here, so a stage that calls NCCL runs eagerly.
        nccl_free = (self.pp == 1 and (self.dp == 1 or self.dp_comm == "fused")
                     and (self.tp == 1 or self.tp_comm in ("fused", "sp")))
        self.use_graph = nccl_free if use_graph is None else (bool(use_graph) and nccl_free)
        self._graph = None
        # Recorded launch plans (runtime/launch_plan.py) for stages that cannot use a CUDA graph:
        # the launches of every slice segment are recorded once and replayed.  Off unless asked
        # for (argument, or TERAPIPE_LAUNCH_PLAN=1); segments must hold this library's launches
        # only, so a stage whose slices all-reduce through NCCL keeps deriving its launches.
        want_plan = (os.environ.get("TERAPIPE_LAUNCH_PLAN", "0") == "1") if launch_plan is None \
            else bool(launch_plan)
        self._plan = None
        if want_plan and not self.use_graph and (self.tp == 1 or self.tp_comm in ("fused", "sp")):
            from .launch_plan import RecordingLibrary, SegmentCache
            self.lib = RecordingLibrary(self.lib)
            self._plan = SegmentCache(self.lib, on_error=lambda rc, name: F.check(rc, name))
        # Stages that cannot put the whole step into one CUDA graph (they talk to their pipeline
        # neighbours through NCCL) still capture every launch-only part of the step (one token
        # slice forward or backward, the weight gradients, the optimizer) in a graph of its own
        # and replay it between the NCCL calls, so the host issues one graph launch instead of
        # ~16 kernel launches per layer.  A segment that all-reduces through NCCL is not captured.
        seg_ok = (not self.use_graph and self._plan is None
                  and (self.tp == 1 or self.tp_comm != "nccl")
                  and os.environ.get("TERAPIPE_SEGMENT_GRAPHS", "1") != "0")
        if segment_graphs is not None:
            seg_ok = seg_ok and bool(segment_graphs)
        self._seg_graphs = {} if seg_ok else None
        self._cap_stream = None
        self.timeline = None   # set to a utils.trace.SliceTimeline to record per-slice device times
        self.step_count = 0
        self._streams_ready = False
        # launches of this library's own kernels (NCCL and torch kernels are not counted):
        # per layer and slice 7 forward (2 LN, 4 GEMM, attention) and 9 backward (4 GEMM,
        # 2 LN, 3 attention); per layer 10 after the last slice (4 weight-gradient GEMMs, 4 bias
        # column sums, 2 LayerNorm-gradient reductions); plus 2 for the optimizer
        n_slices = len(self.batch_slices) * len(self.seq_slices)
        self.launches_per_step = n_slices * self.n_layers * 16 + self.n_layers * 10 + 2
        self.launch_count = 0
        self._ar_calls_per_step = n_slices * self.n_layers * 4 + 1
        # sequence parallel: all-gather pushes per step (2 per layer and slice forward; backward one
        # per LayerNorm whose input gradient feeds another GEMM, plus the received output gradient)
        self._ag_calls_per_step = n_slices * (2 * self.n_layers + self.n_layers + max(self.n_layers - 1, 0)
                                              + (0 if self.is_last else 1)) + 1
        self._ag_calls = 0
        if self.sp:
            # one flag kernel per all-gather, two group barriers, the sums of the LayerNorm
            # gradients over the group and the three counter updates of a step
            self.launches_per_step += (self._ag_calls_per_step - 1) + 2 + 2 * self.n_layers + 3
        elif self.tp_comm == "fused":
            self.launches_per_step += 1      # the epoch counter update
        self._ag_stream, self._ag_pending = None, False
        self._first_step_synced = False
        self._ag_in_kernel = os.environ.get("TERAPIPE_AG_PUSH", "0") == "1"

    # ------------------------------------------------------------------ parameters
    def param(self, layer: int, name: str, buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        buf = self.model if buf is None else buf
        shape = self.layout.shapes[name]
        off = self.layout.offsets[layer][name]
        return buf[off:off + math.prod(shape)].view(shape)

    _HEAD_PADDED = ("attn.in_proj.weight", "attn.in_proj.bias", "attn.out_proj.weight")

    def _pad_heads(self, name: str, w: torch.Tensor) -> torch.Tensor:
        """A parameter (or gradient, or moment) of the model's own shape -> the shape the kernels
        use: every head of the local q/k/v rows (output-projection columns) widened from D to
        Dk with zeros.  Identity for the other parameters and when D is 64 or 128."""
        if self.Dk == self.D or name not in self._HEAD_PADDED:
            return w
        h, D, pad = self.h, self.D, self.Dk - self.D
        if name == "attn.in_proj.weight":
            return torch.nn.functional.pad(w.reshape(h, 3, D, -1), (0, 0, 0, pad)).reshape(3 * self.Hl, -1)
        if name == "attn.in_proj.bias":
            return torch.nn.functional.pad(w.reshape(h, 3, D), (0, pad)).reshape(3 * self.Hl)
        return torch.nn.functional.pad(w.reshape(-1, h, D), (0, pad)).reshape(-1, self.Hl)

    def _unpad_heads(self, name: str, w: torch.Tensor) -> torch.Tensor:
        """Inverse of :meth:`_pad_heads`: the kernels' shape -> the model's own shape."""
        if self.Dk == self.D or name not in self._HEAD_PADDED:
            return w
        h, D, Dk = self.h, self.D, self.Dk
        if name == "attn.in_proj.weight":
            return w.reshape(h, 3, Dk, -1)[:, :, :D].reshape(3 * h * D, -1)
        if name == "attn.in_proj.bias":
            return w.reshape(h, 3, Dk)[:, :, :D].reshape(3 * h * D)
        return w.reshape(-1, h, Dk)[:, :, :D].reshape(-1, h * D)

    def get_param(self, layer: int, name: str, buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The parameter in the model's own shape (a view unless heads are padded)."""
        return self._unpad_heads(name, self.param(layer, name, buf))

    def set_param(self, layer: int, name: str, value: torch.Tensor,
                  buf: Optional[torch.Tensor] = None) -> None:
        """Store a tensor of the model's own shape into the flat buffer ``buf``."""
        self.param(layer, name, buf).copy_(self._pad_heads(name, value.to(self.device)))

    def _init_weights(self, init: str) -> None:
        """``"reference"``: the full master matrix of every layer is drawn on the CPU from
        the global generator seeded with ``seed`` in the portable layer's order, then sliced
        (bit-identical to the portable path for any TP/PP layout).  ``"device"``: the full
        matrix is drawn on the GPU from a generator keyed by (seed, layer, matrix); still
        independent of the TP/PP layout, and fast enough for 10^10-parameter stacks."""
        H, Fw = self.H, self.cfg.ffn_embedding_dim
        full = {"attn.in_proj.weight": (3 * H, H), "attn.out_proj.weight": (H, H),
                "fc1.weight": (Fw, H), "fc2.weight": (H, Fw)}
        if init == "reference":
            torch.manual_seed(self.seed)
        for li, gid in enumerate(range(self.cfg.n_layers)):
            mine = gid in self.layer_ids
            local = gid - self.layer_ids.start
            for mi, (name, shape) in enumerate(full.items()):
                if init == "reference":
                    w = torch.empty(shape)
                    torch.nn.init.xavier_normal_(w)
                    if not mine:
                        continue
                    w = w.to(self.device)
                else:
                    if not mine:
                        continue
                    g = torch.Generator(device=self.device)
                    g.manual_seed((self.seed * 1000003 + gid) * 8 + mi)
                    std = math.sqrt(2.0 / (shape[0] + shape[1]))
                    w = torch.randn(shape, device=self.device, generator=g) * std
                if name in ("attn.in_proj.weight", "fc1.weight"):
                    nrow = shape[0] // self.tp
                    w = w[self.tp_idx * nrow:(self.tp_idx + 1) * nrow]
                else:
                    ncol = shape[1] // self.tp
                    w = w[:, self.tp_idx * ncol:(self.tp_idx + 1) * ncol]
                self.set_param(local, name, w, self.master)
                del w
            if mine:
                for name in ("attn_ln.weight", "fc_ln.weight"):
                    self.param(local, name, self.master).fill_(1.0)
        self.model.copy_(self.master)
        if self.dtype != torch.float32:
            # the 16-bit copy is authoritative at start, as when a model is cast with .half()
            self.master.copy_(self.model)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {f"layers.layers.{l}.{name}": self.get_param(l, name).clone()
                for l in range(self.n_layers) for name in PARAM_ORDER}

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        for l in range(self.n_layers):
            for name in PARAM_ORDER:
                self.set_param(l, name, sd[f"layers.layers.{l}.{name}"], self.master)
        self.model.copy_(self.master)
        if self.dtype != torch.float32:
            self.master.copy_(self.model)

    def named_grads(self, unscale=True) -> Dict[str, torch.Tensor]:
        s = 1.0 / self.loss_scale if unscale else 1.0
        return {f"layers.layers.{l}.{name}": self.get_param(l, name, self.grad).clone() * s
                for l in range(self.n_layers) for name in PARAM_ORDER}

    # ------------------------------------------------------------------ buffers
    def _alloc_activations(self) -> None:
        dev, dt, rows = self.device, self.dtype, self.rows
        H, Hl, Fl = self.H, self.Hl, self.Fl

        def buf(width, dtype=dt):
            return torch.empty(rows, width, dtype=dtype, device=dev)

        tmax = max(self.seq_slices) * max(self.batch_slices)
        self.tmax = tmax
        self.ar = None
        self._pool_off = {}
        if self.tp_comm in ("fused", "sp"):
            # matrices that receive all-reduced (or, sequence parallel, all-gathered) results live
            # at the same offset of a peer-mapped pool on every tensor-parallel rank
            from ..parallel.symm import FusedAllReduceContext
            n_mats = (4 if self.sp else 2) * self.n_layers
            pool = (n_mats * (rows * H * self.es + 256) + tmax * H * self.es
                    + self.n_layers * 4 * H * 4 + 65536)
            self.ar = FusedAllReduceContext(mpu.get_model_parallel_group(), tmax, H, pool)
            self.ar_epoch_base = torch.zeros(1, dtype=torch.int32, device=dev)
            self._ar_calls = 0
            # TERAPIPE_AR_EXCHANGE=1 selects the one-hop form of the fused all-reduce (every
            # rank receives every partial tile); the default is reduce-scatter + all-gather
            self.lib.tp_gemm_ar_set_exchange(int(os.environ.get("TERAPIPE_AR_EXCHANGE", "0") == "1"))

        if self.sp:
            # flag words and counters of the sequence-parallel collectives (zero-filled pool)
            self._ag_flags, self._off_ag_flags = self.ar.alloc((16,), torch.int32)
            self._bar_flags, self._off_bar_flags = self.ar.alloc((16,), torch.int32)
            self.ag_epoch_base = torch.zeros(1, dtype=torch.int32, device=dev)
            self.bar_epoch_base = torch.zeros(1, dtype=torch.int32, device=dev)
            self._push_counter = torch.zeros(1, dtype=torch.int32, device=dev)
            self._ag_flag_ptrs = self.ar.out_ptrs(self._off_ag_flags)
            self._bar_flag_ptrs = self.ar.out_ptrs(self._off_bar_flags)
            # per layer: folded LayerNorm gamma/beta gradient sums of this rank's token shard
            self._ln_pack, self._off_ln_pack = self.ar.alloc((max(self.n_layers, 1), 4 * H), torch.float32)

        def sym(name, nrows, pooled=True):
            if self.ar is None or not pooled:
                return torch.empty(nrows, H, dtype=dt, device=dev)
            t, off = self.ar.alloc((nrows, H), dt)
            self._pool_off[name] = off
            return t

        sp = self.sp
        # replicated activations: the all-reduced layer outputs are pooled; sequence parallel: the
        # all-gathered LayerNorm outputs and the gradients of the layer outputs are pooled instead
        self.X = [buf(H)] + [sym(f"X{l + 1}", rows, not sp) for l in range(self.n_layers)]
        if sp and self.n_layers:
            self.X[-1].zero_()   # rows of other ranks' shards are never written; the loss sums all
        self.ln1 = [sym(f"ln1_{l}", rows, sp) for l in range(self.n_layers)]
        self.ln2 = [sym(f"ln2_{l}", rows, sp) for l in range(self.n_layers)]
        self.xmid = [sym(f"xmid{l}", rows, not sp) for l in range(self.n_layers)]
        self.qkv = [buf(3 * Hl) for _ in range(self.n_layers)]
        self.ao = [buf(Hl) for _ in range(self.n_layers)]
        self.fa = [buf(Fl) for _ in range(self.n_layers)]
        self.fz = [buf(Fl) for _ in range(self.n_layers)] if self.act == "gelu" else None
        self.stats = [torch.empty(4, rows, dtype=torch.float32, device=dev) for _ in range(self.n_layers)]
        self.lse = [torch.empty(self.B * self.h, self.L, dtype=torch.float32, device=dev)
                    for _ in range(self.n_layers)]
        self.delta = [torch.empty(self.B * self.h, self.L, dtype=torch.float32, device=dev)
                      for _ in range(self.n_layers)]
        # gradients, full length (see the module docstring)
        self.dMid = [sym(f"dMid{l}", rows, sp) for l in range(self.n_layers)]
        self.dFc = [buf(Fl) for _ in range(self.n_layers)]
        self.dQKV = [buf(3 * Hl) for _ in range(self.n_layers)]
        self.dAO = [buf(Hl) for _ in range(self.n_layers)]
        self.dXo = [sym(f"dXo{l}", rows, sp) for l in range(self.n_layers)]   # d(layer output); the last one is
        self.dY = self.dXo[-1] if self.n_layers else None    # received from the next stage
        self.dX0 = buf(H) if not self.is_first else None    # gradients sent to the previous stage
        self.dA = torch.empty(tmax, H, dtype=dt, device=dev)
        self.dln = sym("dln", tmax, not sp)
        # LayerNorm parameter gradients: every backward launch adds its per-CTA partial sums
        # into persistent slots; one reduction per layer folds them after the last slice
        self.ln_parts = self.lib.tp_layernorm_bwd_parts(int(tmax))
        self.ln_slots = [torch.zeros(2, self.ln_parts, 2 * H, dtype=torch.float32, device=dev)
                         for _ in range(self.n_layers)]
        numel = self.L * self.B * H
        if self.is_last and self.n_layers:
            # loss = mean(output): the seed gradient is the same constant everywhere
            self.dXo[-1].fill_(self.loss_scale / numel)
        # slice bookkeeping: (batch offset, b, token offset c, t, first row)
        self.slices = []
        boff = 0
        for b in self.batch_slices:
            c = 0
            per_batch = []
            for t in self.seq_slices:
                per_batch.append((boff, b, c, t, self.L * boff + c * b))
                c += t
            self.slices.append(per_batch)
            boff += b

    # ------------------------------------------------------------------ raw launches
    def _gemm(self, a, lda, b, ldb, out, ldo, M, N, K, a_mn=0, b_mn=0, out_f32=0, accumulate=0,
              bias=None, residual=None, ldr=0, act=0, aux_out=None, dact=0, aux_in=None, ld_aux=0):
        st = self.lib.tp_gemm(self.dt, a_mn, b_mn, a, lda, b, ldb, out, ldo, out_f32, accumulate,
                              M, N, K, 1.0, bias, residual, ldr, act, aux_out, dact, aux_in, ld_aux,
                              0, self._status_ptr, self._stream)
        if st:
            F.check(st, "tp_gemm")

    def _ln(self, fn_name, *args):
        """An entry point of the library whose status must be zero (LayerNorm, column sums, ...);
        a rejected or failed launch raises."""
        st = getattr(self.lib, fn_name)(*args)
        if st:
            F.check(st, fn_name)

    def _p(self, layer, name, buf=None):
        base = (self.model if buf is None else buf)
        return base.data_ptr() + self.layout.offsets[layer][name] * base.element_size()

    def _all_reduce_rows(self, tensor, r0, T):
        dist.all_reduce(tensor[r0:r0 + T], group=mpu.get_model_parallel_group())

    def _gemm_ar(self, a, lda, b, ldb, out_name, row0, M, N, K, b_mn=0, bias=None, residual=None,
                 ldr=0):
        """Fused GEMM + tensor-parallel all-reduce into rows ``[row0, row0+M)`` of the pooled
        matrix ``out_name`` on every rank; bias and residual are added once, by the tile's owner."""
        ar = self.ar
        self._ar_calls += 1
        off = self._pool_off[out_name] + row0 * N * self.es
        st = self.lib.tp_gemm_ar(self.dt, b_mn, a, lda, b, ldb, N, M, N, K, bias, residual, ldr,
                                 ar.tp, ar.rank, self._ar_calls, self.ar_epoch_base.data_ptr(),
                                 ar.max_tiles, ar.stage_ptrs, ar.flag_a_ptrs, ar.flag_b_ptrs,
                                 ar.out_ptrs(off), self._status_ptr, self._stream)
        if st:
            F.check(st, "tp_gemm_ar")

    # ------------------------------------------------------------------ sequence-parallel helpers
    def _pool_ptrs(self, name, row):
        """Addresses of row ``row`` of the pooled matrix ``name`` in every rank's memory."""
        return self.ar.out_ptrs(self._pool_off[name] + row * self.H * self.es)

    def _gemm_ag(self, a, lda, b, ldb, out, ldo, M, N, K, rpr, wait=True, b_mn=0, bias=None, act=0,
                 aux_out=None, dact=0, aux_in=None, ld_aux=0):
        """All-gather -> GEMM: A's rows were pushed into this rank's memory by the group (the
        most recent push); rows of other ranks are awaited inside the kernel."""
        st = self.lib.tp_gemm_ag(self.dt, b_mn, a, lda, b, ldb, out, ldo, M, N, K, bias, act, aux_out,
                                 dact, aux_in, ld_aux,
                                 self._ag_flags.data_ptr() if wait else None,
                                 self.ag_epoch_base.data_ptr(), self._ag_calls, rpr, self.tp_idx,
                                 self._status_ptr, self._stream)
        if st:
            F.check(st, "tp_gemm_ag")

    def _gemm_rs(self, a, lda, b, ldb, out, ldo, M, N, K, rpr, b_mn=0, bias=None, residual=None, ldr=0):
        """GEMM -> reduce-scatter: rows ``[tp_idx * rpr, (tp_idx + 1) * rpr)`` of the summed
        product (+ bias + residual) land in ``out``; the other rows are not written."""
        ar = self.ar
        self._ar_calls += 1
        st = self.lib.tp_gemm_rs(self.dt, b_mn, a, lda, b, ldb, out, ldo, M, N, K, bias, residual, ldr,
                                 ar.tp, ar.rank, rpr, self._ar_calls, self.ar_epoch_base.data_ptr(),
                                 ar.max_tiles, ar.stage_ptrs, ar.flag_a_ptrs, self._status_ptr,
                                 self._stream)
        if st:
            F.check(st, "tp_gemm_rs")

    def _ag_async(self, name, row, rows):
        """All-gather of rows ``[row, row + rows)`` of the pooled matrix ``name`` (just written
        locally on the current stream): copy-engine copies to every peer plus a flag, on a side
        stream, so that the consumer (``_gemm_ag``, which starts with this rank's own row blocks)
        runs meanwhile.  ``TERAPIPE_AG_PUSH=1`` selects the variant in which the producing
        LayerNorm kernel stores to the peers itself."""
        self._ag_calls += 1
        if self._ag_stream is None:
            self._ag_stream = torch.cuda.Stream()
        side = self._ag_stream
        side.wait_stream(torch.cuda.current_stream())
        off = self._pool_off[name] + row * self.H * self.es
        local = self.ar.buf.local_ptr + off
        st = self.lib.tp_ag_copy(local, rows * self.H * self.es, self.ar.out_ptrs(off), self._ag_flag_ptrs,
                                 self.tp, self.tp_idx, self._ag_calls, self.ag_epoch_base.data_ptr(),
                                 side.cuda_stream)
        if st:
            F.check(st, "tp_ag_copy")
        self._ag_pending = True

    def _ag_join(self):
        """The side stream's copies become part of the current stream's order again (end of a
        slice; required before a captured segment closes)."""
        if self._ag_pending:
            torch.cuda.current_stream().wait_stream(self._ag_stream)
            self._ag_pending = False

    def _ln_fwd_push(self, x, gamma, beta, dst_name, row, mean, rstd, rows):
        if not self._ag_in_kernel:
            dst = self.ar.buf.local_ptr + self._pool_off[dst_name] + row * self.H * self.es
            self._ln("tp_layernorm_fwd", self.dt, x, gamma, beta, dst, mean, rstd, rows, self.H, 1e-5,
                                      self._stream)
            return self._ag_async(dst_name, row, rows)
        self._ag_calls += 1
        st = self.lib.tp_layernorm_fwd_push(self.dt, x, gamma, beta, self._pool_ptrs(dst_name, row), mean,
                                            rstd, rows, self.H, 1e-5, self.tp, self.tp_idx,
                                            self._ag_flag_ptrs, self._ag_calls,
                                            self.ag_epoch_base.data_ptr(),
                                            self._push_counter.data_ptr(), self._stream)
        if st:
            F.check(st, "tp_layernorm_fwd_push")

    def _ln_bwd_push(self, dy, x, mean, rstd, gamma, dres, dst_name, row, slots, rows):
        if not self._ag_in_kernel:
            dst = self.ar.buf.local_ptr + self._pool_off[dst_name] + row * self.H * self.es
            self._ln("tp_layernorm_bwd_accum", self.dt, dy, x, mean, rstd, gamma, dres, dst, slots, rows,
                                            self.H, self._stream)
            return self._ag_async(dst_name, row, rows)
        self._ag_calls += 1
        st = self.lib.tp_layernorm_bwd_accum_push(self.dt, dy, x, mean, rstd, gamma, dres,
                                                  self._pool_ptrs(dst_name, row), slots, rows, self.H,
                                                  self.tp, self.tp_idx, self._ag_flag_ptrs,
                                                  self._ag_calls, self.ag_epoch_base.data_ptr(),
                                                  self._push_counter.data_ptr(), self._stream)
        if st:
            F.check(st, "tp_layernorm_bwd_accum_push")

    def _forward_slice_sp(self, sl) -> None:
        """Sequence-parallel forward of one token slice: this rank normalises and keeps the
        residual stream of its ``T / tp`` rows only; LayerNorm outputs are pushed to every rank
        (all-gather) for the column-parallel products, row-parallel products reduce-scatter."""
        boff, b, c, t, r0 = sl
        T, H, Hl, Fl, es = t * b, self.H, self.Hl, self.Fl, self.es
        lib, dt, s = self.lib, self.dt, self._stream
        rpr = T // self.tp
        m0 = r0 + self.tp_idx * rpr            # first row of this rank's shard
        for l in range(self.n_layers):
            st = self.stats[l].data_ptr()
            self._ln_fwd_push(self.X[l].data_ptr() + m0 * H * es, self._p(l, "attn_ln.weight"),
                              self._p(l, "attn_ln.bias"), f"ln1_{l}", m0, st + m0 * 4,
                              st + (self.rows + m0) * 4, rpr)
            qkv_base = self.qkv[l].data_ptr() + self.L * boff * 3 * Hl * es
            qkv = self.qkv[l].data_ptr() + r0 * 3 * Hl * es
            self._gemm_ag(self.ln1[l].data_ptr() + r0 * H * es, H, self._p(l, "attn.in_proj.weight"), H,
                          qkv, 3 * Hl, T, 3 * Hl, H, rpr, bias=self._p(l, "attn.in_proj.bias"))
            ao = self.ao[l].data_ptr() + r0 * Hl * es
            lse = self.lse[l].data_ptr() + boff * self.h * self.L * 4
            rc = lib.tp_attn_fwd_scaled(dt, self.Dk, self.attn_scale, qkv_base, b, self.h, t, c, ao, Hl,
                                        lse, self.L, self._status_ptr, s)
            if rc:
                F.check(rc, "tp_attn_fwd_scaled")
            self._gemm_rs(ao, Hl, self._p(l, "attn.out_proj.weight"), Hl,
                          self.xmid[l].data_ptr() + r0 * H * es, H, T, H, Hl, rpr,
                          bias=self._p(l, "attn.out_proj.bias"),
                          residual=self.X[l].data_ptr() + r0 * H * es, ldr=H)
            self._ln_fwd_push(self.xmid[l].data_ptr() + m0 * H * es, self._p(l, "fc_ln.weight"),
                              self._p(l, "fc_ln.bias"), f"ln2_{l}", m0, st + (2 * self.rows + m0) * 4,
                              st + (3 * self.rows + m0) * 4, rpr)
            fa = self.fa[l].data_ptr() + r0 * Fl * es
            fz = self.fz[l].data_ptr() + r0 * Fl * es if self.fz is not None else None
            self._gemm_ag(self.ln2[l].data_ptr() + r0 * H * es, H, self._p(l, "fc1.weight"), H, fa, Fl,
                          T, Fl, H, rpr, bias=self._p(l, "fc1.bias"), act=_ACT[self.act], aux_out=fz,
                          ld_aux=Fl)
            self._gemm_rs(fa, Fl, self._p(l, "fc2.weight"), Fl,
                          self.X[l + 1].data_ptr() + r0 * H * es, H, T, H, Fl, rpr,
                          bias=self._p(l, "fc2.bias"),
                          residual=self.xmid[l].data_ptr() + r0 * H * es, ldr=H)
        self._ag_join()

    # ------------------------------------------------------------------ forward of one slice
    def _forward_slice(self, sl) -> None:
        if self.sp:
            return self._forward_slice_sp(sl)
        boff, b, c, t, r0 = sl
        T, H, Hl, Fl, es = t * b, self.H, self.Hl, self.Fl, self.es
        lib, dt, s = self.lib, self.dt, self._stream
        tp0 = self.tp_idx == 0
        for l in range(self.n_layers):
            x = self.X[l].data_ptr() + r0 * H * es
            ln1 = self.ln1[l].data_ptr() + r0 * H * es
            st = self.stats[l].data_ptr()
            self._ln("tp_layernorm_fwd", dt, x, self._p(l, "attn_ln.weight"), self._p(l, "attn_ln.bias"), ln1,
                                 st + r0 * 4, st + (self.rows + r0) * 4, T, H, 1e-5, s)
            qkv_base = self.qkv[l].data_ptr() + self.L * boff * 3 * Hl * es
            qkv = self.qkv[l].data_ptr() + r0 * 3 * Hl * es
            self._gemm(ln1, H, self._p(l, "attn.in_proj.weight"), H, qkv, 3 * Hl, T, 3 * Hl, H,
                       bias=self._p(l, "attn.in_proj.bias"))
            ao = self.ao[l].data_ptr() + r0 * Hl * es
            lse = self.lse[l].data_ptr() + boff * self.h * self.L * 4
            rc = lib.tp_attn_fwd_scaled(dt, self.Dk, self.attn_scale, qkv_base, b, self.h, t, c, ao, Hl,
                                        lse, self.L, self._status_ptr, s)
            if rc:
                F.check(rc, "tp_attn_fwd_scaled")
            xmid = self.xmid[l].data_ptr() + r0 * H * es
            if self.ar is not None:
                self._gemm_ar(ao, Hl, self._p(l, "attn.out_proj.weight"), Hl, f"xmid{l}", r0, T, H, Hl,
                              bias=self._p(l, "attn.out_proj.bias"), residual=x, ldr=H)
            else:
                self._gemm(ao, Hl, self._p(l, "attn.out_proj.weight"), Hl, xmid, H, T, H, Hl,
                           bias=self._p(l, "attn.out_proj.bias") if tp0 else None,
                           residual=x if tp0 else None, ldr=H)
                if self.tp > 1:
                    self._all_reduce_rows(self.xmid[l], r0, T)
            ln2 = self.ln2[l].data_ptr() + r0 * H * es
            self._ln("tp_layernorm_fwd", dt, xmid, self._p(l, "fc_ln.weight"), self._p(l, "fc_ln.bias"), ln2,
                                 st + (2 * self.rows + r0) * 4, st + (3 * self.rows + r0) * 4, T, H,
                                 1e-5, s)
            fa = self.fa[l].data_ptr() + r0 * Fl * es
            fz = self.fz[l].data_ptr() + r0 * Fl * es if self.fz is not None else None
            self._gemm(ln2, H, self._p(l, "fc1.weight"), H, fa, Fl, T, Fl, H,
                       bias=self._p(l, "fc1.bias"), act=_ACT[self.act], aux_out=fz, ld_aux=Fl)
            xo = self.X[l + 1].data_ptr() + r0 * H * es
            if self.ar is not None:
                self._gemm_ar(fa, Fl, self._p(l, "fc2.weight"), Fl, f"X{l + 1}", r0, T, H, Fl,
                              bias=self._p(l, "fc2.bias"), residual=xmid, ldr=H)
            else:
                self._gemm(fa, Fl, self._p(l, "fc2.weight"), Fl, xo, H, T, H, Fl,
                           bias=self._p(l, "fc2.bias") if tp0 else None,
                           residual=xmid if tp0 else None, ldr=H)
                if self.tp > 1:
                    self._all_reduce_rows(self.X[l + 1], r0, T)

    # ------------------------------------------------------------------ backward of one slice
    def _backward_slice(self, sl) -> None:
        """Data gradients of one token slice through every layer of the stage (last layer
        first).  Weight and bias gradients are left to :meth:`_weight_grads`."""
        if self.sp:
            return self._backward_slice_sp(sl)
        boff, b, c, t, r0 = sl
        T, H, Hl, Fl, es = t * b, self.H, self.Hl, self.Fl, self.es
        lib, dt, s = self.lib, self.dt, self._stream
        g = self.grad
        dln = self.dln.data_ptr()
        for l in reversed(range(self.n_layers)):
            st = self.stats[l].data_ptr()
            fa = self.fa[l].data_ptr() + r0 * Fl * es
            aux = (self.fz[l].data_ptr() + r0 * Fl * es) if self.fz is not None else fa
            xmid = self.xmid[l].data_ptr() + r0 * H * es
            x = self.X[l].data_ptr() + r0 * H * es
            ao = self.ao[l].data_ptr() + r0 * Hl * es
            dcur = self.dXo[l].data_ptr() + r0 * H * es
            dmid = self.dMid[l].data_ptr() + r0 * H * es
            dfc = self.dFc[l].data_ptr() + r0 * Fl * es
            dqkv = self.dQKV[l].data_ptr() + r0 * 3 * Hl * es
            dao = self.dAO[l].data_ptr() + r0 * Hl * es
            # ---- FFN
            self._gemm(dcur, H, self._p(l, "fc2.weight"), Fl, dfc, Fl, T, Fl, H, b_mn=1,
                       dact=_ACT[self.act], aux_in=aux, ld_aux=Fl)
            if self.ar is not None:
                self._gemm_ar(dfc, Fl, self._p(l, "fc1.weight"), H, "dln", 0, T, H, Fl, b_mn=1)
            else:
                self._gemm(dfc, Fl, self._p(l, "fc1.weight"), H, dln, H, T, H, Fl, b_mn=1)
                if self.tp > 1:
                    self._all_reduce_rows(self.dln, 0, T)
            slots = self.ln_slots[l].data_ptr()
            self._ln("tp_layernorm_bwd_accum", dt, dln, xmid, st + (2 * self.rows + r0) * 4,
                                       st + (3 * self.rows + r0) * 4, self._p(l, "fc_ln.weight"), dcur,
                                       dmid, slots + self.ln_parts * 2 * H * 4, T, H, s)
            # ---- attention
            self._gemm(dmid, H, self._p(l, "attn.out_proj.weight"), Hl, dao, Hl, T, Hl, H, b_mn=1)
            qkv_base = self.qkv[l].data_ptr() + self.L * boff * 3 * Hl * es
            dao_base = self.dAO[l].data_ptr() + self.L * boff * Hl * es
            lse = self.lse[l].data_ptr() + boff * self.h * self.L * 4
            delta = self.delta[l].data_ptr() + boff * self.h * self.L * 4
            rc = lib.tp_attn_bwd_scaled(dt, self.Dk, self.attn_scale, qkv_base, b, self.h, t, c, self.L,
                                        ao, Hl, dao_base, Hl, lse, self.L, delta, dqkv, 3 * Hl,
                                        self._status_ptr, s)
            if rc:
                F.check(rc, "tp_attn_bwd_scaled")
            if self.ar is not None:
                self._gemm_ar(dqkv, 3 * Hl, self._p(l, "attn.in_proj.weight"), H, "dln", 0, T, H, 3 * Hl,
                              b_mn=1)
            else:
                self._gemm(dqkv, 3 * Hl, self._p(l, "attn.in_proj.weight"), H, dln, H, T, H, 3 * Hl, b_mn=1)
                if self.tp > 1:
                    self._all_reduce_rows(self.dln, 0, T)
            if l > 0:
                dnext = self.dXo[l - 1].data_ptr() + r0 * H * es
            elif self.is_first:
                dnext = self.dA.data_ptr()
            else:
                dnext = self.dX0.data_ptr() + r0 * H * es
            self._ln("tp_layernorm_bwd_accum", dt, dln, x, st + r0 * 4, st + (self.rows + r0) * 4,
                                       self._p(l, "attn_ln.weight"), dmid, dnext, slots, T, H, s)

    def _backward_slice_sp(self, sl) -> None:
        """Sequence-parallel data gradients of one token slice (last layer first).  Data gradients
        of column-parallel layers reduce-scatter onto this rank's rows; the LayerNorm backward
        runs on those rows and pushes its result to every rank, where the data-gradient product of
        the preceding row-parallel layer (and, after the last slice, the weight gradients) need
        all rows."""
        boff, b, c, t, r0 = sl
        T, H, Hl, Fl, es = t * b, self.H, self.Hl, self.Fl, self.es
        lib, dt, s = self.lib, self.dt, self._stream
        rpr = T // self.tp
        m0 = r0 + self.tp_idx * rpr
        dln = self.dln.data_ptr()
        dln_mine = dln + self.tp_idx * rpr * H * es
        n = self.n_layers
        if not self.is_last and n:
            # the output gradient arrived from the next stage as this rank's shard: all-gather it
            self._ag_async(f"dXo{n - 1}", m0, rpr)
        for l in reversed(range(n)):
            st = self.stats[l].data_ptr()
            fa = self.fa[l].data_ptr() + r0 * Fl * es
            aux = (self.fz[l].data_ptr() + r0 * Fl * es) if self.fz is not None else fa
            ao = self.ao[l].data_ptr() + r0 * Hl * es
            dfc = self.dFc[l].data_ptr() + r0 * Fl * es
            dqkv = self.dQKV[l].data_ptr() + r0 * 3 * Hl * es
            dao = self.dAO[l].data_ptr() + r0 * Hl * es
            slots = self.ln_slots[l].data_ptr()
            # ---- FFN: d(fc1 out) from all rows of d(layer output); the seed gradient of the last
            # stage is a constant every rank holds, everything else was pushed by the group
            seeded = self.is_last and l == n - 1
            self._gemm_ag(self.dXo[l].data_ptr() + r0 * H * es, H, self._p(l, "fc2.weight"), Fl, dfc, Fl,
                          T, Fl, H, rpr, wait=not seeded, b_mn=1, dact=_ACT[self.act], aux_in=aux,
                          ld_aux=Fl)
            self._gemm_rs(dfc, Fl, self._p(l, "fc1.weight"), H, dln, H, T, H, Fl, rpr, b_mn=1)
            self._ln_bwd_push(dln_mine, self.xmid[l].data_ptr() + m0 * H * es,
                              st + (2 * self.rows + m0) * 4, st + (3 * self.rows + m0) * 4,
                              self._p(l, "fc_ln.weight"), self.dXo[l].data_ptr() + m0 * H * es,
                              f"dMid{l}", m0, slots + self.ln_parts * 2 * H * 4, rpr)
            # ---- attention
            self._gemm_ag(self.dMid[l].data_ptr() + r0 * H * es, H, self._p(l, "attn.out_proj.weight"),
                          Hl, dao, Hl, T, Hl, H, rpr, b_mn=1)
            qkv_base = self.qkv[l].data_ptr() + self.L * boff * 3 * Hl * es
            dao_base = self.dAO[l].data_ptr() + self.L * boff * Hl * es
            lse = self.lse[l].data_ptr() + boff * self.h * self.L * 4
            delta = self.delta[l].data_ptr() + boff * self.h * self.L * 4
            rc = lib.tp_attn_bwd_scaled(dt, self.Dk, self.attn_scale, qkv_base, b, self.h, t, c, self.L,
                                        ao, Hl, dao_base, Hl, lse, self.L, delta, dqkv, 3 * Hl,
                                        self._status_ptr, s)
            if rc:
                F.check(rc, "tp_attn_bwd_scaled")
            self._gemm_rs(dqkv, 3 * Hl, self._p(l, "attn.in_proj.weight"), H, dln, H, T, H, 3 * Hl, rpr,
                          b_mn=1)
            x_mine = self.X[l].data_ptr() + m0 * H * es
            dmid_mine = self.dMid[l].data_ptr() + m0 * H * es
            if l > 0:
                self._ln_bwd_push(dln_mine, x_mine, st + m0 * 4, st + (self.rows + m0) * 4,
                                  self._p(l, "attn_ln.weight"), dmid_mine, f"dXo{l - 1}", m0, slots, rpr)
            else:
                # gradient of the stage input: only this rank's rows exist (they go to the same
                # tensor-parallel rank of the previous stage, or nowhere on the first stage)
                dnext = (self.dA.data_ptr() + self.tp_idx * rpr * H * es) if self.is_first \
                    else self.dX0.data_ptr() + m0 * H * es
                self._ln("tp_layernorm_bwd_accum", dt, dln_mine, x_mine, st + m0 * 4, st + (self.rows + m0) * 4,
                                           self._p(l, "attn_ln.weight"), dmid_mine, dnext, slots, rpr,
                                           H, s)
        self._ag_join()

    def _weight_grads(self) -> None:
        """Weight and bias gradients of every layer over all ``L*B`` rows at once:
        ``dW += dY^T X`` with the token dimension as the (long) GEMM K dimension."""
        R, H, Hl, Fl = self.rows, self.H, self.Hl, self.Fl
        lib, dt, s, g = self.lib, self.dt, self._stream, self.grad
        # Data-parallel reduction overlapped with these products: as soon as the gradients of a
        # layer are complete (layers are visited last to first), its reduction - and with the fused
        # kernel its Adam update and parameter push - starts on a side stream (NCCL: on NCCL's own
        # stream) underneath the next layer's four long-K GEMMs.
        overlap = self._dp_overlap and not self.sp
        works = []
        if overlap and self.dp_sym is not None:
            self._dp_begin_update()
        for l in reversed(range(self.n_layers)):
            if l != self.n_layers - 1 and overlap:
                self._dp_layer_done(l + 1, works)
            dxo, dmid = self.dXo[l].data_ptr(), self.dMid[l].data_ptr()
            dfc, dqkv = self.dFc[l].data_ptr(), self.dQKV[l].data_ptr()
            self._gemm(dxo, H, self.fa[l].data_ptr(), Fl, self._p(l, "fc2.weight", g), Fl, H, Fl, R,
                       a_mn=1, b_mn=1, out_f32=1, accumulate=1)
            self._ln("tp_colsum", dt, dxo, H, R, H, self._p(l, "fc2.bias", g), s)
            self._gemm(dfc, Fl, self.ln2[l].data_ptr(), H, self._p(l, "fc1.weight", g), H, Fl, H, R,
                       a_mn=1, b_mn=1, out_f32=1, accumulate=1)
            self._ln("tp_colsum", dt, dfc, Fl, R, Fl, self._p(l, "fc1.bias", g), s)
            self._gemm(dmid, H, self.ao[l].data_ptr(), Hl, self._p(l, "attn.out_proj.weight", g), Hl,
                       H, Hl, R, a_mn=1, b_mn=1, out_f32=1, accumulate=1)
            self._ln("tp_colsum", dt, dmid, H, R, H, self._p(l, "attn.out_proj.bias", g), s)
            self._gemm(dqkv, 3 * Hl, self.ln1[l].data_ptr(), H, self._p(l, "attn.in_proj.weight", g),
                       H, 3 * Hl, H, R, a_mn=1, b_mn=1, out_f32=1, accumulate=1)
            self._ln("tp_colsum", dt, dqkv, 3 * Hl, R, 3 * Hl, self._p(l, "attn.in_proj.bias", g), s)
            slots = self.ln_slots[l].data_ptr()
            if self.sp:
                # this rank's slots hold the sums over its token shards only: fold them into a
                # peer-visible pack; the sums of all ranks are added after the barrier below
                pack = self._ln_pack.data_ptr() + l * 4 * H * 4
                self._ln("tp_layernorm_bwd_finish_assign", slots, self.ln_parts, H, pack, pack + H * 4, s)
                self._ln("tp_layernorm_bwd_finish_assign", slots + self.ln_parts * 2 * H * 4, self.ln_parts, H,
                                                   pack + 2 * H * 4, pack + 3 * H * 4, s)
                continue
            self._ln("tp_layernorm_bwd_finish", slots, self.ln_parts, H, self._p(l, "attn_ln.weight", g),
                                        self._p(l, "attn_ln.bias", g), s)
            self._ln("tp_layernorm_bwd_finish", slots + self.ln_parts * 2 * H * 4, self.ln_parts, H,
                                        self._p(l, "fc_ln.weight", g), self._p(l, "fc_ln.bias", g), s)
        if overlap and self.n_layers:
            self._dp_layer_done(0, works)
            if self.dp_sym is not None:
                torch.cuda.current_stream().wait_stream(self._dp_stream)
            else:
                self._dp_works = works
        if self.sp and self.n_layers:
            self._group_barrier(2)
            for l in range(self.n_layers):
                off = self._off_ln_pack + l * 4 * H * 4
                self._ln("tp_peer_sum", self._p(l, "attn_ln.weight", g), 2 * H, self.ar.out_ptrs(off), self.tp,
                                self.tp_idx, s)
                self._ln("tp_peer_sum", self._p(l, "fc_ln.weight", g), 2 * H, self.ar.out_ptrs(off + 2 * H * 4),
                                self.tp, self.tp_idx, s)

    def _group_barrier(self, index: int) -> None:
        """Device-side barrier of the tensor-parallel group (``index`` 1 or 2 within a step)."""
        st = self.lib.tp_group_barrier(self._bar_flag_ptrs, self.tp, self.tp_idx, index,
                                       self.bar_epoch_base.data_ptr(), self._status_ptr, self._stream)
        if st:
            F.check(st, "tp_group_barrier")

    # ------------------------------------------------------------------ one iteration
    def _refresh_handles(self):
        self._stream = torch.cuda.current_stream().cuda_stream
        self._status_ptr = self.status.data_ptr()
        if self._plan is not None:
            self._plan.validate((self._stream, self._status_ptr))

    def _segment(self, key, fn, *args):
        """Run one launch-only part of the step: directly, through the recorded plan, or as a
        CUDA graph of its own (first call eager, second call captured, then replayed)."""
        if self._plan is not None:
            self._plan.run(key, fn, *args)
        elif self._seg_graphs is not None:
            self._run_graphed(key, fn, *args)
        else:
            fn(*args)

    def _run_graphed(self, key, fn, *args):
        ent = self._seg_graphs.get(key)
        ar0, ag0 = getattr(self, "_ar_calls", 0), self._ag_calls
        if ent is None:
            # first time: eager (kernel attributes get set, nothing may be captured before that)
            fn(*args)
            self._seg_graphs[key] = [None, getattr(self, "_ar_calls", 0) - ar0, self._ag_calls - ag0]
            return
        if ent[0] is None:
            if self._cap_stream is None:
                self._cap_stream = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            outer = self._stream
            # thread-local capture mode: NCCL's watchdog thread may query events meanwhile
            with torch.cuda.stream(self._cap_stream):
                graph.capture_begin(capture_error_mode="thread_local")
                try:
                    self._stream = self._cap_stream.cuda_stream
                    fn(*args)
                finally:
                    graph.capture_end()
                    self._stream = outer
            if self.ar is not None:
                self._ar_calls = ar0     # the captured launches did not run
            self._ag_calls = ag0
            ent[0] = graph
        ent[0].replay()
        # call indices baked into the graph stay in step with the host's counters
        if self.ar is not None:
            self._ar_calls += ent[1]
        self._ag_calls += ent[2]

    def _setup_streams(self):
        if self._streams_ready:
            return
        self.recv_stream = torch.cuda.Stream()
        # One 2-rank process group per pipeline link: its own NCCL communicator and stream, so
        # traffic with the previous stage never queues behind traffic with the next stage (on
        # a shared communicator the pre-posted receives would hold back every send).
        self._link_prev = mpu.get_pipeline_parallel_succ_group()
        self._link_next = mpu.get_pipeline_parallel_pred_group()
        self._streams_ready = True

    def _post_recvs(self, forward: bool):
        """Pre-post every receive of a pass on a side stream so that transfers overlap the
        compute of earlier slices; returns the work handles in consumption order."""
        works = {}
        src = mpu.get_pipeline_prev_rank() if forward else mpu.get_pipeline_next_rank()
        group = self._link_prev if forward else self._link_next
        buf = self.X[0] if forward else self.dY
        order = [(bi, si) for bi in range(len(self.batch_slices)) for si in range(len(self.seq_slices))]
        if not forward:
            order = order[::-1]
        # fork the side stream from the current one (required under graph capture) and join it
        # back: it only carries event nodes, the receives themselves run on NCCL's stream
        self.recv_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.recv_stream):
            for bi, si in order:
                lo, hi = self._link_rows(self.slices[bi][si])
                works[(bi, si)] = dist.irecv(buf[lo:hi], src, group=group)
        torch.cuda.current_stream().wait_stream(self.recv_stream)
        return works

    def _link_rows(self, sl):
        """Row range of a token slice that crosses a pipeline link from this rank: all of it, or
        (sequence parallel) this rank's shard, which goes to the same tensor-parallel rank of the
        neighbouring stage."""
        _, b, _, t, r0 = sl
        T = t * b
        if not self.sp:
            return r0, r0 + T
        rpr = T // self.tp
        return r0 + self.tp_idx * rpr, r0 + (self.tp_idx + 1) * rpr

    def _forward_backward(self):
        pipelined = self.pp > 1
        if pipelined:
            self._setup_streams()
        nb, ns = len(self.batch_slices), len(self.seq_slices)
        if self.timeline is not None:
            self.timeline.begin_iteration()
        sends = []
        recvs = self._post_recvs(True) if (pipelined and not self.is_first) else None
        for bi in range(nb):
            for si in range(ns):
                sl = self.slices[bi][si]
                if recvs is not None:
                    recvs[(bi, si)].wait()
                if self.timeline is not None:
                    with self.timeline.slice("forward", bi, si):
                        self._segment(("forward", bi, si), self._forward_slice, sl)
                else:
                    self._segment(("forward", bi, si), self._forward_slice, sl)
                if pipelined and not self.is_last:
                    lo, hi = self._link_rows(sl)
                    sends.append(dist.isend(self.X[self.n_layers][lo:hi],
                                            mpu.get_pipeline_next_rank(), group=self._link_next))
        if self.is_last:
            self.loss_buf.copy_(self.X[self.n_layers].sum(dtype=torch.float32))
        recvs = self._post_recvs(False) if (pipelined and not self.is_last) else None
        for bi in reversed(range(nb)):
            for si in reversed(range(ns)):
                sl = self.slices[bi][si]
                if recvs is not None:
                    recvs[(bi, si)].wait()
                if self.timeline is not None:
                    with self.timeline.slice("backward", bi, si):
                        self._segment(("backward", bi, si), self._backward_slice, sl)
                else:
                    self._segment(("backward", bi, si), self._backward_slice, sl)
                if pipelined and not self.is_first:
                    lo, hi = self._link_rows(sl)
                    sends.append(dist.isend(self.dX0[lo:hi], mpu.get_pipeline_prev_rank(),
                                            group=self._link_prev))
        if self.dp > 1 and self.dp_sym is None:
            self._weight_grads()           # starts NCCL all-reduces: not for a captured segment
        else:
            self._segment(("weight_grads",), self._weight_grads)
        for w in sends:
            w.wait()

    # ------------------------------------------------------------------ data-parallel update
    def _dp_begin_update(self):
        """Fused path, once per step before the first layer's reduction: advance Adam's bias
        correction and the call counter of the reduction kernel's flags."""
        F.adam_tick(self.adam_state)
        self.lib.tp_advance_counter(self.dp_epoch_base.data_ptr(), self.n_layers, self._stream)
        self._dp_calls = 0
        if self._dp_stream is None:
            self._dp_stream = torch.cuda.Stream()

    def _dp_layer_update(self, l, stream_handle):
        """Fused reduction of layer ``l``: peer-load every replica's gradients of the chunk this
        replica owns, Adam on that chunk, peer-store the new 16-bit parameters into every
        replica; then clear the layer's gradients (the kernel's closing handshake guarantees that
        no replica still reads them)."""
        lo, hi, b, e = self._dp_ranges[l]
        self._dp_calls += 1
        gp, mp_, fp = self._dp_ptrs
        st = self.lib.tp_dp_reduce_adam(
            self.dt, self.dp, self.dp_sym.rank, self._dp_calls, self.dp_epoch_base.data_ptr(), gp, mp_, fp,
            self.master.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(), b, e,
            self.adam_state.data_ptr(), self.lr, 0.9, 0.999, 1e-8, 0.0,
            1.0 / (self.loss_scale * self.dp), self._status_ptr, stream_handle)
        if st:
            F.check(st, "tp_dp_reduce_adam")
        self.grad[lo:hi].zero_()

    def _dp_layer_done(self, l, works):
        """The gradients of layer ``l`` are complete on the current stream: start reducing them."""
        if self.dp_sym is not None:
            side = self._dp_stream
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._dp_layer_update(l, side.cuda_stream)
        else:
            lo = self.layout.offsets[l][PARAM_ORDER[0]]
            hi = self.layout.offsets[l + 1][PARAM_ORDER[0]] if l + 1 < self.n_layers else self.layout.total
            works.append(dist.all_reduce(self.grad[lo:hi], group=mpu.get_data_parallel_group(),
                                         async_op=True))

    def _reduce_and_update(self):
        if self.dp_sym is not None:
            if self._dp_overlap and not self.sp:
                return                     # done layer by layer underneath the weight gradients
            self._dp_begin_update()
            for l in reversed(range(self.n_layers)):
                self._dp_layer_update(l, self._stream)
            return
        if self.dp > 1:
            if self._dp_works is not None:
                for w in self._dp_works:   # per-layer all-reduces started under the weight gradients
                    w.wait()
                self._dp_works = None
            else:
                dist.all_reduce(self.grad, group=mpu.get_data_parallel_group())
        F.adam_tick(self.adam_state)
        F.fused_adam(self.grad, self.master, self.exp_avg, self.exp_avg_sq, self.model,
                     self.adam_state, lr=self.lr, grad_scale=1.0 / (self.loss_scale * self.dp))

    def _iteration(self, update=True):
        if not self._first_step_synced:
            # Kernels that wait for a peer on the device are bounded by the wait limit; the first
            # step follows minutes of set-up whose length differs between ranks (weight
            # initialisation, module loading), so the ranks of the groups meet on the host first.
            self._first_step_synced = True
            if (self.ar is not None or self.dp_sym is not None) and dist.is_initialized():
                torch.cuda.synchronize()
                for group in (mpu.get_model_parallel_group(), mpu.get_data_parallel_group()):
                    if group is not None and dist.get_world_size(group) > 1:
                        dist.barrier(group=group)
        self._refresh_handles()
        if self.ar is not None:
            # call indices restart at 1 every iteration; the device counter supplies the rest, so
            # a replayed CUDA graph still produces fresh, growing epochs
            self.lib.tp_advance_counter(self.ar_epoch_base.data_ptr(), self._ar_calls_per_step,
                                        self._stream)
            self._ar_calls = 0
        if self.sp:
            self.lib.tp_advance_counter(self.ag_epoch_base.data_ptr(), self._ag_calls_per_step,
                                        self._stream)
            self.lib.tp_advance_counter(self.bar_epoch_base.data_ptr(), 2, self._stream)
            self._ag_calls = 0
            # no rank may push this step's rows into a peer's buffers while that peer still reads
            # last step's (its weight-gradient products come last)
            self._group_barrier(1)
        self._dp_overlap = bool(update and self.dp > 1 and self.dp_overlap)
        self._dp_works = None
        self._forward_backward()
        if update and not (self.dp_sym is not None and self._dp_overlap and not self.sp):
            if self._seg_graphs is not None and (self.dp == 1 or self.dp_sym is not None):
                # (a recorded launch plan only sees calls made through self.lib: not this one)
                self._segment(("update",), self._reduce_and_update)
            else:
                self._reduce_and_update()

    def set_input(self, x: torch.Tensor) -> None:
        """Copy this replica's ``[L, B, H]`` input into the stage-0 activation buffer.  Rows are
        regrouped per batch slice (each batch slice owns a contiguous ``[L, b, H]`` block)."""
        assert self.is_first
        x = x.to(self.device, self.dtype, non_blocking=True)
        if len(self.batch_slices) == 1:
            self.X[0].view(self.L, self.B, self.H).copy_(x)
        else:
            boff = 0
            for b in self.batch_slices:
                dst = self.X[0][self.L * boff:self.L * (boff + b)].view(self.L, b, self.H)
                dst.copy_(x[:, boff:boff + b])
                boff += b

    def output(self) -> torch.Tensor:
        """The stage output as ``[L, B, H]`` (a copy when several batch slices exist)."""
        y = self.X[self.n_layers]
        if len(self.batch_slices) == 1:
            return y.view(self.L, self.B, self.H)
        parts, boff = [], 0
        for b in self.batch_slices:
            parts.append(y[self.L * boff:self.L * (boff + b)].view(self.L, b, self.H))
            boff += b
        return torch.cat(parts, dim=1)

    def loss(self) -> torch.Tensor:
        """Device scalar: mean of the final output (valid on the last stage after a step).  Under
        sequence parallelism every tensor-parallel rank holds the sum of its own rows; the ranks
        add them up here (an NCCL all-reduce of one number: call it outside graph capture, on
        every rank of the group)."""
        total = self.loss_buf
        if self.sp:
            total = self.loss_buf.clone()
            dist.all_reduce(total, group=mpu.get_model_parallel_group())
        return total / float(self.L * self.B * self.H)

    def compute_grads(self) -> None:
        """Forward + backward without the optimizer; scaled grads stay in ``self.grad``."""
        self.grad.zero_()
        self._iteration(update=False)
        if self.dp > 1:
            dist.all_reduce(self.grad, group=mpu.get_data_parallel_group())
            self.grad.div_(self.dp)

    def step(self) -> None:
        """One training iteration on the current stream.  With ``use_graph`` the first call
        runs eagerly (it also sets up kernel attributes) and records the iteration into a
        CUDA graph; later calls replay the graph."""
        if self.use_graph and self._graph is not None:
            self._graph.replay()
        else:
            self._iteration()
            if self.use_graph:
                self._capture()
        self.step_count += 1
        self.launch_count += self.launches_per_step

    def _capture(self):
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph):
                self._iteration()
        except (RuntimeError, KernelError) as e:
            # The whole step could not be captured (seen with a 48-layer stage of GPT3-44B width:
            # a launch inside the capture failed although the same step had just run eagerly).
            # Fall back to one graph per launch-only segment, which captures far smaller pieces.
            import warnings
            warnings.warn(f"whole-step CUDA graph capture failed ({type(e).__name__}: {str(e)[:120]}); "
                          "using per-segment graphs instead")
            torch.cuda.synchronize()
            self.use_graph = False
            self._graph = None
            self._ag_pending = False
            if self._plan is None and self._seg_graphs is None:
                self._seg_graphs = {}
            return
        self._graph = graph

    def check_status(self):
        F.check_device_status(self.device)

    def close(self) -> None:
        """Release the peer-mapped buffers (collective over the tensor- and data-parallel groups;
        call it between steps).  The engine must not be used afterwards."""
        self._graph = None
        if self._seg_graphs is not None:
            self._seg_graphs.clear()
        torch.cuda.synchronize()
        if self.ar is not None:
            self.ar.close()
            self.ar = None
        if self.dp_sym is not None:
            self.dp_sym.close()
            self.dp_sym = None
