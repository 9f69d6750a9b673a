"""Public training API: build the parallel layout and the sm_100a engine, feed inputs, step.

    trainer = Trainer("gpt3-1b", batch_size=8, tp=1, pp=world_size,
                      batch_slices=[8], seq_slices=[128] * 16)
    loss = trainer.train_step(host_input)      # H2D copy, forward, backward, Adam, loss D2H

``seq_slices="auto"`` plans batch and token slices with the dynamic program over the B200 kernel
model.  ``batch_size`` is the batch of ONE data-parallel replica; the data-parallel size is
``world_size // (tp * pp)``.  Inputs are hidden states ``[seq, batch, hidden]`` (the
benchmark harness has no embedding, as in the reference, terapipe.py:48-49); the loss is
the mean of the final output.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import parallel as mpu
from ..models import TransformerConfig
from .engine import StageEngine

_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16,
           torch.float16: torch.float16, torch.bfloat16: torch.bfloat16}


class Trainer:
    def __init__(self, model: str, batch_size: int, tp: int = 1, pp: int = 1,
                 batch_slices: Optional[Sequence[int]] = None,
                 seq_slices: Optional[Sequence[int]] = None, dtype="fp16",
                 n_layers: Optional[int] = None, activation: str = "gelu", use_graph=None,
                 tp_comm: str = "nccl", dp_comm: str = "nccl", lr: float = 1e-10, seed: int = 0, init: str = "device",
                 loss_scale: float = 128.0):
        if dist.is_initialized():
            if not mpu.model_parallel_is_initialized():
                mpu.initialize_model_parallel(tp, pp, verbose=False)
        elif tp * pp != 1:
            raise RuntimeError("tp*pp > 1 needs torch.distributed to be initialised")
        self.topo = mpu.get_topology()
        self.config = TransformerConfig.from_predefined_model(
            model, n_devices=self.topo.world_size, batch_size=batch_size, n_layers=n_layers,
            activation=activation)
        if isinstance(seq_slices, str):
            if seq_slices != "auto":
                raise ValueError("seq_slices is a list of lengths or 'auto'")
            # slice schedule from the dynamic program over the B200 kernel model
            from ..planner.latency_model import auto_schedule
            batch_slices, seq_slices, _ = auto_schedule(model, batch_size, tp, pp,
                                                        fused_tp=tp_comm == "fused", n_layers=n_layers)
        batch_slices = list(batch_slices) if batch_slices else [batch_size]
        seq_slices = list(seq_slices) if seq_slices else [self.config.seq_len]
        self.dtype = _DTYPES[dtype]
        self.seed = seed
        self.engine = StageEngine(self.config, batch_slices, seq_slices, dtype=self.dtype,
                                  loss_scale=loss_scale, lr=lr, seed=seed, init=init,
                                  use_graph=use_graph, tp_comm=tp_comm, dp_comm=dp_comm)
        self._staging = None
        # host mirror of the device status word (bounded device waits report through it)
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_event = None

    @property
    def is_first_stage(self) -> bool:
        return self.engine.is_first

    @property
    def is_last_stage(self) -> bool:
        return self.engine.is_last

    def synthetic_input(self, step: int, pinned: bool = False) -> Optional[torch.Tensor]:
        """N(0,1) hidden states on the host for this replica (None on later stages).  All
        tensor-parallel ranks of a replica draw the same values (seeded by replica and step)."""
        if not self.is_first_stage:
            return None
        c = self.config
        g = torch.Generator().manual_seed(1000003 * (self.seed + 1) + 7919 * self.engine.dp_idx + step)
        x = torch.randn(c.seq_len, c.batch_size, c.embedding_dim, generator=g).to(self.dtype)
        return x.pin_memory() if pinned else x

    def load_input(self, x: Optional[torch.Tensor]) -> None:
        if self.is_first_stage and x is not None:
            self.engine.set_input(x)

    def train_step(self, x: Optional[torch.Tensor] = None) -> Optional[float]:
        """One iteration end to end.  ``x`` is the replica's host (ideally pinned) or device
        input on first-stage ranks; returns the loss as a Python float on last-stage ranks."""
        self._raise_on_device_timeout()          # status of the previous step (already on the host)
        self.load_input(x)
        self.engine.step()
        if self.is_last_stage:
            # one synchronising read brings back the loss and the status word together
            both = torch.stack([self.engine.loss().reshape(()),
                                self.engine.status[0].to(torch.float32)]).tolist()
            self._check_code(int(both[1]))
            return float(both[0])
        self._status_host.copy_(self.engine.status, non_blocking=True)
        self._status_event = torch.cuda.Event()
        self._status_event.record()
        return None

    def _check_code(self, code: int) -> None:
        if code != 0:
            from ..ops.lib import CHECK_CODES, CheckFailed, CommTimeout
            self.engine.status.zero_()
            if code in CHECK_CODES:
                raise CheckFailed(f"an index check of the checked kernel build failed during the "
                                  f"step (code {code})")
            raise CommTimeout(f"a device-side wait timed out during the step (code {code}): "
                              "a peer did not reach the same kernel within the wait limit")

    def _raise_on_device_timeout(self) -> None:
        """Raise :class:`CommTimeout` if the previous step left a time-out code in the status
        word.  Ranks that do not read a loss learn of it here, one step later, without ever
        stalling the host on the device."""
        if self._status_event is not None:
            self._status_event.synchronize()
            self._status_event = None
            self._check_code(int(self._status_host[0]))

    def finish(self) -> None:
        """Wait for the device and surface a pending time-out (call after the last step)."""
        torch.cuda.synchronize()
        self._status_event = None
        self._check_code(int(self.engine.status.item()))

    def close(self) -> None:
        """Free the engine's peer-mapped memory and forget the parallel layout, so that another
        Trainer with a different layout can be built in the same process (collective)."""
        self.engine.close()
        self.engine = None
        mpu.destroy_model_parallel()

    def compute_grads(self, x: Optional[torch.Tensor] = None):
        self.load_input(x)
        self.engine.compute_grads()
        return self.engine.named_grads()
