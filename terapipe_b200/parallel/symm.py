"""Symmetric (peer-mapped) device memory for the fused tensor-parallel kernels.

Every rank of a group allocates buffers of the same size, exchanges their CUDA IPC handles
through ``torch.distributed`` and maps the peers' buffers, so a kernel on any rank can load
from and store to the same offset in every rank's buffer over NVLink.  Only plain loads and
stores (and system-scope release/acquire flags) are used on peer memory.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch
import torch.distributed as dist

from ..ops.lib import KernelError, cuda_lib


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class SymmetricBuffer:
    """``nbytes`` of zero-filled device memory on every rank of ``group``.

    ``ptrs[r]`` is the address, valid in this process, of rank ``r``'s buffer
    (``ptrs[group_rank]`` is the local one).  ``local`` is a uint8 torch view of the local buffer.
    """

    def __init__(self, nbytes: int, group=None):
        lib = cuda_lib()
        lib.tp_symm_alloc.restype = ctypes.c_void_p
        lib.tp_symm_alloc.argtypes = [ctypes.c_longlong]
        lib.tp_ipc_import.restype = ctypes.c_void_p
        lib.tp_ipc_import.argtypes = [ctypes.c_char_p]
        lib.tp_ipc_export.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        lib.tp_ipc_close.argtypes = [ctypes.c_void_p]
        lib.tp_symm_free.argtypes = [ctypes.c_void_p]
        self._lib = lib
        self.group = group
        self.nbytes = int(nbytes)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.local_ptr = lib.tp_symm_alloc(self.nbytes)
        if not self.local_ptr:
            raise KernelError(f"could not allocate {nbytes} bytes of peer-mappable memory")
        handle = ctypes.create_string_buffer(64)
        if lib.tp_ipc_export(self.local_ptr, handle) != 0:
            raise KernelError("cudaIpcGetMemHandle failed")
        gathered: List[bytes] = [None] * self.world
        dist.all_gather_object(gathered, handle.raw, group=group)
        self.ptrs: List[int] = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
                continue
            p = lib.tp_ipc_import(h)
            if not p:
                raise KernelError(f"could not map the buffer of group rank {r} (no peer access?)")
            self.ptrs.append(p)
        self.local = torch.as_tensor(_RawCudaBuffer(self.local_ptr, self.nbytes),
                                     device=torch.device("cuda", torch.cuda.current_device()))
        dist.barrier(group=group)

    def view(self, offset_bytes: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset_bytes:offset_bytes + nbytes].view(dtype).view(*shape)

    def ptr_array(self, offset_bytes: int = 0):
        """ctypes array of ``world`` pointers to ``offset_bytes`` inside every rank's buffer."""
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + offset_bytes
        return arr

    def close(self) -> None:
        """Unmap the peers' buffers and free the local one.  Collective over the group; call it
        between steps, with no kernel that uses the buffers in flight."""
        if self.local_ptr is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self._lib.tp_ipc_close(p)
        dist.barrier(group=self.group)
        self.local = None
        self._lib.tp_symm_free(self.local_ptr)
        self.local_ptr = None


class FusedAllReduceContext:
    """Staging tiles, flags and the call counter shared by all fused GEMM + all-reduce calls
    of one tensor-parallel group, plus a pool from which the matrices that receive reduced
    results are carved (they must sit at the same offset on every rank)."""

    TILE_BYTES = 128 * 128 * 2
    KMAX_TP = 8

    def __init__(self, group, max_rows: int, max_cols: int, pool_bytes: int):
        self.group = group
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_tiles = ((max_rows + 127) // 128) * ((max_cols + 127) // 128)
        # two halves: with two ranks the kernel exchanges partials in one hop and alternates the
        # half from call to call (a rank may start its next call while its peer still reduces)
        stage_bytes = 2 * self.tp * self.max_tiles * self.TILE_BYTES
        flag_a_bytes = self.max_tiles * self.KMAX_TP * 4
        flag_b_bytes = self.max_tiles * 4
        self._off_flag_a = stage_bytes
        self._off_flag_b = stage_bytes + flag_a_bytes
        self._off_pool = (self._off_flag_b + flag_b_bytes + 1023) // 1024 * 1024
        self.buf = SymmetricBuffer(self._off_pool + pool_bytes, group)
        self.stage_ptrs = self.buf.ptr_array(0)
        self.flag_a_ptrs = self.buf.ptr_array(self._off_flag_a)
        self.flag_b_ptrs = self.buf.ptr_array(self._off_flag_b)
        self._pool_used = 0
        self._pool_bytes = pool_bytes
        self.epoch = 0

    def alloc(self, shape, dtype):
        """Carve a matrix out of the pool; returns (local tensor view, byte offset in the pool)."""
        n = 1
        for s in shape:
            n *= s
        nbytes = (n * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        if self._pool_used + nbytes > self._pool_bytes:
            raise KernelError("symmetric pool exhausted")
        off = self._off_pool + self._pool_used
        self._pool_used += nbytes
        return self.buf.view(off, shape, dtype), off

    def out_ptrs(self, pool_offset_bytes: int):
        return self.buf.ptr_array(pool_offset_bytes)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def close(self):
        self.buf.close()
