"""Symmetric-memory data plane: buffers that every rank of a process group maps into its own
address space (CUDA IPC over NVLink / NVSwitch), plus a small control block per rank with barrier
flags and result slots.  The fused compute+collective kernels take the per-rank pointer tables
built here and move data with plain peer loads and stores.

Plumbing only goes through ``torch.distributed`` (one ``all_gather_object`` of the IPC handles per
buffer); the reference has no counterpart: its collectives are all ``torch.distributed`` calls
(Merak/core/mpu/mappings.py:30-120, Merak/core/merak_engine.py:552-621)."""
from __future__ import annotations

import ctypes
import socket
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

MAX_RANKS = 16


class _DeviceMemory:
    """Exposes a raw device allocation through ``__cuda_array_interface__`` so that a torch tensor
    can alias it (the tensor keeps this object, and with it the owner, alive)."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SymmBuffer:
    """One allocation per rank, mapped by all ranks.  ``ptrs[k]`` is rank k's buffer as seen from
    this process; ``tensor`` aliases the local one."""

    def __init__(self, local_ptr: int, nbytes: int, ptrs: List[int], rank: int, dtype, device, owner):
        self.local_ptr, self.nbytes, self.ptrs, self.rank = local_ptr, nbytes, ptrs, rank
        raw = torch.as_tensor(_DeviceMemory(local_ptr, nbytes, owner), device=device)
        self.tensor = raw.view(dtype)
        self.table = (ctypes.c_void_p * len(ptrs))(*ptrs)       # host pointer table handed to launches


class SymmGroup:
    """Symmetric allocations of one process group (all ranks on one node)."""

    def __init__(self, group, device: torch.device):
        self.group = group
        self.device = device
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._local: List[int] = []
        self._opened: List[int] = []
        self.epoch = 0
        lib = _lib.kernels()
        self.ctrl = self.alloc(int(lib.mrk_symm_ctrl_bytes()), torch.uint8)

    # -- availability ---------------------------------------------------------------------------
    @staticmethod
    def create(group, device: torch.device) -> Optional["SymmGroup"]:
        """Collective over ``group``.  Returns None on every rank unless all ranks can map each
        other's memory (CUDA devices of one host, kernel library present)."""
        n = dist.get_world_size(group)
        ok = device.type == "cuda" and 1 < n <= MAX_RANKS
        hosts: List[Optional[str]] = [None] * n
        dist.all_gather_object(hosts, (socket.gethostname(), torch.cuda.current_device() if ok else -1), group=group)
        ok = ok and len({h for h, _ in hosts}) == 1 and len({d for _, d in hosts}) == n
        sg = None
        if ok:
            try:
                sg = SymmGroup(group, device)
            except Exception:                          # IPC refused (no peer access, containers, ...)
                sg = None
        flag = torch.tensor([1 if sg is not None else 0], device=device if device.type == "cuda" else "cpu")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            if sg is not None:
                sg.close()
            return None
        return sg

    # -- allocation -----------------------------------------------------------------------------
    def alloc(self, nbytes: int, dtype=torch.uint8) -> SymmBuffer:
        """Collective: every rank allocates ``nbytes`` (zeroed) and maps everyone else's."""
        lib = _lib.kernels()
        nbytes = (int(nbytes) + 255) // 256 * 256
        with torch.cuda.device(self.device):
            out = ctypes.c_void_p()
            _lib.check(lib.mrk_symm_alloc(nbytes, ctypes.byref(out)), "mrk_symm_alloc")
            local = int(out.value)
            self._local.append(local)
            hbytes = int(lib.mrk_ipc_handle_bytes())
            hbuf = (ctypes.c_ubyte * hbytes)()
            _lib.check(lib.mrk_ipc_get_handle(local, hbuf), "mrk_ipc_get_handle")
            handles: List[Optional[bytes]] = [None] * self.n
            dist.all_gather_object(handles, bytes(hbuf), group=self.group)
            ptrs = []
            for k, h in enumerate(handles):
                if k == self.rank:
                    ptrs.append(local)
                    continue
                src = (ctypes.c_ubyte * hbytes).from_buffer_copy(h)
                p = ctypes.c_void_p()
                _lib.check(lib.mrk_ipc_open(src, ctypes.byref(p)), "mrk_ipc_open")
                self._opened.append(int(p.value))
                ptrs.append(int(p.value))
        return SymmBuffer(local, nbytes, ptrs, self.rank, dtype, self.device, self)

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def barrier(self, which: int = 15, budget_ms: int = 5000):
        """Device-side barrier over the group on the current stream (bounded wait)."""
        _lib.check(_lib.kernels().mrk_symm_barrier(self.ctrl.table, self.n, self.rank, which, self.next_epoch(), 1,
                                                   budget_ms, _lib.stream_ptr()), "mrk_symm_barrier")

    def close(self):
        lib = _lib.kernels()
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            lib.mrk_ipc_close(p)
        self._opened = []
        # local allocations stay alive while tensors may still alias them; they go with the process
