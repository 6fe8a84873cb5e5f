"""Sum of row-parallel partial outputs across the GPUs of one node over peer memory (NVLink), without NCCL.

One process per GPU.  Every rank allocates one buffer - a control block, a slot per reduction for its own partial
output and, per reduction, a receive area of 2 x world blocks -, shares it with the other ranks of the node through
CUDA IPC and maps theirs.  A row-parallel linear writes its partial output into its slot;
``PeerReducer.reduce(slot, out)`` then launches ``grb_peer_allreduce_bf16`` (``csrc/peer_reduce.cuh``): every rank
copies its partial into the peers' receive areas, announces it with a flag, waits for the peers' flags and adds all
partials in rank order (FP32): the same bits on every rank.  The launch allocates nothing, does not touch the host
and may be captured in a CUDA graph.

The reference has no counterpart (it runs a linear on one device, ``glc_loader/tbe_device_map.py:46-56``).
"""
from __future__ import annotations

import ctypes

from . import _native


class PeerError(RuntimeError):
    pass


class _RawDeviceBytes:
    """Device memory owned by somebody else, as the CUDA array interface describes it (torch.as_tensor takes a view)."""

    def __init__(self, pointer: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (pointer, False), "version": 2}


class PeerReducer:
    """``slots`` = {name: number of BF16 elements}; every rank must construct it with the same arguments and call
    ``reduce`` in the same order.  Construction is a collective over ``group`` (IPC handles are exchanged)."""

    def __init__(self, slots: dict, *, device=None, group=None, wait_limit_ns: int = 0):
        import torch
        import torch.distributed as dist

        if not dist.is_initialized():
            raise PeerError("torch.distributed is not initialised")
        self.lib = _native.lib()
        self.group = group
        self.wait_limit_ns = int(wait_limit_ns)   # 0: the library's default (two seconds)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise PeerError("at most 8 ranks")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        control = int(self.lib.grb_peer_control_bytes())
        control = (control + 255) // 256 * 256
        self.offsets, at = {}, control   # name -> (partial offset, elements, receive-area offset, block bytes)
        for name, elems in slots.items():
            if elems <= 0 or elems % 8:
                raise PeerError(f"slot {name}: the element count must be a positive multiple of 8")
            block = (2 * int(elems) + 255) // 256 * 256
            self.offsets[name] = (at, int(elems), at + block, block)
            at += block * (1 + 2 * self.world)
        # One device allocation of its own, zeroed (flags and call counter start at 0), mapped by every peer.  A
        # failure on one rank must not leave the others waiting in a collective: every rank goes through the same
        # collectives whatever happens locally, and all of them raise if any of them failed.
        self.bytes, self.local_ptr, self.buffer, self.pointers, self.opened = at, None, None, [], []
        error = None
        handle = (ctypes.c_uint8 * 64)()
        local = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            rc = self.lib.grb_peer_alloc(at, ctypes.byref(local), handle)
        if rc != 0:
            error = f"grb_peer_alloc failed with code {rc}"
        else:
            self.local_ptr = int(local.value)
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (int(self.device.index), bytes(handle) if error is None else None, at), group=group)
        if error is None:
            for r, (peer_device, peer_handle, peer_bytes) in enumerate(gathered):
                if peer_handle is None or peer_bytes != at:
                    error = f"rank {r} has no buffer to map or one of another size"
                    break
                if r == self.rank:
                    self.pointers.append(self.local_ptr)
                    continue
                mapped = ctypes.c_void_p()
                with torch.cuda.device(self.device):
                    rc = self.lib.grb_peer_open((ctypes.c_uint8 * 64).from_buffer_copy(peer_handle), ctypes.byref(mapped))
                if rc != 0:
                    error = f"cannot map the buffer of rank {r} (device {peer_device}) from device {self.device.index}: code {rc}"
                    break
                self.pointers.append(int(mapped.value))
                self.opened.append(int(mapped.value))
        agreed = torch.tensor([0 if error else 1], device=self.device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)   # also: nobody launches before everybody has mapped everything
        if not int(agreed.item()):
            self._release()
            raise PeerError(error or "another rank could not set up its peer buffers")
        self.buffer = torch.as_tensor(_RawDeviceBytes(self.local_ptr, at), device=self.device)   # a view, no copy
        self.controls = (ctypes.c_void_p * self.world)(*self.pointers)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def _release(self):
        import torch

        with torch.cuda.device(self.device):
            for p in self.opened:
                self.lib.grb_peer_close(p)
            self.opened = []
            self.buffer = None
            if self.local_ptr is not None:
                self.lib.grb_peer_free(self.local_ptr)
            self.local_ptr = None

    def close(self):
        """Unmaps the peers' buffers and frees the local one.  Collective: every rank calls it, none launches afterwards."""
        import torch
        import torch.distributed as dist

        if self.local_ptr is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)   # nobody unmaps or frees what somebody may still be writing to
        with torch.cuda.device(self.device):
            for p in self.opened:
                self.lib.grb_peer_close(p)
            self.opened = []
        dist.barrier(group=self.group)   # nobody frees what somebody still has mapped
        self._release()

    def slot(self, name: str, rows: int, cols: int):
        """The local slot as a BF16 [rows, cols] tensor: the linear's output buffer."""
        import torch

        at, elems, _, _ = self.offsets[name]
        if rows * cols > elems:
            raise PeerError(f"slot {name} holds {elems} elements, {rows * cols} asked for")
        return self.buffer[at:at + 2 * rows * cols].view(torch.bfloat16).view(rows, cols)

    def reduce(self, name: str, out, stream=None):
        """out[...] = sum over ranks of their slot `name` (as many elements as `out` has).  Asynchronous."""
        import torch

        at, elems, receive_at, block = self.offsets[name]
        n = out.numel()
        if n > elems or n % 8 or out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise PeerError("out must be a contiguous BF16 tensor of a multiple of 8 elements that fits the slot")
        receives = (ctypes.c_void_p * self.world)(*[p + receive_at for p in self.pointers])
        stream = torch.cuda.current_stream(self.device) if stream is None else stream
        rc = self.lib.grb_peer_allreduce_bf16(self.local_ptr + at, receives, self.controls, block, self.rank, self.world,
                                              out.data_ptr(), n, self.wait_limit_ns, self.status.data_ptr(), stream.cuda_stream)
        if rc != 0:
            raise PeerError(f"grb_peer_allreduce_bf16 failed with code {rc}")
        return out

    def check_status(self) -> int:
        """The device status word (synchronises); nonzero after a wait ran out: results must be discarded."""
        return int(self.status.item())
