"""Buffers that every rank of one box can address, for the head-sharded prefill whose epilogue stores its tiles
straight into the peers' output buffers (raftinfer_b200/csrc/peer.cu).  One process per GPU; the handles travel
through torch.distributed."""
from __future__ import annotations

import torch

from . import kernels as K


class _DevicePointer:
    """Lets torch view raw device memory without copying (the CUDA array interface)."""

    def __init__(self, pointer, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (pointer, False),
                                         "version": 3, "strides": None}


_TYPESTR = {torch.bfloat16: ("<u2", torch.uint16), torch.float32: ("<f4", torch.float32),
            torch.uint32: ("<u4", torch.uint32), torch.int32: ("<i4", torch.int32)}


class SharedBuffer:
    """`shape`/`dtype` device memory on this rank, mapped by every other rank.  `pointers[r]` is rank r's buffer as
    seen from this process; `local` is a torch view of this rank's own."""

    def __init__(self, shape, dtype, rank, world, dist, device):
        typestr, view_dtype = _TYPESTR[dtype]
        count = 1
        for n in shape:
            count *= n
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        self.rank, self.world = rank, world
        self._own, handle = K.shared_alloc(nbytes)
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle)
        else:
            handles[0] = handle
        self.pointers = [self._own if r == rank else K.shared_open(handles[r]) for r in range(world)]
        raw = torch.as_tensor(_DevicePointer(self._own, shape, typestr), device=device)
        self.local = raw.view(dtype) if view_dtype != dtype else raw
        self._dist = dist

    def close(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self._dist.barrier()  # nobody unmaps or frees while a peer may still store
        for r, pointer in enumerate(self.pointers):
            if r != self.rank:
                K.shared_close(pointer)
        if self.world > 1:
            self._dist.barrier()
        K.shared_free(self._own)
        self.pointers = []
