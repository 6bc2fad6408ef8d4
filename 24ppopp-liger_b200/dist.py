"""Process-group plumbing: builds a liger communicator from a torch.distributed group.

torch.distributed is used only to exchange the fixed-size segment handles (the role MPI_Bcast of
the ncclUniqueId plays in the reference, src/communicator.h:29-37); all data-path traffic is done
by this library's own kernels over peer memory.
"""
import ctypes as C

from . import capi


class Comm:
    """Owns a liger_comm*; `data` is the device address of the local data region."""

    def __init__(self, rank, world_size, data_bytes, channels=8, group=None):
        import torch
        import torch.distributed as dist
        lib = capi.lib()
        self._lib = lib
        self.rank, self.world_size = rank, world_size
        h = C.c_void_p()
        capi.check(lib.liger_comm_create(C.byref(h), rank, world_size, data_bytes, channels))
        self.handle = h
        if world_size > 1:
            blob = (C.c_uint8 * capi.COMM_HANDLE_BYTES)()
            capi.check(lib.liger_comm_export(h, blob))
            mine = torch.tensor(list(blob), dtype=torch.uint8)
            if dist.get_backend(group) == "nccl":
                mine = mine.cuda()
            gathered = [torch.empty_like(mine) for _ in range(world_size)]
            dist.all_gather(gathered, mine, group=group)
            allb = bytes(torch.cat([g.cpu() for g in gathered]).tolist())
            capi.check(lib.liger_comm_connect(h, allb))
            dist.barrier(group=group)
        self.data = lib.liger_comm_data(h)
        self.data_bytes = lib.liger_comm_data_bytes(h)

    def tensor(self, offset_bytes, shape, dtype=None):
        """A torch view of the local data region (no copy, not owned)."""
        import torch
        dtype = dtype or torch.float16
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        assert offset_bytes + nbytes <= self.data_bytes
        # build a tensor aliasing device memory through the CUDA array interface
        class _Alias:
            pass
        a = _Alias()
        a.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (self.data + offset_bytes, False),
                                      "version": 2}
        t = torch.as_tensor(a, device="cuda")
        return t.view(dtype).reshape(shape)

    def close(self):
        if self.handle:
            self._lib.liger_comm_destroy(self.handle)
            self.handle = None
