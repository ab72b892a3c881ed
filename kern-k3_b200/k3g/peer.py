"""Symmetric buffers and peer address tables for the NVLink collectives (one process per GPU).

This is the stand-in for the part of the reference's external runtime that maps each rank's copy
of an `export`ed buffer into the other ranks and hands kernels a device array of u64 addresses
(xiaguan/kern-k3 scripts/gen_collectives_p2p.py:77-86).  Handles travel through
torch.distributed (any backend); memory is allocated and opened through the C ABI
(k3g_peer_alloc / k3g_peer_export / k3g_peer_open), so device memory is plain cudaMalloc memory
whose CUDA IPC handle is valid in the peer processes.

`Allocator` is the seam the CPU tests replace: the exchange and the table layout are host logic
and are exercised with gloo ranks and a fake allocator.
"""
import ctypes


def shard_rows(tokens, world):
    """Rows per rank, NCCL block order: rank r owns rows [r * own, (r + 1) * own), own = ceil(tokens / world)
    (xiaguan/kern-k3 source/k3_prefill.cu:1-11)."""
    return (tokens + world - 1) // world


def collective_units(tokens, world, width=7168, vec_per_block=32768):
    """The one grid width every collective of a replay shares, = the epoch increment
    (xiaguan/kern-k3 scripts/gen_collectives_rs.py:44-45: ceil(ceil(tokens / tp) * 7168 / 32768))."""
    return max(1, (shard_rows(tokens, world) * width + vec_per_block - 1) // vec_per_block)


class CudaAllocator:
    """Real allocator: cudaMalloc + CUDA IPC through the C ABI."""

    def __init__(self):
        from . import call
        self._call = call

    def alloc(self, nbytes):
        p = ctypes.c_void_p()
        self._call("k3g_peer_alloc", int(nbytes), p)
        return int(p.value)

    def export(self, ptr):
        h = (ctypes.c_ubyte * 64)()
        self._call("k3g_peer_export", ptr, h)
        return bytes(h)

    def open(self, handle):
        p = ctypes.c_void_p()
        self._call("k3g_peer_open", handle, p)
        return int(p.value)

    def close(self, ptr):
        self._call("k3g_peer_close", ptr)

    def free(self, ptr):
        self._call("k3g_peer_free", ptr)

    def upload_table(self, addrs):
        import torch
        return torch.tensor(addrs, dtype=torch.int64, device="cuda")


class SymmetricBuffer:
    """One rank's copy of an exported buffer plus the addresses of every rank's copy.

    ptr: this rank's device address; addrs[r]: rank r's copy as seen from this process (addrs[rank] == ptr);
    table: device array of those addresses (what the kernels take as `*_peer`)."""

    def __init__(self, name, nbytes, ptr, addrs, table, allocator, rank):
        self.name, self.nbytes, self.ptr, self.addrs, self.table = name, nbytes, ptr, addrs, table
        self._alloc, self._rank = allocator, rank

    def tensor(self, dtype, shape):
        """A torch view of this rank's copy (no ownership)."""
        import numpy as np
        import torch
        n = int(np.prod(shape))
        esz = torch.empty(0, dtype=dtype).element_size()
        assert n * esz <= self.nbytes

        class _Arr:
            __cuda_array_interface__ = {"shape": (n * esz,), "typestr": "|u1", "data": (self.ptr, False), "version": 3}
        return torch.as_tensor(_Arr(), device="cuda").view(dtype).view(*shape)

    def close_peers(self):
        """Unmap the peers' copies (this rank's own memory stays allocated: a peer may still have it mapped)."""
        for r, a in enumerate(self.addrs):
            if r != self._rank and a is not None:
                self._alloc.close(a)
        self.addrs = [a if r == self._rank else None for r, a in enumerate(self.addrs)]

    def free_own(self):
        if self.ptr is not None:
            self._alloc.free(self.ptr)
            self.ptr = None

    def release(self):
        self.close_peers()
        self.free_own()


class PeerGroup:
    """Creates symmetric buffers across the ranks of a torch.distributed group."""

    def __init__(self, rank, world, allocator=None, group=None):
        self.rank, self.world, self.group = rank, world, group
        self.alloc = allocator if allocator is not None else CudaAllocator()
        self.buffers = []

    def _all_gather(self, obj):
        if self.world == 1:
            return [obj]
        import torch.distributed as dist
        out = [None] * self.world
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def symmetric(self, name, nbytes):
        nbytes = (int(nbytes) + 255) // 256 * 256
        ptr = self.alloc.alloc(nbytes)
        records = self._all_gather((self.rank, name, nbytes, self.alloc.export(ptr)))
        addrs = []
        for r, (rr, nm, nb, handle) in enumerate(records):
            if rr != r or nm != name or nb != nbytes:
                raise RuntimeError("symmetric(%r, %d): rank %d announced (%r, %r, %r)" % (name, nbytes, r, rr, nm, nb))
            addrs.append(ptr if r == self.rank else self.alloc.open(handle))
        buf = SymmetricBuffer(name, nbytes, ptr, addrs, self.alloc.upload_table(addrs), self.alloc, self.rank)
        self.buffers.append(buf)
        return buf

    def release(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)      # nobody unmaps while a peer may still touch the memory
        for b in self.buffers:
            b.close_peers()
        if self.world > 1:
            dist.barrier(group=self.group)      # nobody frees exported memory while a peer still has it mapped
        for b in self.buffers:
            b.free_own()
        self.buffers = []
