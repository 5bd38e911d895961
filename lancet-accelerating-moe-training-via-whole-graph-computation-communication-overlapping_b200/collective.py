"""`_all_to_all` / `_all_to_allv` host mirror (python/raf/distributed/op.py:158-170 of the reference:
`all_to_all(x)`, `all_to_allv(x, send_counts)`)."""
import ctypes

import torch

from . import _capi
from ._capi import check
from .dist import ProcessFabric, _up, tensor_from_ptr
from .ops import _ptr, _stream


class Communicator:
    """NCCL communicator for the stand-alone `_all_to_all` op.  Rank 0 creates the id; it is
    broadcast through the torch.distributed group (the reference broadcasts it over MPI,
    src/distributed/cuda/nccl_communicator.cc:35-43)."""

    def __init__(self, device, group=None):
        import torch.distributed as dist
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        L = _capi.lib()
        buf = ctypes.create_string_buffer(128)
        if self.rank == 0:
            check(L.lancet_comm_unique_id(buf))
        box = [buf.raw]
        dist.broadcast_object_list(box, src=0, group=group)
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(L.lancet_comm_init_rank(box[0], self.world, self.rank, ctypes.byref(self.handle)))

    def all_to_all(self, x, out=None):
        """out chunk i <- rank i's chunk `rank`; x is split evenly along its flattened extent."""
        if not x.is_cuda or not x.is_contiguous():
            raise ValueError("all_to_all needs a contiguous CUDA tensor")
        nbytes = x.numel() * x.element_size()
        if nbytes % self.world:
            raise ValueError("Cannot evenly distribute input tensor to all ranks.")
        out = torch.empty_like(x) if out is None else out
        check(_capi.lib().lancet_all_to_all(_ptr(x), _ptr(out), nbytes // self.world, self.handle, _stream(x)))
        return out

    def all_to_allv(self, x, send_counts):
        """`_all_to_allv` over NCCL: x viewed [W, n_chunks, chunk]; for (peer i, chunk j) only the first
        send_counts[i*n_chunks+j] elements count.  Returns (out, recv_counts); out is zero past the counts."""
        if not x.is_cuda or not x.is_contiguous() or not send_counts.is_cuda:
            raise ValueError("all_to_allv needs contiguous CUDA tensors")
        if send_counts.dtype not in (torch.int64, torch.uint64) or send_counts.numel() % self.world:
            raise ValueError("send_counts must be a 64-bit tensor of world * n_chunks entries")
        n_chunks = send_counts.numel() // self.world
        if x.numel() % (self.world * n_chunks):
            raise ValueError("Cannot evenly distribute input tensor to all ranks and chunks.")
        out = torch.empty_like(x)
        rc = torch.empty_like(send_counts)
        check(_capi.lib().lancet_all_to_allv(_ptr(x), _ptr(out), _ptr(send_counts), _ptr(rc), n_chunks, x.element_size(),
                                             x.numel() // (self.world * n_chunks), self.handle, _stream(x)))
        return out, rc

    def all_to_all_tuple(self, xs):
        """`_all_to_all` of a tuple of tensors in one grouped exchange; returns the list of outputs."""
        outs = [torch.empty_like(x) for x in xs]
        n = len(xs)
        sizes = [x.numel() * x.element_size() for x in xs]
        total = sum(sizes)
        ws = torch.empty(2 * max(total, 1), dtype=torch.uint8, device=xs[0].device)
        send = (ctypes.c_void_p * n)(*[x.data_ptr() for x in xs])
        recv = (ctypes.c_void_p * n)(*[o.data_ptr() for o in outs])
        nb = (ctypes.c_size_t * n)(*sizes)
        check(_capi.lib().lancet_all_to_all_tuple(send, recv, nb, n, _ptr(ws), ctypes.c_void_p(ws.data_ptr() + total),
                                                  total, self.handle, _stream(xs[0])))
        return outs

    def close(self):
        if self.handle:
            _capi.lib().lancet_comm_destroy(self.handle)
            self.handle = ctypes.c_void_p()


class SymmAllToAll:
    """All-to-all(v) over peer memory for tensors of a fixed byte size: the receive side lives in
    symmetric memory mapped once at construction."""

    def __init__(self, nbytes, device, fabric=None, group=None, n_chunks=1, timeout_s=5.0):
        self.device = torch.device(device)
        self.fabric = fabric if fabric is not None else ProcessFabric(self.device, group)
        self.W, self.rank = self.fabric.world, self.fabric.rank
        if nbytes % (self.W * n_chunks * 16):
            raise ValueError("tensor bytes must be a multiple of 16 * world * n_chunks")
        self.nbytes, self.n_chunks = nbytes, n_chunks
        data = _up(nbytes)
        cnt = _up(self.W * n_chunks * 8)
        bases = self.fabric.alloc(data + cnt + 256)
        mk = lambda off: (ctypes.c_void_p * 16)(*[b + off for b in bases])
        self.peer_recv, self.peer_counts, self.peer_flags = mk(0), mk(data), mk(data + cnt)
        self.base = bases[self.rank]
        self.cnt_off = data
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch = 0
        self.timeout_ns = int(timeout_s * 1e9)
        if self.fabric.real and self.W > 1:
            torch.cuda.synchronize(self.device)
            self.fabric.dist.barrier(group=self.fabric.group)

    def _barrier(self, like):
        if not self.fabric.real or self.W == 1:
            return
        self.epoch += 1
        check(_capi.lib().lancet_p2p_barrier(self.peer_flags, self.W, self.rank, self.epoch, self.timeout_ns,
                                             _ptr(self.status), _stream(like)))

    def recv_view(self, like):
        return tensor_from_ptr(self.base, tuple(like.shape), like.dtype, self.device)

    def counts_view(self):
        return tensor_from_ptr(self.base + self.cnt_off, (self.W * self.n_chunks * 2,), torch.int32,
                               self.device).view(torch.int64)

    def send(self, x):
        check(_capi.lib().lancet_all_to_all_p2p(_ptr(x), self.peer_recv, self.nbytes // self.W, self.W, self.rank,
                                                _stream(x)))

    def sendv(self, x, send_counts):
        """send_counts: device int64/uint64 [W * n_chunks] element counts."""
        chunk_elems = x.numel() // (self.W * self.n_chunks)
        check(_capi.lib().lancet_all_to_allv_p2p(_ptr(x), self.peer_recv, _ptr(send_counts), self.peer_counts,
                                                 self.n_chunks, x.element_size(), chunk_elems, self.W, self.rank,
                                                 _stream(x)))

    def all_to_all(self, x):
        self._barrier(x)          # peers have finished reading the previous result
        self.send(x)
        self._barrier(x)
        return self.recv_view(x)

    def all_to_allv(self, x, send_counts):
        self._barrier(x)
        self.sendv(x, send_counts)
        self._barrier(x)
        return self.recv_view(x), self.counts_view()

    def check(self):
        check(_capi.lib().lancet_p2p_status(_ptr(self.status), _stream(self.status)))

    def close(self):
        torch.cuda.synchronize(self.device)
        self.fabric.close()
