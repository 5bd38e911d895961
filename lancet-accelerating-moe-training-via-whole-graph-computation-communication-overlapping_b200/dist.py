"""Expert-parallel MoE layer plan over NVLink peer memory (one process per GPU).

Rank r of W owns experts [r*LE, (r+1)*LE).  Each rank maps every peer's receive buffer
[W][LE][C][M] once at construction (like RAF's communicator, which is created before the first step:
src/distributed/cuda/nccl_communicator.cc:27-60); afterwards `dispatch` and `combine` only enqueue
kernels.  `torch.distributed` is used for the one-time exchange of memory handles.
"""
import ctypes

import torch

from . import _capi
from ._capi import check
from .ops import _DT, _ptr, _stream

_TYPESTR = {torch.float32: "<f4", torch.float16: "<f2", torch.bfloat16: "<i2", torch.int32: "<i4"}


class _RawCuda:
    def __init__(self, ptr, nelem, typestr):
        self.__cuda_array_interface__ = {"shape": (nelem,), "typestr": typestr, "data": (ptr, False), "version": 2}


def tensor_from_ptr(ptr, shape, dtype, device):
    """A torch view of device memory owned by the library (no copy)."""
    n = 1
    for s in shape:
        n *= s
    t = torch.as_tensor(_RawCuda(ptr, n, _TYPESTR[dtype]), device=device)
    if dtype == torch.bfloat16:
        t = t.view(torch.bfloat16)
    return t.view(*shape)


def _up(v, a=256):
    return (v + a - 1) // a * a


class ProcessFabric:
    """Symmetric memory between the ranks of a torch.distributed group on one node (CUDA IPC)."""

    def __init__(self, device, group=None):
        import torch.distributed as dist
        self.dist, self.group, self.device = dist, group, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.real = True
        self._owned, self._opened = [], []

    def alloc(self, nbytes):
        L = _capi.lib()
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            check(L.lancet_symm_alloc(nbytes, ctypes.byref(ptr), handle))
            self._owned.append(ptr.value)
            handles = [None] * self.world
            self.dist.all_gather_object(handles, handle.raw, group=self.group)
            peers = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    peers.append(ptr.value)
                else:
                    p = ctypes.c_void_p()
                    check(L.lancet_symm_open(h, ctypes.byref(p)))
                    self._opened.append(p.value)
                    peers.append(p.value)
        return peers

    def close(self):
        L = _capi.lib()
        for p in self._opened:
            L.lancet_symm_close(ctypes.c_void_p(p))
        self._opened = []
        if self.world > 1:
            self.dist.barrier(group=self.group)
        for p in self._owned:
            L.lancet_symm_free(ctypes.c_void_p(p))
        self._owned = []


class LocalFabric:
    """W virtual ranks inside one process on one GPU (tests): `alloc` returns the same table of W
    buffers to every rank.  The flag barrier is skipped: the ranks' kernels run one after another
    on one stream, which already orders them (kernels that wait on one another must never be
    launched separately on one GPU)."""

    def __init__(self, world, rank, shared):
        self.world, self.rank, self.shared = world, rank, shared
        self.real = False
        self._n = 0

    def alloc(self, nbytes):
        key = self._n
        self._n += 1
        if key not in self.shared:
            self.shared[key] = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(self.world)]
        return [t.data_ptr() for t in self.shared[key]]

    def close(self):
        pass


class DistChunkedMoE:
    """Chunk-chained top-k dispatch and combine with the all-to-all fused into the kernels."""

    ROW_ALIGN = 256     # stage windows of the staged exchange end on whole tiles of the grouped GEMM (256 rows per CTA pair)

    def __init__(self, S, M, k=2, capacity_factor=1.25, n_chunks=4, dtype=torch.float16, device="cuda",
                 local_experts=2, fabric=None, group=None, timeout_s=5.0, remote_zero=False, train=False):
        self.device = torch.device(device)
        self.fabric = fabric if fabric is not None else ProcessFabric(self.device, group)
        self.W, self.rank = self.fabric.world, self.fabric.rank
        if self.W > 16:
            raise ValueError("at most 16 ranks per node")
        if S % n_chunks:
            raise ValueError("S must be divisible by n_chunks")
        self.S, self.M, self.k, self.n, self.LE = S, M, k, n_chunks, local_experts
        self.E = local_experts * self.W
        self.cf = float(capacity_factor)
        self.dtype = dtype
        L = _capi.lib()
        self.Sp = S // n_chunks
        self.C = L.lancet_moe_capacity(self.Sp, self.E, self.cf * n_chunks, k)
        item = torch.empty((), dtype=dtype).element_size()
        self.recv_bytes = _up(self.W * self.LE * self.C * M * item)
        flag_bytes = _up(16 * 4)
        cnt_bytes = _up(self.W * self.LE * 4)
        self.train = train
        n_regions = 5 if train else 3            # recv x2, expert_out, and for training d_expert_out, d_expert_in
        chain_bytes = _up(self.W * (n_chunks + 1) * self.LE * 4)
        total = n_regions * self.recv_bytes + flag_bytes + 2 * cnt_bytes + 2 * chain_bytes
        bases = self.fabric.alloc(total)
        mk = lambda off: (ctypes.c_void_p * 16)(*[b + off for b in bases])
        self.peer_recv = [mk(0), mk(self.recv_bytes)]
        self.peer_eo = mk(2 * self.recv_bytes)
        self.peer_deo = mk(3 * self.recv_bytes) if train else None
        self.peer_dxe = mk(4 * self.recv_bytes) if train else None
        self.peer_flags = mk(n_regions * self.recv_bytes)
        cnt_off = n_regions * self.recv_bytes + flag_bytes
        self.peer_counts = [mk(cnt_off), mk(cnt_off + cnt_bytes)]
        chain_off = cnt_off + 2 * cnt_bytes
        self.peer_chain = [mk(chain_off), mk(chain_off + chain_bytes)]
        self.base = bases[self.rank]
        d = self.device
        self.gates_s = torch.empty((n_chunks, k, self.Sp), dtype=torch.float32, device=d)
        self.idx_loc = torch.empty((n_chunks, 2 * k, self.Sp), dtype=torch.int32, device=d)
        self.capused = torch.zeros((n_chunks + 1, self.E), dtype=torch.int32, device=d)
        self.elems = torch.zeros((n_chunks, self.E), dtype=torch.uint64, device=d)
        self.out = torch.empty((S, M), dtype=dtype, device=d)
        self.status = torch.zeros(1, dtype=torch.int32, device=d)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=d)   # barrier epoch, kept on the device (graph replay)
        nws = L.lancet_moe_dispatch_chunked_workspace_bytes(S, self.E, k, n_chunks)
        self.ws = torch.empty(max(nws, 256), dtype=torch.uint8, device=d)
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        self.parity = 0
        self.flags = 0 if remote_zero else _capi.P2P_NO_REMOTE_ZERO
        shape = (self.W, self.LE, self.C, M)
        self.recv = [tensor_from_ptr(self.base + i * self.recv_bytes, shape, dtype, d) for i in range(2)]
        self.expert_out = tensor_from_ptr(self.base + 2 * self.recv_bytes, shape, dtype, d)
        if train:
            self.d_expert_out = tensor_from_ptr(self.base + 3 * self.recv_bytes, shape, dtype, d)
            self.d_expert_in = tensor_from_ptr(self.base + 4 * self.recv_bytes, shape, dtype, d)
            self.dgates = torch.empty((n_chunks, k, self.Sp), dtype=torch.float32, device=d)
            self.dx = torch.empty((S, M), dtype=dtype, device=d)
        self.counts = [tensor_from_ptr(self.base + cnt_off + i * cnt_bytes, (self.W * self.LE,), torch.int32, d)
                       for i in range(2)]
        # staged (pipelined) exchange: the owners' view of how each chunk's rows arrive, and the row windows per stage
        G = self.W * self.LE
        self.chain = [tensor_from_ptr(self.base + chain_off + i * chain_bytes, (self.W, n_chunks + 1, self.LE),
                                      torch.int32, d) for i in range(2)]
        self.win_begin = torch.zeros((n_chunks, G), dtype=torch.int32, device=d)
        self.win_end = torch.zeros((n_chunks, G), dtype=torch.int32, device=d)
        self.swin_begin = torch.zeros((n_chunks, G), dtype=torch.int32, device=d)   # per stage, incremental protocol
        self.swin_end = torch.zeros((n_chunks, G), dtype=torch.int32, device=d)
        if self.fabric.real and self.W > 1:
            torch.cuda.synchronize(d)
            self.fabric.dist.barrier(group=self.fabric.group)

    # -- kernels -------------------------------------------------------------------------------
    def barrier(self):
        """All ranks' earlier kernels on this stream have finished when later kernels start."""
        if not self.fabric.real or self.W == 1:
            return
        check(_capi.lib().lancet_p2p_barrier_counted(self.peer_flags, self.W, self.rank, _ptr(self.epoch_dev),
                                                     self.timeout_ns, _ptr(self.status), _stream(self.status)))

    def dispatch(self, x, gate):
        """Gate all chunks, scatter rows into the owners' receive buffers, meet the peers.
        Returns this rank's expert input [W, LE, C, M] (block g from rank g)."""
        self.dispatch_send(x, gate)
        return self.dispatch_finish()

    def dispatch_send(self, x, gate):
        self.parity ^= 1
        check(_capi.lib().lancet_moe_dispatch_chunked_p2p(
            _ptr(x), _ptr(gate), _DT[gate.dtype], self.cf, self.S, self.M, self.LE, self.W, self.rank, self.k, self.n,
            _DT[x.dtype], _ptr(self.gates_s), _ptr(self.idx_loc), _ptr(self.capused), _ptr(self.elems),
            self.peer_recv[self.parity], self.peer_counts[self.parity], _ptr(self.ws), self.ws.numel(), self.flags,
            _stream(x)))

    def dispatch_finish(self):
        x = self.out
        self.barrier()
        if self.flags & _capi.P2P_NO_REMOTE_ZERO:
            # every source told us how many rows of its block are live; the rest is zero-filled here
            check(_capi.lib().lancet_moe_zero_tail(_ptr(self.recv[self.parity]), _ptr(self.counts[self.parity]),
                                                   self.M, self.C, self.W * self.LE, _DT[self.dtype], _stream(x)))
        return self.recv[self.parity]

    def combine(self, from_expert_out=False, out=None):
        """Gather the expert outputs of this rank's tokens from their owners and weight them.
        With from_expert_out the experts have written `self.expert_out`; otherwise the experts are
        the identity and the receive buffer itself is read back."""
        out = self.out if out is None else out
        if from_expert_out:
            self.barrier()
            table = self.peer_eo
        else:
            table = self.peer_recv[self.parity]
        check(_capi.lib().lancet_moe_combine_chunked_p2p(
            table, _ptr(self.gates_s), _ptr(self.idx_loc), self.S, self.M, self.C, self.LE, self.W, self.rank, self.k,
            self.n, _DT[self.dtype], _ptr(out), _stream(out)))
        return out

    # -- staged exchange: chunk c+1 travels while the experts work on chunk c ---------------------
    def stage_gate(self, gate):
        """Gate all chunks and tell every owner where each chunk's rows of this rank's blocks will lie."""
        self.parity ^= 1
        check(_capi.lib().lancet_moe_gate_chunked_p2p(
            _ptr(gate), _DT[gate.dtype], self.cf, self.S, self.M, self.LE, self.W, self.rank, self.k, self.n,
            _ptr(self.gates_s), _ptr(self.idx_loc), _ptr(self.capused), _ptr(self.elems), self.peer_chain[self.parity],
            _ptr(self.ws), self.ws.numel(), _stream(gate)))

    def stage_gate_chunks(self, gate_rows, c0, c1):
        """Incremental form of stage_gate: gate chunks [c0, c1) from the probabilities of their tokens only (the
        chunks must come in order, after `begin_step`) and tell the owners where their rows will lie."""
        check(_capi.lib().lancet_moe_gate_chunks_p2p(
            _ptr(gate_rows), _DT[gate_rows.dtype], self.cf, self.S, self.M, self.LE, self.W, self.rank, self.k, self.n, c0, c1,
            _ptr(self.gates_s), _ptr(self.idx_loc), _ptr(self.capused), _ptr(self.elems), self.peer_chain[self.parity],
            _ptr(self.ws), self.ws.numel(), _stream(gate_rows)))

    def begin_step(self):
        """Switch to the other set of receive buffers (stage_gate does this itself)."""
        self.parity ^= 1

    def stage_window(self, slot, c0, c1, prev_c0=-1):
        """Row window of the stage covering chunks [c0, c1), valid once that stage's barrier has been passed; prev_c0 is
        the first chunk of the stage before it.  Returns (row_begin, row_end) int32 [W*LE]; the last stage also fills
        the row totals."""
        cnt = self.counts[self.parity]
        check(_capi.lib().lancet_moe_stage_window(_ptr(self.chain[self.parity]), self.W, self.LE, self.n, self.ROW_ALIGN, prev_c0, c0, c1,
                                                  _ptr(self.swin_begin[slot]), _ptr(self.swin_end[slot]), _ptr(cnt),
                                                  _stream(cnt)))
        return self.swin_begin[slot], self.swin_end[slot]

    def zero_tail(self, buf=None):
        """Zero the rows of `buf` (default: the receive buffer) past each block's row total."""
        buf = self.recv[self.parity] if buf is None else buf
        cnt = self.counts[self.parity]
        check(_capi.lib().lancet_moe_zero_tail(_ptr(buf), _ptr(cnt), self.M, self.C, self.W * self.LE, _DT[self.dtype], _stream(cnt)))

    def stage_dispatch(self, x, c0, c1=None):
        """Scatter the rows of chunks [c0, c1) into the owners' receive buffers (follow with barrier())."""
        c1 = c0 + 1 if c1 is None else c1
        check(_capi.lib().lancet_moe_dispatch_rows_p2p(
            _ptr(x), _ptr(self.idx_loc), self.S, self.M, self.C, self.LE, self.W, self.rank, self.k, self.n, c0, c1,
            _DT[x.dtype], self.peer_recv[self.parity], _stream(x)))

    def stage_prepare(self, buf=None, zero=True):
        """After the first barrier of a pass: row windows of every stage, row totals, and (zero=True) zero-fill of the
        rows of `buf` (default: the receive buffer) that no token owns; callers that keep the zero-fill off their
        critical path pass zero=False and call zero_tail on another stream.  Returns (win_begin, win_end, counts)."""
        L = _capi.lib()
        cnt = self.counts[self.parity]
        if buf is None:
            buf = self.recv[self.parity]
            check(L.lancet_moe_stage_windows(_ptr(self.chain[self.parity]), self.W, self.LE, self.n, self.ROW_ALIGN,
                                             _ptr(self.win_begin), _ptr(self.win_end), _ptr(cnt), _stream(cnt)))
        if zero:
            check(L.lancet_moe_zero_tail(_ptr(buf), _ptr(cnt), self.M, self.C, self.W * self.LE, _DT[self.dtype], _stream(cnt)))
        return self.win_begin, self.win_end, cnt

    def stage_combine(self, c0, c1=None, out=None):
        """Combine the tokens of chunks [c0, c1) from the owners' expert outputs (rows must be complete: see MoELayer)."""
        c1 = c0 + 1 if c1 is None else c1
        out = self.out if out is None else out
        o = out[c0 * self.Sp:c1 * self.Sp]
        check(_capi.lib().lancet_moe_combine_chunked_p2p(
            self.peer_eo, _ptr(self.gates_s[c0:c1]), _ptr(self.idx_loc[c0:c1]), (c1 - c0) * self.Sp, self.M, self.C,
            self.LE, self.W, self.rank, self.k, c1 - c0, _DT[self.dtype], _ptr(o), _stream(o)))
        return o

    def stage_combine_backward(self, dout, c0, c1=None):
        c1 = c0 + 1 if c1 is None else c1
        d = dout[c0 * self.Sp:c1 * self.Sp]
        check(_capi.lib().lancet_moe_combine_bwd_p2p(
            _ptr(d), _ptr(self.gates_s[c0:c1]), _ptr(self.idx_loc[c0:c1]), self.peer_deo, self.peer_eo,
            _ptr(self.dgates[c0:c1]), (c1 - c0) * self.Sp, self.M, self.C, self.LE, self.W, self.rank, self.k, c1 - c0,
            _DT[self.dtype], _stream(d)))

    def stage_dispatch_backward(self, c0, c1=None):
        c1 = c0 + 1 if c1 is None else c1
        o = self.dx[c0 * self.Sp:c1 * self.Sp]
        check(_capi.lib().lancet_moe_combine_chunked_p2p(
            self.peer_dxe, None, _ptr(self.idx_loc[c0:c1]), (c1 - c0) * self.Sp, self.M, self.C, self.LE, self.W, self.rank,
            self.k, c1 - c0, _DT[self.dtype], _ptr(o), _stream(o)))
        return o

    # -- backward ------------------------------------------------------------------------------
    def combine_backward_send(self, dout, part=0):
        """Backward of combine, fused with the exchange: gate-weighted rows of dout go to the owners'
        d_expert_out buffers, dgates = <expert output row, dout row>.  part 1 sends the rows only, part 2 computes the
        gate gradients only (a schedule can start the expert GEMMs after part 1 and run part 2 beside them; part 2 must
        have finished before this rank passes the step's last barrier, because the owners then reuse expert_out)."""
        check(_capi.lib().lancet_moe_combine_bwd_part_p2p(
            _ptr(dout), _ptr(self.gates_s), _ptr(self.idx_loc), self.peer_deo, self.peer_eo, _ptr(self.dgates), self.S,
            self.M, self.C, self.LE, self.W, self.rank, self.k, self.n, _DT[self.dtype], part, _stream(dout)))

    def combine_backward_finish(self):
        """Meet the peers, zero the rows of d_expert_out that no token owns; returns (d_expert_out, dgates)."""
        self.barrier()
        check(_capi.lib().lancet_moe_zero_tail(_ptr(self.d_expert_out), _ptr(self.counts[self.parity]), self.M, self.C,
                                               self.W * self.LE, _DT[self.dtype], _stream(self.out)))
        return self.d_expert_out, self.dgates

    def dispatch_backward(self):
        """Backward of dispatch, fused with the exchange: dx[s] = sum of the d_expert_in rows of token s,
        gathered from their owners (the experts have written `self.d_expert_in`)."""
        self.barrier()
        check(_capi.lib().lancet_moe_combine_chunked_p2p(
            self.peer_dxe, None, _ptr(self.idx_loc), self.S, self.M, self.C, self.LE, self.W, self.rank, self.k,
            self.n, _DT[self.dtype], _ptr(self.dx), _stream(self.dx)))
        return self.dx

    def check(self):
        """Raises LancetError(LANCET_ERR_TIMEOUT) if a bounded wait ran out since construction."""
        check(_capi.lib().lancet_p2p_status(_ptr(self.status), _stream(self.status)))

    def close(self):
        torch.cuda.synchronize(self.device)
        self.recv, self.expert_out, self.counts, self.chain = None, None, None, None
        self.d_expert_out, self.d_expert_in = None, None
        self.fabric.close()
