"""Chunked MoE layer plan: buffers are allocated once (like a RAF OpEnv, whose constructor sees the
concrete shapes), `dispatch` / `combine` only enqueue kernels."""
import ctypes

import torch

from . import _capi
from ._capi import check
from .ops import _DT, _ptr, _stream


class ChunkedMoE:
    """Dispatch and combine of S tokens in n_chunks chained chunks sharing one [E,C,M] buffer.

    Mirrors the reference's partitioned MoE layer (moe_encode x n with capacity factor cf*n,
    src/pass/dist_optimization/partition_exprs.cc:1709-1795) without its merge/redispatch step.
    """

    def __init__(self, S, M, E, k=1, capacity_factor=1.0, n_chunks=1, dtype=torch.float16,
                 gate_dtype=torch.float32, device="cuda"):
        if S % n_chunks:
            raise ValueError("S must be divisible by n_chunks")
        self.S, self.M, self.E, self.k, self.n = S, M, E, k, n_chunks
        self.cf = float(capacity_factor)
        self.dtype, self.gate_dtype = dtype, gate_dtype
        self.device = torch.device(device)
        L = _capi.lib()
        self.Sp = S // n_chunks
        self.C = L.lancet_moe_capacity(self.Sp, E, self.cf * n_chunks, k)
        d = self.device
        self.gates_s = torch.empty((n_chunks, k, self.Sp), dtype=torch.float32, device=d)
        self.idx_loc = torch.empty((n_chunks, 2 * k, self.Sp), dtype=torch.int32, device=d)
        self.capused = torch.zeros((n_chunks + 1, E), dtype=torch.int32, device=d)
        self.elems = torch.zeros((n_chunks, E), dtype=torch.uint64, device=d)
        self.dispatched = torch.empty((E, self.C, M), dtype=dtype, device=d)
        self.out = torch.empty((S, M), dtype=dtype, device=d)
        nws = L.lancet_moe_dispatch_chunked_workspace_bytes(S, E, k, n_chunks)
        self.ws = torch.empty(max(nws, 256), dtype=torch.uint8, device=d)

    def dispatch(self, x, gate):
        check(_capi.lib().lancet_moe_dispatch_chunked(
            _ptr(x), _ptr(gate), _DT[gate.dtype], self.cf, self.S, self.M, self.E, self.k, self.n, _DT[x.dtype],
            _ptr(self.gates_s), _capi.F32, _ptr(self.idx_loc), _ptr(self.capused), _ptr(self.elems),
            _ptr(self.dispatched), _ptr(self.ws), self.ws.numel(), _stream(x)))
        return self.dispatched

    def scatter(self, x, out=None):
        """Move another [S, M] tensor with the routing of the last `dispatch` (no gating)."""
        out = self.dispatched if out is None else out
        check(_capi.lib().lancet_moe_scatter_chunked(_ptr(x), _ptr(self.idx_loc), _ptr(self.capused), _ptr(out), self.S, self.M,
                                                     self.C, self.E, self.k, self.n, _DT[x.dtype], _stream(x)))
        return out

    def combine(self, expert_out=None, out=None):
        eo = self.dispatched if expert_out is None else expert_out
        out = self.out if out is None else out
        check(_capi.lib().lancet_moe_combine_chunked(
            _ptr(eo), _ptr(self.gates_s), _capi.F32, _ptr(self.idx_loc), self.S, self.M, self.C, self.E, self.k,
            self.n, _DT[eo.dtype], _ptr(out), _stream(eo)))
        return out
