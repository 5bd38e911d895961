"""Gating through the entry point that needs no workspace and allocates nothing.

Some hosts cannot give the library scratch memory: their memory pool already owns the device, the
operator was bound after workspaces were planned, or the step loop must avoid cudaMalloc's
device-wide synchronisation.  `lancet_moe_gate_static` keeps its scratch in a fixed array inside
the library.  This file is collected last so that a run stopping at the first failure has already
run every other test."""
import ctypes

import numpy as np
import pytest
import torch

import lancet_b200 as LB
from lancet_b200 import _capi
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _gate_both_ways(L, gate, cap0, C, M, k):
    S, E = gate.shape
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for static in (False, True):
        gs = torch.full((k, S), -7.0, dtype=torch.float32, device=DEV)
        il = torch.full((2 * k, S), -7, dtype=torch.int32, device=DEV)
        cap = torch.full((E,), -7, dtype=torch.int32, device=DEV)
        el = torch.zeros((E,), dtype=torch.int64, device=DEV)
        if static:
            rc = L.lancet_moe_gate_static(_ptr(gate), _capi.F32, S, E, k, _ptr(cap0), C, M, _ptr(gs), _capi.F32,
                                          _ptr(il), _ptr(cap), _ptr(el), 0, stream)
        else:
            nws = L.lancet_moe_gate_workspace_bytes(S, E, k)
            ws = torch.empty(nws, dtype=torch.uint8, device=DEV)
            rc = L.lancet_moe_gate(_ptr(gate), _capi.F32, S, E, k, _ptr(cap0), C, M, _ptr(gs), _capi.F32, _ptr(il),
                                   _ptr(cap), _ptr(el), _ptr(ws), nws, 0, stream)
        _capi.check(rc)
        torch.cuda.synchronize()
        outs.append([t.cpu().numpy() for t in (gs, il, cap, el)])
    return outs


def test_static_scratch_gate_equals_workspace_gate_twice():
    L = _capi.lib()
    assert L.lancet_moe_gate_static_max_bytes() == 4 << 20
    rng = np.random.default_rng(11)
    # two calls in a row with different shapes: the second one runs over the first one's leftovers
    for S, E, k, M in ((5000, 16, 2, 64), (3001, 7, 1, 8)):
        gate = torch.softmax(torch.from_numpy(rng.standard_normal((S, E)).astype(np.float32)), dim=1).to(DEV)
        cap0 = torch.from_numpy(rng.integers(0, 3, E).astype(np.int32)).to(DEV)
        C = LB.moe_capacity(S, E, 1.25, k)
        plain, static = _gate_both_ways(L, gate, cap0, C, M, k)
        for a, b in zip(plain, static):
            np.testing.assert_array_equal(a, b)     # integers and fp32 gates: bit-exact
        # and against the CPU oracle directly, so that a fault shared by both CUDA entry points cannot hide
        want = O.moe_gate(gate.cpu().numpy(), cap0.cpu().numpy(), C, M, k)
        for a, b in zip(static, want):
            np.testing.assert_array_equal(a.astype(np.int64) if a.dtype.kind in "iu" else a,
                                          np.asarray(b).astype(np.int64) if np.asarray(b).dtype.kind in "iu" else b)


def test_static_scratch_large_call_after_small_one():
    """More than 256 token tiles take the extra tile-scan pass, which reads per-tile histograms and totals from the
    scratch: run it right after a smaller call so that it meets that call's leftovers."""
    L = _capi.lib()
    rng = np.random.default_rng(12)
    for S, E, k, M in ((4000, 8, 1, 8), (70000, 8, 1, 8), (1000, 4, 2, 8), (66000, 6, 2, 8)):
        gate = torch.softmax(torch.from_numpy(rng.standard_normal((S, E)).astype(np.float32)), dim=1).to(DEV)
        cap0 = torch.zeros(E, dtype=torch.int32, device=DEV)
        C = LB.moe_capacity(S, E, 1.0, k)
        plain, static = _gate_both_ways(L, gate, cap0, C, M, k)
        for a, b in zip(plain, static):
            np.testing.assert_array_equal(a, b)
        want = O.moe_gate(gate.cpu().numpy(), np.zeros(E, np.int32), C, M, k)
        np.testing.assert_array_equal(static[1], want[1])


def test_static_scratch_size_boundary():
    """The largest token count whose scratch still fits the array is accepted, the next tile's worth is rejected."""
    L = _capi.lib()
    E, k = 8, 1
    limit = L.lancet_moe_gate_static_max_bytes()
    lo, hi = 1, 4_000_000
    while lo < hi:                                   # largest S with workspace_bytes(S) <= limit
        mid = (lo + hi + 1) // 2
        if L.lancet_moe_gate_workspace_bytes(mid, E, k) <= limit:
            lo = mid
        else:
            hi = mid - 1
    S_ok = lo
    assert L.lancet_moe_gate_workspace_bytes(S_ok, E, k) <= limit < L.lancet_moe_gate_workspace_bytes(S_ok + 1, E, k)
    gate = torch.softmax(torch.randn((S_ok + 1, E), device=DEV), dim=1)
    cap0 = torch.zeros(E, dtype=torch.int32, device=DEV)
    C = LB.moe_capacity(S_ok, E, 1.0, k)
    plain, static = _gate_both_ways(L, gate[:S_ok].contiguous(), cap0, C, 8, k)
    for a, b in zip(plain, static):
        np.testing.assert_array_equal(a, b)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    gs = torch.empty((k, S_ok + 1), dtype=torch.float32, device=DEV)
    il = torch.empty((2 * k, S_ok + 1), dtype=torch.int32, device=DEV)
    cap = torch.empty((E,), dtype=torch.int32, device=DEV)
    el = torch.zeros((E,), dtype=torch.int64, device=DEV)
    rc = L.lancet_moe_gate_static(_ptr(gate), _capi.F32, S_ok + 1, E, k, _ptr(cap0), C, 8, _ptr(gs), _capi.F32, _ptr(il),
                                  _ptr(cap), _ptr(el), 0, stream)
    assert rc == 1 and b"built-in array" in L.lancet_last_error()
    torch.cuda.synchronize()


def test_static_scratch_rejects_oversize():
    L = _capi.lib()
    one = ctypes.c_void_p(256)
    S = 2_000_000                                   # k*S*4 bytes alone exceed the 4 MiB array
    rc = L.lancet_moe_gate_static(one, _capi.F32, S, 8, 1, None, 10, 8, one, _capi.F32, one, one, one, 0, None)
    assert rc == 1
    assert b"built-in array" in L.lancet_last_error()
    torch.cuda.synchronize()
