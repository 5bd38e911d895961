"""Fused dispatch/exchange/combine over peer memory: W virtual ranks on one GPU against the oracle
(per-rank chained encode -> simulated all-to-all -> experts -> all-to-all -> decode), the bounded
barrier wait, and (when the box has >= 2 GPUs) real processes over NVLink."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import lancet_b200 as LB
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def oracle_rank_encode(x, gate, E, k, n, cf):
    """Chained chunks with locations as rows of the shared buffer (what the device produces)."""
    S, M = x.shape
    Sp = S // n
    C = O.capacity(Sp, E, cf * n, k)
    disp = np.zeros((E, C, M), x.dtype)
    cap = np.zeros(E, np.int32)
    parts = []
    for i in range(n):
        sl = slice(i * Sp, (i + 1) * Sp)
        gs, il, cap2, el = O.moe_gate(gate[sl], cap, C, M, k)
        disp += O.moe_encode_fwd(il, x[sl], E, C, cap, global_loc=True)
        raw = O.moe_gate(gate[sl], np.zeros(E, np.int32), 1 << 30, M, k)[1]
        gl = il.copy()
        for j in range(k):
            gl[2 * j + 1] = il[2 * j + 1] + cap[raw[2 * j]]
        parts.append((gs, gl))
        cap = cap2
    return disp, parts, C


@pytest.mark.parametrize("W,S,M,k,n,cf,remote_zero", [(2, 1024, 64, 2, 4, 1.25, True), (4, 512, 32, 2, 2, 1.25, True),
                                                      (4, 512, 32, 1, 1, 1.0, True), (2, 1024, 64, 2, 4, 1.25, False)])
def test_virtual_ranks_match_oracle(W, S, M, k, n, cf, remote_zero):
    LE = 2
    E = LE * W
    shared = {}
    plans = [LB.DistChunkedMoE(S, M, k, cf, n, torch.float16, DEV, LE, fabric=LB.LocalFabric(W, r, shared),
                               remote_zero=remote_zero) for r in range(W)]
    rng = np.random.default_rng(W * 100 + S + k)
    xs = [torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).half() for _ in range(W)]
    gates = [torch.softmax(torch.from_numpy(rng.standard_normal((S, E)).astype(np.float32)), dim=1) for _ in range(W)]
    for rep in range(2):                       # two steps: exercises the double-buffered receive side
        for p in plans:                        # stale contents must not survive
            for b in p.recv:
                b.fill_(5.0)
        for r, p in enumerate(plans):          # virtual ranks: all sends, then all local finishes
            p.dispatch_send(xs[r].to(DEV), gates[r].to(DEV))
        recvs = [p.dispatch_finish() for p in plans]
        torch.cuda.synchronize()
        enc = [oracle_rank_encode(xs[r].numpy(), gates[r].numpy(), E, k, n, cf) for r in range(W)]
        want_recv = O.all_to_all([e[0] for e in enc])               # [E,C,M] viewed [W, LE*C*M]
        for r in range(W):
            assert plans[r].C == enc[r][2]
            np.testing.assert_array_equal(recvs[r].cpu().numpy().reshape(E, -1, M), want_recv[r])
        # experts: multiply by (1 + global expert id), written to the symmetric output buffer
        for r, p in enumerate(plans):
            scale = torch.arange(1, LE + 1, device=DEV, dtype=torch.float32).add(r * LE).view(1, LE, 1, 1)
            p.expert_out.copy_((recvs[r].float() * scale).half())
        outs = [p.combine(from_expert_out=True).cpu().numpy() for p in plans]
        # oracle: expert outputs travel back through the all-to-all, then decode
        eo = [(want_recv[r].reshape(W, LE, -1, M).astype(np.float32) *
               (np.arange(1, LE + 1, dtype=np.float32) + r * LE).reshape(1, LE, 1, 1)).astype(np.float16)
              for r in range(W)]
        back = O.all_to_all([e.reshape(E, -1, M) for e in eo])
        for r in range(W):
            ref = np.concatenate([O.moe_decode_fwd(back[r].astype(np.float32), gs, gl) for gs, gl in enc[r][1]])
            np.testing.assert_array_equal(outs[r].astype(np.float32), torch.from_numpy(ref).half().float().numpy())
        # identity experts read the receive buffers directly
        outs_id = [p.combine().cpu().numpy() for p in plans]
        idb = O.all_to_all([w.reshape(E, -1, M) for w in want_recv])
        for r in range(W):
            ref = np.concatenate([O.moe_decode_fwd(idb[r].astype(np.float32), gs, gl) for gs, gl in enc[r][1]])
            np.testing.assert_array_equal(outs_id[r].astype(np.float32), torch.from_numpy(ref).half().float().numpy())


def test_barrier_wait_is_bounded():
    """A peer that never arrives: the wait gives up after its limit, the status word names the peer,
    the context stays usable.  (Host-made failure: the second rank's flag is simply never written.)"""
    import ctypes
    from lancet_b200 import _capi
    L = _capi.lib()
    flags0 = torch.zeros(16, dtype=torch.int32, device=DEV)
    flags1 = torch.zeros(16, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    table = (ctypes.c_void_p * 16)(flags0.data_ptr(), flags1.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _capi.check(L.lancet_p2p_barrier(table, 2, 0, 1, 20_000_000, ctypes.c_void_p(status.data_ptr()), stream))
    t1.record()
    rc = L.lancet_p2p_status(ctypes.c_void_p(status.data_ptr()), stream)
    assert rc == _capi.ERR_TIMEOUT and b"rank 1" in L.lancet_last_error()
    assert 15.0 < t0.elapsed_time(t1) < 500.0
    assert flags1.cpu()[0].item() == 1                 # our own arrival was published
    # a world of one never waits
    status.zero_()
    _capi.check(L.lancet_p2p_barrier((ctypes.c_void_p * 16)(flags0.data_ptr()), 1, 0, 5, 20_000_000,
                                     ctypes.c_void_p(status.data_ptr()), stream))
    assert L.lancet_p2p_status(ctypes.c_void_p(status.data_ptr()), stream) == 0
    assert torch.ones(4, device=DEV).sum().item() == 4.0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_processes_over_nvlink():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "p2p_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "p2p worker ok" in r.stdout


def test_all_to_all_peer_memory_virtual_ranks():
    """tests/python/distributed/test_alltoall.py:22-59 pattern and a random payload, W virtual ranks."""
    W, n = 4, 4 * 1024
    shared = {}
    ops = [LB.SymmAllToAll(n * 4, DEV, fabric=LB.LocalFabric(W, r, shared)) for r in range(W)]
    rng = np.random.default_rng(9)
    bufs = [rng.standard_normal((W, n // W)).astype(np.float32) for _ in range(W)]
    bufs[0][:] = 1.0
    xs = [torch.from_numpy(b).to(DEV) for b in bufs]
    for r in range(W):
        ops[r].send(xs[r])
    torch.cuda.synchronize()
    want = O.all_to_all(bufs)
    for r in range(W):
        np.testing.assert_array_equal(ops[r].recv_view(xs[r]).cpu().numpy(), want[r])


def test_all_to_allv_peer_memory_virtual_ranks():
    """Counts (i + j + rank) % 4 + 1 as tests/python/distributed/test_alltoall.py:61-122, plus ragged
    counts that end inside a 16-byte word and a full chunk."""
    W, nch, chunk = 2, 3, 24
    shared = {}
    ops = [LB.SymmAllToAll(W * nch * chunk * 4, DEV, fabric=LB.LocalFabric(W, r, shared), n_chunks=nch) for r in range(W)]
    rng = np.random.default_rng(10)
    bufs = [rng.standard_normal((W, nch * chunk)).astype(np.float32) for _ in range(W)]
    scs = [np.array([(i + j + r) % 4 + 1 for i in range(W) for j in range(nch)], np.uint64) for r in range(W)]
    scs[0][1] = chunk
    scs[1][2] = 0
    scs[1][4] = 7
    xs = [torch.from_numpy(b).to(DEV) for b in bufs]
    for r in range(W):
        ops[r].recv_view(xs[r]).fill_(9.0)
    for r in range(W):
        ops[r].sendv(xs[r], torch.from_numpy(scs[r].astype(np.int64)).to(DEV))
    torch.cuda.synchronize()
    want, want_rc = O.all_to_allv(bufs, scs, nch)
    for r in range(W):
        np.testing.assert_array_equal(ops[r].recv_view(xs[r]).cpu().numpy(), want[r])
        np.testing.assert_array_equal(ops[r].counts_view().cpu().numpy().astype(np.uint64), want_rc[r])


def test_peer_dispatch_rejects_unaligned_rows():
    """Rows that are not a multiple of 16 bytes cannot take the 16-byte peer stores: reported, not launched."""
    plan = LB.DistChunkedMoE(64, 12, 1, 1.0, 1, torch.float16, DEV, 2, fabric=LB.LocalFabric(1, 0, {}))
    x = torch.zeros((64, 12), dtype=torch.float16, device=DEV)
    gate = torch.softmax(torch.randn((64, 2), device=DEV), dim=1)
    with pytest.raises(LB.LancetError) as ei:
        plan.dispatch(x, gate)
    assert ei.value.code == 1 and "16 bytes" in str(ei.value)
    torch.cuda.synchronize()


def test_cta_limits_and_peer_copy():
    """Grid caps change how many CTAs run, never the result; lancet_peer_copy is a plain asynchronous copy."""
    import ctypes
    from lancet_b200 import _capi
    L = _capi.lib()
    W, n = 2, 1 << 16
    shared = {}
    ops = [LB.SymmAllToAll(n * 4, DEV, fabric=LB.LocalFabric(W, r, shared)) for r in range(W)]
    xs = [torch.randn((W, n // W), device=DEV) for _ in range(W)]
    outs = []
    try:
        for cap in (0, 3, 1000):
            _capi.check(L.lancet_set_cta_limits(cap, 0))
            for r in range(W):
                ops[r].recv_view(xs[r]).zero_()
            for r in range(W):
                ops[r].send(xs[r])
            torch.cuda.synchronize()
            outs.append([ops[r].recv_view(xs[r]).clone() for r in range(W)])
    finally:
        _capi.check(L.lancet_set_cta_limits(0, 0))
    for o in outs[1:]:
        for a, b in zip(o, outs[0]):
            assert torch.equal(a, b)
    assert L.lancet_set_cta_limits(-1, 0) == 1
    src = torch.randn(1000, device=DEV)
    dst = torch.zeros(1000, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _capi.check(L.lancet_peer_copy(ctypes.c_void_p(dst.data_ptr()), ctypes.c_void_p(src.data_ptr()), 4000, stream))
    torch.cuda.synchronize()
    assert torch.equal(src, dst)
    assert L.lancet_peer_copy(None, ctypes.c_void_p(src.data_ptr()), 16, stream) == 2
