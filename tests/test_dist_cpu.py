"""World-size-2 gloo ranks on CPU: the exchange semantics the fused GPU path implements (layout
[W][LE][C][M], block g from rank g) checked with a real multi-process all-to-all against the
in-process simulator of the oracle, and the benchmark's reference arm under several ranks."""
import os
import subprocess
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(r, S, M, E):
    rng = np.random.default_rng(500 + r)
    return rng.standard_normal((S, M)).astype(np.float32), rng.random((S, E), dtype=np.float32)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    S, M, LE, k = 256, 8, 2, 2
    E = LE * world
    x, gate = _inputs(rank, S, M, E)
    gs, il, cap, el, disp = O.moe_encode(x, gate, np.zeros(E, np.int32), 1.25, k)
    send = torch.from_numpy(disp.copy())
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send)                 # equal split of the flattened [E,C,M] buffer
    expert_out = recv * float(rank + 1)                # this rank's experts
    back = torch.empty_like(expert_out)
    dist.all_to_all_single(back, expert_out)
    out = O.moe_decode_fwd(back.numpy(), gs, il)
    q.put((rank, recv.numpy(), out))
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_exchange_matches_simulator():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, 29541, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, recv, out = q.get(timeout=120)
        got[r] = (recv, out)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    S, M, LE, k = 256, 8, 2, 2
    E = LE * world
    enc = [O.moe_encode(*_inputs(r, S, M, E), np.zeros(E, np.int32), 1.25, k) for r in range(world)]
    recvs = O.all_to_all([e[4] for e in enc])
    backs = O.all_to_all([recvs[r] * float(r + 1) for r in range(world)])
    for r in range(world):
        np.testing.assert_array_equal(got[r][0], recvs[r])
        np.testing.assert_array_equal(got[r][1], O.moe_decode_fwd(backs[r], enc[r][0], enc[r][1]))
        # block g of rank r's receive buffer holds rank g's rows for r's experts [r*LE, (r+1)*LE)
        C = enc[r][4].shape[1]
        blocks = recvs[r].reshape(world, LE, C, M)
        for g in range(world):
            np.testing.assert_array_equal(blocks[g], enc[g][4][r * LE:(r + 1) * LE])


def test_reference_arm_prints_on_rank0_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--steps", "1", "--warmup", "1"], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip() == ""


def _staged_worker(rank, world, port, q):
    """The staged exchange as real ranks: chained gating, chain tables to the owners, one exchange per chunk;
    after stage c the rows inside the stage's windows must already hold their final values."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    S, M, LE, k, n, cf = 1024, 4, 2, 2, 4, 1.25
    E, Sp = LE * world, S // n
    C = O.capacity(Sp, E, cf * n, k)
    x, gate = _inputs(rank, S, M, E)
    cap = np.zeros(E, np.int32)
    chain = [cap.copy()]
    stage_bufs = []
    for c in range(n):
        sl = slice(c * Sp, (c + 1) * Sp)
        gs, il, cap2, el = O.moe_gate(gate[sl], cap, C, M, k)
        stage_bufs.append(O.moe_encode_fwd(il, x[sl], E, C, cap, global_loc=True))   # only this chunk's rows
        cap = cap2
        chain.append(cap.copy())
    chain = np.stack(chain)                                            # [n+1, E]
    # every owner learns the chain of every source before any row travels
    send = torch.from_numpy(np.ascontiguousarray(chain.reshape(n + 1, world, LE).transpose(1, 0, 2)))
    table = torch.empty_like(send)                                     # [W sources][n+1][LE]
    dist.all_to_all_single(table, send)
    begin, end, counts = O.stage_windows(table.numpy(), 16)
    recv = np.zeros((world, LE, C, M), np.float32)
    snaps = []
    for c in range(n):
        part = torch.from_numpy(stage_bufs[c].copy())
        got = torch.empty_like(part)
        dist.all_to_all_single(got, part)
        recv += got.numpy().reshape(world, LE, C, M)
        snaps.append(recv.copy())
    q.put((rank, recv, snaps, begin, end, counts))
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_staged_exchange_windows_only_cover_arrived_rows():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_staged_worker, args=(r, world, 29547, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        item = q.get(timeout=120)
        got[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    S, M, LE, k, n, cf = 1024, 4, 2, 2, 4, 1.25
    E, Sp = LE * world, S // n
    C = O.capacity(Sp, E, cf * n, k)
    # one-shot reference: chained chunks into one buffer, then a single all-to-all
    full = []
    for r in range(world):
        x, gate = _inputs(r, S, M, E)
        cap = np.zeros(E, np.int32)
        disp = np.zeros((E, C, M), np.float32)
        for c in range(n):
            sl = slice(c * Sp, (c + 1) * Sp)
            gs, il, cap2, el = O.moe_gate(gate[sl], cap, C, M, k)
            disp += O.moe_encode_fwd(il, x[sl], E, C, cap, global_loc=True)
            cap = cap2
        full.append(disp)
    want = O.all_to_all(full)
    for r in range(world):
        recv, snaps, begin, end, counts = got[r]
        final = want[r].reshape(world, LE, C, M)
        np.testing.assert_array_equal(recv, final)
        flat_final = final.reshape(world * LE, C, M)
        live = (np.abs(flat_final).sum(axis=2) > 0).sum(axis=1)
        np.testing.assert_array_equal(counts, live)                    # totals = rows that really arrived
        for c in range(n):
            snap = snaps[c].reshape(world * LE, C, M)
            for g in range(world * LE):
                np.testing.assert_array_equal(snap[g, begin[c, g]:end[c, g]], flat_final[g, begin[c, g]:end[c, g]])
