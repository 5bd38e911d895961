"""Child process of tests/test_p2p_gpu.py::test_two_processes_over_nvlink (one rank per GPU)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import lancet_b200 as LB  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402
from tests.test_p2p_gpu import oracle_rank_encode  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    S, M, k, n, cf, LE = 2048, 256, 2, 4, 1.25, 2
    E = LE * world
    plan = LB.DistChunkedMoE(S, M, k, cf, n, torch.float16, dev, LE)
    xs, gates = [], []
    for r in range(world):
        rng = np.random.default_rng(1000 + r)
        xs.append(torch.from_numpy(rng.standard_normal((S, M)).astype(np.float32)).half())
        gates.append(torch.softmax(torch.from_numpy(rng.standard_normal((S, E)).astype(np.float32)), dim=1))
    enc = [oracle_rank_encode(xs[r].numpy(), gates[r].numpy(), E, k, n, cf) for r in range(world)]
    want_recv = O.all_to_all([e[0] for e in enc])
    back = O.all_to_all([w.reshape(E, -1, M) for w in want_recv])
    ref = np.concatenate([O.moe_decode_fwd(back[rank].astype(np.float32), gs, gl) for gs, gl in enc[rank][1]])
    for step in range(3):
        recv = plan.dispatch(xs[rank].to(dev), gates[rank].to(dev))
        out = plan.combine()
        torch.cuda.synchronize()
        plan.check()
        np.testing.assert_array_equal(recv.cpu().numpy().reshape(E, -1, M), want_recv[rank])
        np.testing.assert_array_equal(out.cpu().numpy().astype(np.float32),
                                      torch.from_numpy(ref).half().float().numpy())
    # whole layer: the two-stream pipelined schedule (exchange of chunk c+1 under the experts of chunk c, real flag
    # barriers between the ranks) gives exactly the results of the unpipelined one
    layer = LB.MoELayer(4096, 256, 512, 2, 1.25, 4, torch.bfloat16, dev, LE, seed=21)
    g = torch.Generator(device=dev).manual_seed(300 + rank)
    lx = torch.randn((4096, 256), device=dev, generator=g).bfloat16()
    lgate = torch.softmax(torch.randn((4096, E), device=dev, generator=g), dim=1)
    ldout = torch.randn((4096, 256), device=dev, generator=g).bfloat16()
    out0 = layer.forward(lx, lgate).clone()
    dx0, dg0 = [t.clone() for t in layer.backward(ldout)]
    w0 = [t.clone() for t in (layer.dw1, layer.dw2, layer.db1, layer.db2)]
    for step in range(3):
        out1 = layer.forward_pipelined(lx, lgate).clone()
        dx1, dg1 = [t.clone() for t in layer.backward_pipelined(ldout)]
    torch.cuda.synchronize()
    layer.moe.check()
    assert torch.equal(out0, out1) and torch.equal(dx0, dx1) and torch.equal(dg0, dg1)
    for a, b in zip(w0, (layer.dw1, layer.dw2, layer.db1, layer.db2)):
        assert torch.equal(a, b)
    assert int(LB.gemm_status(dev).item()) == 0
    dist.barrier()
    layer.moe.close()
    # the block with layer norm, gate projection and residual add inside the chunk pipeline (incremental gating: the
    # owners learn each stage's row layout just before its rows arrive) against the unchunked block, across two ranks
    res = []
    for pipeline in (False, True):
        moe = LB.MoE(2048, 256, 512, E, k=2, capacity_factor=1.25, n_chunks=4, dtype=torch.bfloat16, device=dev, local_experts=LE,
                     seed=7, pipeline=pipeline)
        torch.manual_seed(5)
        ln = torch.nn.LayerNorm(256).to(dev)
        with torch.no_grad():
            moe.wg.weight.copy_(torch.randn_like(moe.wg.weight) * 0.2)
        g = torch.Generator(device=dev).manual_seed(400 + rank)
        bx = torch.randn((2048, 256), device=dev, generator=g).requires_grad_(True)
        bdy = torch.randn((2048, 256), device=dev, generator=g)
        for step in range(2):
            for p in list(moe.parameters()) + [bx]:
                p.grad = None
            by = moe.block_forward(bx, ln)
            by.backward(bdy)
        torch.cuda.synchronize()
        moe.layer.moe.check()
        res.append((by.detach().clone(), bx.grad.clone(), moe.w1.grad.clone(), moe.w2.grad.clone()))
        dist.barrier()
        moe.layer.moe.close()
    for a, b in zip(*res):
        assert torch.equal(a, b)
    # stand-alone _all_to_all over NCCL: rank r sends rows filled with r+1, expects row i = i+1
    # (tests/python/distributed/test_alltoall.py:22-59 of the reference)
    comm = LB.Communicator(dev)
    x = torch.full((world, 4), float(rank + 1), device=dev)
    y = comm.all_to_all(x)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(y.cpu().numpy(), np.arange(1, world + 1, dtype=np.float32)[:, None] * np.ones((1, 4), np.float32))
    big = torch.from_numpy(np.random.default_rng(rank).standard_normal((world, 1 << 18)).astype(np.float32)).to(dev)
    back = comm.all_to_all(comm.all_to_all(big))
    torch.cuda.synchronize()
    assert torch.equal(back, big)
    # tuple form: three tensors of different types in one grouped exchange == three single exchanges
    tup = [big, torch.arange(world * 6, device=dev, dtype=torch.int32).view(world, 6) + 100 * rank,
           torch.randn(world * 10, device=dev).half()]
    got_t = comm.all_to_all_tuple(tup)
    torch.cuda.synchronize()
    for a, x in zip(got_t, tup):
        assert torch.equal(a, comm.all_to_all(x))
    # the same exchange over peer memory, and the count-aware variant
    sa = LB.SymmAllToAll(big.numel() * 4, dev, n_chunks=2)
    got = sa.all_to_all(big)
    torch.cuda.synchronize()
    assert torch.equal(got, comm.all_to_all(big))
    counts = torch.tensor([(i + j + rank) % 4 + 1 for i in range(world) for j in range(2)], dtype=torch.int64, device=dev)
    gv, rc = sa.all_to_allv(big, counts)
    torch.cuda.synchronize()
    sa.check()
    chunk = big.numel() // (world * 2)
    gvh, bigs = gv.cpu().numpy().reshape(world, 2, chunk), None
    for i in range(world):
        for j in range(2):
            c = (rank + j + i) % 4 + 1          # what rank i sent us for chunk j
            assert rc.cpu().numpy()[i * 2 + j] == c
            assert np.all(gvh[i, j, c:] == 0)
    # the NCCL transport of the count-aware exchange gives the same data and counts
    gn, rn = comm.all_to_allv(big, counts)
    torch.cuda.synchronize()
    assert torch.equal(gn, gv.view_as(gn)) and torch.equal(rn.view(torch.int64), rc.view(torch.int64))
    # the same two collectives through the RAF-style registry: RequestDistributed hands the OpEnv the communicator
    from lancet_b200 import raf, _capi
    _capi.lib().lancet_raf_set_communicator(comm.handle, rank, world)
    (y1,), name = raf.call("raf.op._all_to_all", [big])
    assert name == "raf.op.nccl._all_to_all" and torch.equal(y1, comm.all_to_all(big))
    (y2, c2), name = raf.call("raf.op._all_to_allv", [big], [counts.view(torch.uint64)])
    assert name == "raf.op.nccl._all_to_allv" and torch.equal(y2, gn) and torch.equal(c2.view(torch.int64), rn.view(torch.int64))
    _capi.lib().lancet_raf_set_communicator(None, 0, 1)
    comm.close()
    dist.barrier()
    sa.close()
    plan.close()
    if rank == 0:
        print("p2p worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
