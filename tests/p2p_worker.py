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
    dist.barrier()
    plan.close()
    if rank == 0:
        print("p2p worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
