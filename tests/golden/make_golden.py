"""Generate golden vectors from the reference's own torch-CPU MoE operators.

Run in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

It imports models/benchmark/pytorch/utils.py from the reference (FakeMoeEncodeOp,
FakeMoeDecodeOp: lines 313-501 of that file), runs them forward and backward on
seeded inputs and writes tests/golden/moe_ref_*.npz.  The fixtures are committed;
the GPU box has no reference checkout, so tests only ever read the .npz files.
"""
import hashlib
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_utils(ref_root):
    pkg = types.ModuleType("refbench")
    pkg.__path__ = []
    logger = types.ModuleType("refbench.logger")
    import logging
    logger.get_logger = lambda name: logging.getLogger(name)
    sub = types.ModuleType("refbench.pytorch")
    sub.__path__ = []
    sys.modules.update({"refbench": pkg, "refbench.logger": logger, "refbench.pytorch": sub})
    path = os.path.join(ref_root, "models", "benchmark", "pytorch", "utils.py")
    spec = importlib.util.spec_from_file_location("refbench.pytorch.utils", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["refbench.pytorch.utils"] = mod
    spec.loader.exec_module(mod)
    return mod


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def run_case(ref, name, S, E, M, seed, gate_kind, store_data):
    g = torch.Generator().manual_seed(seed)
    if gate_kind == "softmax":
        gate = torch.softmax(torch.randn(S, E, generator=g), dim=1)
    else:
        gate = torch.rand(S, E, generator=g)
    x = torch.randn(S, M, generator=g)
    C = (S + E - 1) // E
    x_r = x.clone().requires_grad_(True)
    gate_r = gate.clone().requires_grad_(True)
    gates_s, idx_loc, capused, elems, disp = ref.FakeMoeEncodeOp.apply(
        x_r, gate_r, torch.zeros(E, dtype=torch.int32), torch.ones(1))
    # cotangents for the encode backward
    d_gates = torch.randn(S, generator=g)
    d_disp = torch.randn(E, C, M, generator=g)
    torch.autograd.backward([gates_s, disp], [d_gates, d_disp])
    enc_dx, enc_dg = x_r.grad.clone(), gate_r.grad.clone()
    # decode on a random "expert output", forward and backward
    eo = torch.randn(E, C, M, generator=g).requires_grad_(True)
    gs_r = gates_s.detach().clone().requires_grad_(True)
    out = ref.FakeMoeDecodeOp.apply(eo, gs_r, idx_loc)
    d_out = torch.randn(S, M, generator=g)
    out.backward(d_out)
    dec_dx, dec_dg = eo.grad.clone(), gs_r.grad.clone()
    rec = dict(
        S=S, E=E, M=M, C=C, seed=seed,
        gate=gate.numpy(), gates_s=gates_s.detach().numpy(), idx_loc=idx_loc.numpy().astype(np.int32),
        capused=capused.numpy().astype(np.int32), elems=elems.numpy().astype(np.int64),
        sha_x=sha(x.numpy()), sha_disp=sha(disp.detach().numpy()), sha_out=sha(out.detach().numpy()),
        sha_enc_dx=sha(enc_dx.numpy()), sha_dec_dx=sha(dec_dx.numpy()),
        d_gates=d_gates.numpy(), enc_dg_nnz=np.array(np.nonzero(enc_dg.numpy())).astype(np.int32),
        enc_dg_val=enc_dg.numpy()[np.nonzero(enc_dg.numpy())], dec_dg=dec_dg.numpy(),
    )
    if store_data:
        rec.update(x=x.numpy(), disp=disp.detach().numpy(), d_disp=d_disp.numpy(), enc_dx=enc_dx.numpy(),
                   eo=eo.detach().numpy(), out=out.detach().numpy(), d_out=d_out.numpy(), dec_dx=dec_dx.numpy())
    np.savez_compressed(os.path.join(HERE, f"moe_ref_{name}.npz"), **rec)
    print(name, "C", C, "dropped", int((idx_loc[0] < 0).sum()), "capused", capused.tolist()[:8])


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    ref_root = sys.argv[1]
    ref = load_reference_utils(ref_root)
    # config "single-rank CPU MoE dispatch/combine": S=2048, E=8, M=512, softmax gate, seed 0
    run_case(ref, "c1_s2048_e8_m512", 2048, 8, 512, 0, "softmax", store_data=False)
    # reference test distribution gate~U[0,1) at its (S, E) grid, small M
    run_case(ref, "u_s1024_e32_m8", 1024, 32, 8, 1, "uniform", store_data=True)
    run_case(ref, "u_s2048_e64_m4", 2048, 64, 4, 2, "uniform", store_data=False)
    # ragged: S not a multiple of E, tiny
    run_case(ref, "rag_s193_e5_m4", 193, 5, 4, 3, "softmax", store_data=True)
    run_case(ref, "two_s64_e2_m16", 64, 2, 16, 4, "softmax", store_data=True)


if __name__ == "__main__":
    main()
