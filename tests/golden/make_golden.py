"""Generate golden vectors from the reference's own torch-CPU MoE operators.

Run in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

It imports models/benchmark/pytorch/utils.py from the reference (FakeMoeEncodeOp,
FakeMoeDecodeOp: lines 313-501 of that file), runs them forward and backward on
seeded inputs and writes tests/golden/moe_ref_*.npz.  The fixtures are committed;
the GPU box has no reference checkout, so tests only ever read the .npz files.

Two more families:
  * top2_ref_*.npz: the reference's top-2 gate, `top2gating` of
    docker/resources/sharded_moe.py:253-324, imported with the absent `deepspeed`
    package stubbed and its Gumbel sampler returning zeros (the deterministic part of
    the gate).  The function's own local variables at its return (indices, locations
    before and after the capacity mask, normalised gates) are recorded through a
    profile hook, so every stored vector was computed by the reference's code.  For the
    small cases the dense dispatch and combine einsums of MOELayer.forward (:476-478,
    :512-514) are stored too.
  * top2chain_ref_*.npz: `top2gating` called on each of n consecutive token chunks (choices, locations before
    the capacity mask, probabilities per chunk), for checking the chained top-2 gate chunk by chunk.
  * chain_ref_*.npz: FakeMoeEncodeOp called on consecutive token chunks with each
    call's used capacity fed to the next one, the way the partition pass chains field 2
    of moe_encode (src/pass/dist_optimization/partition_exprs.cc:1784-1792).  With a
    non-zero used capacity only `indices_locations` and `gates_s` of that operator agree
    with the CUDA operator (drop rule loc >= C - used, tutel_moe_dispatch.cu:199-201);
    its `used_capacity` output is max(loc)+1 instead of min(used + count, C) (:207-209),
    so the chain is fed with the CUDA rule and only the two agreeing outputs are pinned.
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


def load_reference_sharded_moe(ref_root):
    """docker/resources/sharded_moe.py with `deepspeed` (absent here) stubbed: it is only used for timers and logging."""
    import logging
    ds = types.ModuleType("deepspeed")
    ds.__path__ = []
    du = types.ModuleType("deepspeed.utils")
    du.__path__ = []
    dt = types.ModuleType("deepspeed.utils.timer")
    dt.ThroughputTimer = type("ThroughputTimer", (), {})
    dt.SynchronizedWallClockTimer = type("SynchronizedWallClockTimer", (), {})
    du.logger = logging.getLogger("deepspeed")
    du.log_dist = lambda *a, **k: None
    du.timer = dt
    ds.utils = du
    sys.modules.update({"deepspeed": ds, "deepspeed.utils": du, "deepspeed.utils.timer": dt})
    path = os.path.join(ref_root, "docker", "resources", "sharded_moe.py")
    spec = importlib.util.spec_from_file_location("ref_sharded_moe", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    # noise off: the second choice becomes the plain argmax with the first one masked
    mod.gumbel_rsample = lambda shape, device: torch.zeros(shape, device=device)
    return mod


def call_with_locals(fn, *args):
    """Runs fn and returns (result, the function's local variables at its return)."""
    grabbed = {}

    def hook(frame, event, arg):
        if event == "return" and frame.f_code is fn.__code__:
            grabbed.update(frame.f_locals)

    sys.setprofile(hook)
    try:
        res = fn(*args)
    finally:
        sys.setprofile(None)
    return res, grabbed


def run_top2_case(sm, name, S, E, M, cf, seed, dense, spread=0.0):
    g = torch.Generator().manual_seed(seed)
    # `spread` tilts the logits towards the higher-numbered experts, so that their loads exceed the capacity and choices drop
    logits = (torch.randn(S, E, generator=g) + spread * torch.linspace(-1.0, 1.0, E)).requires_grad_(True)
    (l_aux, combine, mask, exp_counts), loc = call_with_locals(sm.top2gating, logits, cf)
    # gradient of the normalised gates with respect to the gate probabilities, by autograd through the reference's code
    d_gs = torch.randn(2, S, generator=g)
    (d_gate,) = torch.autograd.grad([loc["gates1_s"], loc["gates2_s"]], [loc["gates"]], [d_gs[0], d_gs[1]], retain_graph=True)
    logits = logits.detach()
    combine, loc = combine.detach(), {k: (v.detach() if torch.is_tensor(v) else v) for k, v in loc.items()}
    gates = loc["gates"]
    rows = torch.arange(S)
    i1, i2 = loc["indices1_s"], loc["indices2_s"]
    # the choice made on the logits must be the choice the probabilities give (no rounding ties in softmax)
    g_wo1 = gates.masked_fill(torch.nn.functional.one_hot(i1, E).bool(), float("-inf"))
    assert torch.equal(torch.argmax(g_wo1, dim=1), i2), "softmax rounding tie: pick another seed"
    rec = dict(
        S=S, E=E, M=M, C=int(loc["capacity"]), cf=np.float32(cf), seed=seed, logits=logits.numpy(), gate=gates.numpy(),
        idx1=i1.numpy().astype(np.int32), idx2=i2.numpy().astype(np.int32),
        loc1_all=loc["locations1"][rows, i1].numpy().astype(np.int32),      # before the capacity mask
        loc2_all=loc["locations2"][rows, i2].numpy().astype(np.int32),      # offset by the first choices, before the mask
        kept1=loc["mask1"].sum(dim=1).numpy().astype(np.int32), kept2=loc["mask2"].sum(dim=1).numpy().astype(np.int32),
        loc1_s=loc["locations1_s"].numpy().astype(np.int32), loc2_s=loc["locations2_s"].numpy().astype(np.int32),
        gates1_s=loc["gates1_s"].numpy(), gates2_s=loc["gates2_s"].numpy(), exp_counts=exp_counts.numpy().astype(np.int64),
        d_gates_s=d_gs.numpy(), d_gate=d_gate.numpy(),
    )
    if dense:
        x = torch.randn(S, M, generator=g)
        disp = sm.einsum("sec,sm->ecm", mask.type_as(x), x)                  # MOELayer.forward, sharded_moe.py:476-478
        eo = torch.randn(E, rec["C"], M, generator=g)
        out = sm.einsum("sec,ecm->sm", combine.type_as(x), eo)               # :512-514
        rec.update(x=x.numpy(), disp=disp.numpy(), eo=eo.numpy(), out=out.numpy())
    np.savez_compressed(os.path.join(HERE, f"top2_ref_{name}.npz"), **rec)
    print("top2", name, "C", rec["C"], "dropped", int((rec["kept1"] == 0).sum()), int((rec["kept2"] == 0).sum()))


def run_top2_chain_case(sm, name, S, E, n, seed, spread):
    """The reference's top-2 gate on each of n consecutive token chunks: per chunk its choices, its locations before the
    capacity mask and its gate probabilities.  The reference has no chained top-2 operator; a test combines these
    per-chunk vectors with the CUDA operator's chaining rules (tutel_moe_dispatch.cu:199-201, :207-209)."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(S, E, generator=g) + spread * torch.linspace(-1.0, 1.0, E)
    Sp = S // n
    rows = torch.arange(Sp)
    rec = dict(S=S, E=E, n=n, seed=seed, logits=logits.numpy())
    idx1, idx2, l1, l2, gates = [], [], [], [], []
    for c in range(n):
        _, loc = call_with_locals(sm.top2gating, logits[c * Sp:(c + 1) * Sp], 1.0)
        i1, i2 = loc["indices1_s"], loc["indices2_s"]
        g_wo1 = loc["gates"].masked_fill(torch.nn.functional.one_hot(i1, E).bool(), float("-inf"))
        assert torch.equal(torch.argmax(g_wo1, dim=1), i2), "softmax rounding tie: pick another seed"
        idx1.append(i1.numpy().astype(np.int32))
        idx2.append(i2.numpy().astype(np.int32))
        l1.append(loc["locations1"][rows, i1].numpy().astype(np.int32))
        l2.append(loc["locations2"][rows, i2].numpy().astype(np.int32))
        gates.append(loc["gates"].numpy())
    rec.update(idx1=np.stack(idx1), idx2=np.stack(idx2), loc1_all=np.stack(l1), loc2_all=np.stack(l2), gate=np.concatenate(gates))
    np.savez_compressed(os.path.join(HERE, f"top2chain_ref_{name}.npz"), **rec)
    print("top2chain", name, "chunks", n)


def run_chain_case(ref, name, S, E, M, n, seed, first_used=None):
    """n consecutive chunks of S//n tokens through FakeMoeEncodeOp, used capacity chained.  `first_used` = "random"
    starts the chain from a used capacity drawn in [0, C] per expert (as left by earlier partitions) instead of zero."""
    g = torch.Generator().manual_seed(seed)
    gate = torch.softmax(torch.randn(S, E, generator=g) * 1.5, dim=1)
    x = torch.randn(S, M, generator=g)
    Sp = S // n
    C = (Sp + E - 1) // E
    used = torch.zeros(E, dtype=torch.int32)
    if first_used == "random":
        used = torch.randint(0, C + 1, (E,), generator=g).to(torch.int32)
    il, gs, used_in, ref_used_out = [], [], [], []
    for c in range(n):
        sl = slice(c * Sp, (c + 1) * Sp)
        gates_s, idx_loc, capused, elems, disp = ref.FakeMoeEncodeOp.apply(x[sl], gate[sl], used.clone(), torch.ones(1))
        il.append(idx_loc.numpy().astype(np.int32))
        gs.append(gates_s.numpy())
        used_in.append(used.numpy().copy())
        ref_used_out.append(capused.numpy().astype(np.int32))
        # next call's used capacity by the CUDA operator's rule (gen_location_kernel, tutel_moe_dispatch.cu:207-209)
        cnt = torch.bincount(torch.argmax(gate[sl], dim=1), minlength=E).to(torch.int32)
        used = torch.minimum(used + cnt, torch.tensor(C, dtype=torch.int32))
    np.savez_compressed(os.path.join(HERE, f"chain_ref_{name}.npz"), S=S, E=E, M=M, n=n, C=C, seed=seed, gate=gate.numpy(),
                        idx_loc=np.stack(il), gates_s=np.stack(gs), used_in=np.stack(used_in),
                        fake_used_out=np.stack(ref_used_out))
    print("chain", name, "C", C, "dropped per chunk", [int((a[0] < 0).sum()) for a in il], "used_in", used_in[-1].tolist())


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
    # non-zero used capacity: chained chunks (capacity factor 1.0 is all the reference's CPU operator accepts)
    run_chain_case(ref, "s2048_e8_n4", 2048, 8, 4, 4, 5)
    run_chain_case(ref, "s772_e5_n4", 772, 5, 4, 4, 6)
    run_chain_case(ref, "s2048_e8_n2_used", 2048, 8, 4, 2, 7, first_used="random")
    # top-2: shapes where ceil(2S/E * cf) of the reference equals this project's int(cf * ceil(2S/E))
    sm = load_reference_sharded_moe(ref_root)
    run_top2_case(sm, "s4096_e16", 4096, 16, 8, 1.25, 10, dense=False, spread=0.6)
    run_top2_case(sm, "s4096_e2", 4096, 2, 8, 1.25, 11, dense=False)
    run_top2_case(sm, "s512_e4", 512, 4, 8, 1.25, 12, dense=True)
    run_top2_case(sm, "rag_s193_e5", 193, 5, 4, 1.25, 13, dense=True, spread=0.6)
    run_top2_case(sm, "s256_e8_cf05", 256, 8, 4, 0.5, 14, dense=True)
    run_top2_chain_case(sm, "s4096_e4_n4", 4096, 4, 4, 15, 0.5)
    run_top2_chain_case(sm, "s2048_e16_n4", 2048, 16, 4, 16, 0.6)


if __name__ == "__main__":
    main()
