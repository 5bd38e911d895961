"""The benchmark's own result check (bench.py::verify_moe_step) on CPU: fed with the oracle's outputs it passes, and it
notices a wrong row, a stray value in the padding and a wrong combined output."""
import importlib.util
import os

import numpy as np
import torch

from oracle import moe_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


class Ctx:
    world, rank, dist = 1, 0, None


class Plan:
    pass


def make_plan(S=512, E=4, M=64, k=2):
    g = torch.Generator().manual_seed(0)
    gate = torch.softmax(torch.randn(S, E, generator=g) + torch.linspace(-1, 1, E), dim=1)
    x = torch.randn(S, M, generator=g).half()
    C = O.capacity(S, E, 1.0, k)
    gs, il, cap, el = O.moe_gate(gate.numpy(), np.zeros(E, np.int32), C, M, k)
    disp = O.moe_encode_fwd(il, x.numpy(), E, C)
    out = O.moe_decode_fwd(disp, gs, il)
    p = Plan()
    p.k, p.S, p.M, p.C, p.E = k, S, M, C, E
    p.idx_loc, p.gates_s = torch.from_numpy(il)[None], torch.from_numpy(gs)[None]
    state = {"disp": torch.from_numpy(disp), "out": torch.from_numpy(out)}
    p.dispatch = lambda x_, g_: state["disp"]
    p.combine = lambda: state["out"]
    return p, state, x, gate, il


def test_result_check_accepts_oracle_outputs_and_rejects_corruption(monkeypatch):
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    plan, state, x, gate, il = make_plan()
    assert (il[0] < 0).any() and (il[2] < 0).any()                  # the case has dropped choices
    r = bench.verify_moe_step(Ctx(), plan, x, gate)
    assert r["ok"] and r["combine_bit_exact"] and r["recv_rows_ok"] and r["recv_padding_zero"]
    assert r["recv_rows_checked"] == int((il[0] >= 0).sum() + (il[2] >= 0).sum())
    good = state["disp"].clone()
    bad = good.clone()
    bad[1, 3, 5] += 1                                               # one element of a live row
    state["disp"] = bad
    assert not bench.verify_moe_step(Ctx(), plan, x, gate)["recv_rows_ok"]
    bad = good.clone()
    bad[1, 3], bad[1, 4] = good[1, 4].clone(), good[1, 3].clone()  # two rows swapped
    state["disp"] = bad
    assert not bench.verify_moe_step(Ctx(), plan, x, gate)["ok"]
    bad = good.clone()
    bad[0, plan.C - 1, 0] = 1                                       # a value in the zero padding
    state["disp"] = bad
    r = bench.verify_moe_step(Ctx(), plan, x, gate)
    assert not r["recv_padding_zero"] and not r["ok"]
    state["disp"] = good
    out = state["out"].clone()
    out[7] *= 1.5
    state["out"] = out
    r = bench.verify_moe_step(Ctx(), plan, x, gate)
    assert not r["combine_bit_exact"] and not r["ok"]


def test_row_checksums_see_permutations_inside_a_row():
    a = torch.arange(32, dtype=torch.float16).view(2, 16)
    b = a.clone()
    b[0, 3], b[0, 4] = a[0, 4], a[0, 3]
    ca, _ = bench.row_checksums(a)
    cb, _ = bench.row_checksums(b)
    assert ca[0] != cb[0] and ca[1] == cb[1]
