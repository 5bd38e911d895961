"""The operators run through the registry (dispatch + requests + Execute) reproduce the golden vectors
of the reference's own operators."""
import glob
import os

import numpy as np
import pytest
import torch

from lancet_b200 import raf
from oracle import lans_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = sorted(p for p in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "moe_ref_*.npz"))
                if "x" in np.load(p).files)


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[8:-4] for p in GOLDEN])
def test_moe_ops_through_registry(path):
    rec = np.load(path)
    S, E, M, C = (int(rec[k]) for k in ("S", "E", "M", "C"))
    outs, name = raf.call("raf.op.moe_encode", cu(rec["x"]), cu(rec["gate"]), torch.zeros(E, dtype=torch.int32, device=DEV), 1.0)
    assert name == "raf.op.cuda.moe_encode"
    gs, il, cap, el, disp = outs
    np.testing.assert_array_equal(il.cpu().numpy(), rec["idx_loc"])
    np.testing.assert_array_equal(cap.cpu().numpy(), rec["capused"])
    np.testing.assert_array_equal(gs.cpu().numpy(), rec["gates_s"])
    np.testing.assert_array_equal(disp.cpu().numpy(), rec["disp"])
    (out,), name = raf.call("raf.op.moe_decode", cu(rec["eo"]), gs, il)
    assert name == "raf.op.cuda.moe_decode"
    np.testing.assert_array_equal(out.cpu().numpy(), rec["out"])
    (dx,), _ = raf.call("raf.op.moe_encode_dx", cu(rec["d_disp"]), il)
    np.testing.assert_array_equal(dx.cpu().numpy(), rec["enc_dx"])
    (dg,), _ = raf.call("raf.op.moe_encode_dg", cu(rec["d_gates"]), il, E)
    ref_dg = np.zeros((S, E), np.float32)
    ref_dg[tuple(rec["enc_dg_nnz"])] = rec["enc_dg_val"]
    np.testing.assert_array_equal(dg.cpu().numpy(), ref_dg)
    (ddx,), _ = raf.call("raf.op.moe_decode_dx", cu(rec["d_out"]), gs, il, E, C)
    np.testing.assert_array_equal(ddx.cpu().numpy(), rec["dec_dx"])
    (ddg,), _ = raf.call("raf.op.moe_decode_dg", cu(rec["d_out"]), cu(rec["eo"]), il)
    np.testing.assert_allclose(ddg.cpu().numpy(), rec["dec_dg"], rtol=1e-5, atol=1e-5)


def test_lans_through_registry_with_device_step():
    shapes = [(33, 65), (9000,), (5,)]
    rng = np.random.default_rng(0)
    p = [rng.normal(0, 0.02, s).astype(np.float32) for s in shapes]
    g = [rng.normal(0, 1e-3, s).astype(np.float32) for s in shapes]
    m = [rng.normal(0, 1e-4, s).astype(np.float32) for s in shapes]
    v = [rng.uniform(0, 1e-6, s).astype(np.float32) for s in shapes]
    wp, wm, wv = lans_oracle.lans_step(g, p, m, v, step=7, lr=1e-3)
    tl = [cu(a) for a in g + p + m + v]
    step = torch.tensor(7.0, device=DEV)            # the reference passes step as a 0-d device tensor
    outs, name = raf.call("raf.op.lans", tl, step, 1e-3, 0.9, 0.999, 1e-6, 1, 0.01, 1, 1, True)
    assert name == "raf.op.cuda.lans"
    for i in range(3):
        np.testing.assert_allclose(tl[3 + i].cpu().numpy(), wp[i], rtol=1e-5, atol=1e-8)
        np.testing.assert_allclose(tl[6 + i].cpu().numpy(), wm[i], rtol=1e-5, atol=1e-10)


def test_matmul_nt_dispatch_and_decline():
    a = torch.randn(300, 128, device=DEV).bfloat16()
    b = (torch.randn(512, 128, device=DEV) * 0.1).bfloat16()
    (y,), name = raf.call("raf.op.matmul_nt", a, b)
    assert name == "raf.op.cublas.matmul_nt"
    want = a.float() @ b.float().t()
    assert torch.allclose(y.float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()))
    with pytest.raises(raf.RafError, match="declined"):       # fp32 operands: the tensor-core op declines
        raf.call("raf.op.matmul_nt", a.float(), b.float())


def test_expert_gemm_family_through_registry():
    """matmul / matmul_tn / dense (the forward, data-gradient and weight-gradient contractions of an expert layer,
    src/op/grad/gemm.cc:31-36) and sparse_expert_matmul_nt dispatch to the tensor-core ops under the reference's names."""
    g = torch.Generator(device=DEV).manual_seed(4)
    a = torch.randn((384, 128), device=DEV, generator=g).bfloat16()
    w = (torch.randn((128, 512), device=DEV, generator=g) * 0.1).bfloat16()
    tol = lambda y, want: torch.allclose(y.float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()))
    (y,), name = raf.call("raf.op.matmul", a, w)
    assert name == "raf.op.cublas.matmul" and tol(y, a.float() @ w.float())
    (y,), name = raf.call("raf.op.dense", a, w.t().contiguous())
    assert name == "raf.op.cublas.dense" and tol(y, a.float() @ w.float())
    dy = torch.randn((384, 512), device=DEV, generator=g).bfloat16()
    (dw,), name = raf.call("raf.op.matmul_tn", a, dy)
    assert name == "raf.op.cublas.matmul_tn" and dw.shape == (128, 512) and tol(dw, a.float().t() @ dy.float())
    with pytest.raises(raf.RafError, match="declined"):
        raf.call("raf.op.matmul", a.float(), w.float())
    # count-aware expert matmul in the [C, G, M] layout of the partitioned graphs
    C, G, M, N = 256, 3, 128, 256
    x = torch.randn((C, G, M), device=DEV, generator=g).half()
    wt = (torch.randn((N, M), device=DEV, generator=g) * 0.1).half()
    rows = [200, 0, 77]
    nelem = torch.tensor([r * M for r in rows], dtype=torch.int64, device=DEV).view(torch.uint64)
    (out,), name = raf.call("raf.op.sparse_expert_matmul_nt", x, wt, nelem, 0, 1, 1)
    assert name == "raf.op.cublas.sparse_expert_matmul_nt"
    want = torch.zeros((C, G, N), device=DEV)
    for gi, r in enumerate(rows):
        want[:r, gi] = x[:r, gi].float() @ wt.float().t()
    assert tol(out, want)
    for gi, r in enumerate(rows):
        assert (out[r:, gi] == 0).all()


def test_partitioned_graph_ops_through_registry():
    """n chained moe_encode + moe_merge_masks + moe_redispatch, as the reference's scheduler emits them
    (tests/python/op/cuda/test_cuda_moe.py:387-471), all through dispatch."""
    from oracle import moe_oracle as O
    rng = np.random.default_rng(3)
    S, M, E, n = 1024, 16, 2, 4
    x = rng.standard_normal((S, M)).astype(np.float32)
    gate = rng.random((S, E), dtype=np.float32)
    cap = torch.zeros(E, dtype=torch.int32, device=DEV)
    ils, ds = [], []
    for i in range(n):
        sl = slice(i * S // n, (i + 1) * S // n)
        (gs, il, cap, el, d), _ = raf.call("raf.op.moe_encode", cu(x[sl]), cu(gate[sl]), cap, float(n))
        ils.append(il); ds.append(d)
    (mil,), name = raf.call("raf.op.moe_merge_masks", ils, E)
    assert name == "raf.op.cuda.moe_merge_masks"
    (md,), name = raf.call("raf.op.moe_redispatch", ds, ils)
    assert name == "raf.op.cuda.moe_redispatch"
    np.testing.assert_array_equal(mil.cpu().numpy(), O.moe_merge_masks([t.cpu().numpy() for t in ils], E))
    np.testing.assert_array_equal(md.cpu().numpy(), O.moe_redispatch([t.cpu().numpy() for t in ds], [t.cpu().numpy() for t in ils]))
    want = O.moe_encode_bpr(x, gate, 2, 1, 2.0)
    got, name = raf.call("raf.op.moe_encode_batch_prioritized", cu(x), cu(gate), 2, 1, 2.0)
    assert name == "raf.op.cuda.moe_encode_batch_prioritized"
    for a, b in zip(got, want):
        np.testing.assert_array_equal(a.cpu().numpy() if a.dtype != torch.uint64 else a.cpu().view(torch.int64).numpy().astype(np.uint64), b)


def test_cpp_host_through_registry(tmp_path):
    """A C++ program (no Python, no torch) drives moe_encode / moe_decode through the registry."""
    import shutil
    import subprocess
    import lancet_b200 as LB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc on this box")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    shim = os.path.join(LB.build.CSRC, "raf_shim")
    exe = str(tmp_path / "raf_host_example")
    libdir = os.path.dirname(LB.build.LIB_PATH)
    subprocess.run([nvcc, "-std=c++17", "-O1", "-I", shim, os.path.join(root, "tests", "cpp", "raf_host_example.cc"),
                    "-L", libdir, "-llancet_b200", "-Xlinker", "-rpath", "-Xlinker", libdir, "-o", exe], check=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "raf host example ok" in r.stdout, r.stdout + r.stderr
