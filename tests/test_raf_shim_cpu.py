"""The RAF-style registry without a GPU: dialect priorities, declarations (output shapes and dtypes
of src/op/declare/moe.cc of the reference) and error messages."""
import os
import subprocess

import pytest
import torch

import lancet_b200 as LB
from lancet_b200 import raf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", autouse=True)
def built():
    LB.build.build()


@pytest.mark.parametrize("flags", [[], ["-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer"]],
                         ids=["plain", "asan_ubsan"])
def test_registry_cpp(tmp_path, flags):
    """The registry's host code, also under the address and undefined-behaviour sanitizers (the reference offers them for
    its host code through RAF_USE_SANITIZER, cmake/modules/Sanitizer.cmake:77-93)."""
    shim = os.path.join(LB.build.CSRC, "raf_shim")
    exe = str(tmp_path / "test_raf_shim")
    cmd = ["g++", "-std=c++17", "-O1"] + flags + ["-I", shim, os.path.join(ROOT, "tests", "cpp", "test_raf_shim.cc"),
                                                   os.path.join(shim, "registry.cc"), "-o", exe]
    built = subprocess.run(cmd, capture_output=True, text=True)
    if built.returncode != 0 and flags:
        pytest.skip("sanitizer runtime not available: " + built.stderr[-200:])
    assert built.returncode == 0, built.stderr
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0 and "raf shim ok" in r.stdout, r.stdout + r.stderr


def test_dialect_names_and_priorities():
    assert raf.dialect_ops("raf.op.moe_encode") == [("raf.op.cuda.moe_encode", "20")]
    assert raf.dialect_ops("raf.op._all_to_all") == [("raf.op.nccl._all_to_all", "10")]
    assert raf.dialect_ops("raf.op.lans") == [("raf.op.cuda.lans", "20")]
    assert raf.dialect_ops("raf.op.matmul_nt") == [("raf.op.cublas.matmul_nt", "15")]
    assert raf.dialect_ops("raf.op._all_to_allv") == [("raf.op.nccl._all_to_allv", "10")]
    assert raf.dialect_ops("raf.op.sparse_expert_matmul_nt") == [("raf.op.cublas.sparse_expert_matmul_nt", "20")]
    for op in ("matmul", "matmul_tn", "dense"):
        assert raf.dialect_ops("raf.op." + op) == [("raf.op.cublas." + op, "15")]
    for op in ("moe_decode", "moe_encode_dx", "moe_encode_dg", "moe_decode_dx", "moe_decode_dg",
               "moe_encode_batch_prioritized", "moe_merge_masks", "moe_redispatch", "moe_redispatch_expert_input"):
        assert raf.dialect_ops("raf.op." + op) == [("raf.op.cuda." + op, "20")]


def test_declarations():
    x = torch.zeros(2048, 512)
    gate = torch.zeros(2048, 8)
    used = torch.zeros(8, dtype=torch.int32)
    outs = raf.declare("raf.op.moe_encode", x, gate, used, 1.0)
    assert outs == [((2048,), torch.float32), ((2, 2048), torch.int32), ((8,), torch.int32), ((8,), torch.uint64),
                    ((8, 256, 512), torch.float32)]
    outs = raf.declare("raf.op.moe_encode", x.half(), gate.half(), used, 2.0)
    assert outs[4] == ((8, 512, 512), torch.float16)
    il = torch.zeros(2, 2048, dtype=torch.int32)
    assert raf.declare("raf.op.moe_decode", torch.zeros(8, 256, 512), torch.zeros(2048), il) == [((2048, 512), torch.float32)]
    assert raf.declare("raf.op.moe_encode_dg", torch.zeros(2048), il, 8) == [((2048, 8), torch.float32)]
    assert raf.declare("raf.op.moe_decode_dx", x, torch.zeros(2048), il, 8, 256) == [((8, 256, 512), torch.float32)]
    assert raf.declare("raf.op._all_to_all", [torch.zeros(4, 6)]) == [((4, 6), torch.float32)]
    outs = raf.declare("raf.op.moe_encode_batch_prioritized", x, gate, 4, 1, 4.0)
    assert outs[1] == ((2, 512), torch.int32) and outs[4] == ((8, 256, 512), torch.float32)
    assert raf.declare("raf.op.moe_merge_masks", [il, il, il], 8) == [((2, 3 * 2048), torch.int32)]
    assert raf.declare("raf.op.moe_redispatch", [torch.zeros(8, 16, 4).half()] * 2, [il, il]) == [((8, 16, 4), torch.float16)]
    h = torch.zeros(1, dtype=torch.float16)
    assert raf.declare("raf.op.matmul", h.expand(6, 4).contiguous(), h.expand(4, 8).contiguous()) == [((6, 8), torch.float16)]
    assert raf.declare("raf.op.matmul_tn", h.expand(4, 6).contiguous(), h.expand(4, 8).contiguous()) == [((6, 8), torch.float16)]
    assert raf.declare("raf.op.dense", h.expand(6, 4).contiguous(), h.expand(8, 4).contiguous()) == [((6, 8), torch.float16)]
    ne = torch.zeros(10, dtype=torch.uint64)
    assert raf.declare("raf.op.sparse_expert_matmul_nt", torch.zeros(256, 5, 64).half(), torch.zeros(128, 64).half(), ne, 1, 2,
                       1) == [((256, 5, 128), torch.float16)]
    with pytest.raises(raf.RafError, match="after stride"):
        raf.declare("raf.op.sparse_expert_matmul_nt", torch.zeros(256, 4, 64).half(), torch.zeros(128, 64).half(), ne, 1, 2, 1)
    assert raf.declare("raf.op._all_to_allv", [torch.zeros(4, 2, 6)], [torch.zeros(8, dtype=torch.uint64)]) == [
        ((4, 2, 6), torch.float32), ((8,), torch.uint64)]
    with pytest.raises(raf.RafError, match="matching shape in dim 0"):
        raf.declare("raf.op.moe_encode", x, torch.zeros(100, 8), used, 1.0)
    with pytest.raises(raf.RafError, match="no declaration"):
        raf.declare("raf.op.not_an_op", x)
