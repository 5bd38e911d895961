"""Boundary tests that need no GPU: the C-ABI library builds, loads, exports every symbol the
header declares, and rejects invalid calls before touching the device."""
import ctypes

import pytest

import lancet_b200
from lancet_b200 import _capi


@pytest.fixture(scope="module")
def L():
    lancet_b200.build.build()
    return _capi.lib()


def test_exports_every_declared_symbol(L):
    names = _capi.header_symbols()
    assert len(names) >= 16
    for n in names:
        assert hasattr(L, n), "library does not export %s" % n
    assert sorted(_capi.SIGNATURES) == names


def test_capacity_formula(L):
    # (int)(cf * ceil_div(k*S, E)): reference src/op/declare/moe.cc:46
    assert L.lancet_moe_capacity(2048, 8, 1.0, 1) == 256
    assert L.lancet_moe_capacity(16384, 2, 1.25, 2) == 20480
    assert L.lancet_moe_capacity(16384, 16, 1.25, 2) == 2560
    assert L.lancet_moe_capacity(193, 5, 1.0, 1) == 39
    assert L.lancet_moe_capacity(1024, 32, 2.0, 1) == 64
    from oracle import moe_oracle as O
    for S, E, cf, k in [(1000, 7, 1.3, 1), (77, 3, 0.5, 2), (4096, 64, 4.0, 1)]:
        assert L.lancet_moe_capacity(S, E, cf, k) == O.capacity(S, E, cf, k)


def test_invalid_arguments_launch_nothing(L):
    one = ctypes.c_void_p(16)
    assert L.lancet_moe_gate(one, 0, 8, 4, 3, None, 2, 4, one, 0, one, one, one, one, 1 << 20, 0, None) == 1
    assert b"k must be 1 or 2" in L.lancet_last_error()
    assert L.lancet_moe_gate(None, 0, 8, 4, 1, None, 2, 4, one, 0, one, one, one, one, 1 << 20, 0, None) == 2
    assert L.lancet_moe_gate(one, 0, 8, 4, 1, None, 2, 4, one, 0, one, one, one, one, 8, 0, None) == 1
    assert b"workspace" in L.lancet_last_error()
    assert L.lancet_moe_gate(one, 7, 8, 4, 1, None, 2, 4, one, 0, one, one, one, one, 1 << 20, 0, None) == 1
    assert L.lancet_moe_encode_fwd(one, 1, None, None, None, one, one, 8, 4, 2, 4, 0, 64, None) == 1
    assert L.lancet_moe_encode_fwd(one, 1, None, None, None, one, one, 8, 4, 2, 4, 0, 1, None) == 2  # GLOBAL_LOC w/o capused
    assert L.lancet_moe_decode_fwd(None, 0, one, 1, one, one, 8, 4, 2, 4, 0, None) == 2
    assert L.lancet_moe_decode_fwd(one, 0, one, 1, one, one, -1, 4, 2, 4, 0, None) == 1
    numels = (ctypes.c_int64 * 1)(10)
    ptrs = (ctypes.c_void_p * 1)(16)
    assert L.lancet_lans(one, 1 << 20, 1, numels, ptrs, ptrs, ptrs, ptrs, 1, 1, 1e-3, .9, .999, 1e-6, 1, .01, 1, 1, 1,
                         0, None) == 6  # fp16 unsupported, as the reference (lans.cc:150-153)
    assert L.lancet_lans(one, 1 << 20, 1, numels, ptrs, ptrs, ptrs, ptrs, 0, 0, 1e-3, .9, .999, 1e-6, 1, .01, 1, 1, 1,
                         0, None) == 1  # step 0
    assert L.lancet_lans(one, 8, 1, numels, ptrs, ptrs, ptrs, ptrs, 0, 1, 1e-3, .9, .999, 1e-6, 1, .01, 1, 1, 1,
                         0, None) == 1  # workspace too small


def test_invalid_arguments_of_the_layer_norm_loss_and_split_combine_entries(L):
    one = ctypes.c_void_p(16)
    # layer norm: the width must be a multiple of 128 the kernels are built for; null operands
    assert L.lancet_layer_norm_fwd(one, one, one, one, 0, one, one, 4, 100, 1e-5, None) == 1
    assert L.lancet_layer_norm_fwd(one, one, one, one, 0, one, one, 4, 384, 1e-5, None) == 6     # 128 x 3: not instantiated
    assert L.lancet_layer_norm_fwd(None, one, one, one, 0, one, one, 4, 256, 1e-5, None) == 2
    assert L.lancet_layer_norm_fwd(one, one, one, one, 0, one, one, 0, 256, 1e-5, None) == 0    # no rows: nothing to do
    assert L.lancet_layer_norm_bwd(one, one, 0, one, one, one, one, one, one, 4, 256, one, 8, None) == 1   # workspace too small
    assert L.lancet_layer_norm_workspace_bytes(8192, 1024) > 0 and L.lancet_layer_norm_workspace_bytes(8192, 100) == 0
    # loss: the vocabulary cannot be wider than a row; null operands
    assert L.lancet_softmax_xent_fwd(one, 16, one, 4, 17, 2, one, one, None) == 1
    assert L.lancet_softmax_xent_fwd(None, 16, one, 4, 10, 2, one, one, None) == 2
    assert L.lancet_softmax_xent_bwd(one, 16, one, 4, 10, 8, 2, one, None, 1.0, one, 16, None) == 1   # fewer columns than classes
    assert L.lancet_softmax_xent_fwd(one, 16, one, 0, 10, 2, one, one, None) == 0
    # the two halves of the backward combine: part is 0, 1 or 2
    ptrs = (ctypes.c_void_p * 2)(16, 16)
    assert L.lancet_moe_combine_bwd_part_p2p(one, one, one, ptrs, ptrs, one, 8, 8, 4, 1, 2, 0, 2, 1, 0, 3, None) == 1
    assert b"part" in L.lancet_last_error()
    assert L.lancet_set_chained_launch(1) == 0


def test_workspace_queries(L):
    assert L.lancet_moe_gate_workspace_bytes(16384, 16, 2) >= 2 * 16384 * 4 + 64 * 32 * 4
    assert L.lancet_moe_gate_workspace_bytes(0, 8, 1) > 0
    assert L.lancet_moe_gate_workspace_bytes(10, 8, 3) == 0
    numels = (ctypes.c_int64 * 3)(10, 100000, 0)
    assert L.lancet_lans_workspace_bytes(3, numels) > 0


def test_ops_refuse_cpu_tensors():
    import torch
    with pytest.raises(ValueError):
        lancet_b200.moe_decode(torch.zeros(2, 2, 4), torch.zeros(4), torch.zeros(2, 4, dtype=torch.int32))
