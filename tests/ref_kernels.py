"""ctypes loader for oracle/_ref/libraf_ref_kernels.so: the reference project's own CUDA kernels (gating locations,
encode/decode and gradients, batch-prioritized locations, merge_masks, redispatch, LANS), built unmodified from the
reference tree by oracle/ref_build/build_ref.py.  Test infrastructure: the checker the product's kernels are compared
with on the same GPU.  Every call synchronises its stream and returns the CUDA error code."""
import ctypes
import os

import numpy as np
import torch

PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libraf_ref_kernels.so")
_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_SIG = {
    "raf_ref_gen_location": [_P] * 5 + [_I] * 4 + [_P],
    "raf_ref_encode_forward": [_I] + [_P] * 5 + [_I] * 4 + [_P],
    "raf_ref_encode_backward_data": [_I] + [_P] * 4 + [_I] * 4 + [_P],
    "raf_ref_encode_backward_gate": [_I] + [_P] * 3 + [_I] * 2 + [_P],
    "raf_ref_decode_forward": [_I] + [_P] * 5 + [_I] * 4 + [_P],
    "raf_ref_decode_backward_data": [_I] + [_P] * 5 + [_I] * 4 + [_P],
    "raf_ref_decode_backward_gate": [_I] + [_P] * 5 + [_I] * 3 + [_P],
    "raf_ref_gen_location_bpr": [_P] * 6 + [_I] * 6 + [_P],
    "raf_ref_merge_masks": [_P] * 5 + [_I] * 3 + [_P],
    "raf_ref_redispatch": [_I] + [_P] * 4 + [_I] * 5 + [_P],
    "raf_ref_redispatch_expert_input": [_I] + [_P] * 4 + [_I] * 7 + [_P],
    "raf_ref_lans": [_P] * 4 + [_P, _I, _P, _P] + [_F] * 4 + [_I, _F, _I, _I, _I, _F, _P],
}
_lib = None


def available():
    return os.path.exists(PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(PATH)
        for name, sig in _SIG.items():
            fn = getattr(_lib, name)
            fn.argtypes, fn.restype = sig, _I
    return _lib


def ptr(t):
    return None if t is None else t.data_ptr()


def table(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


def ok(rc):
    assert rc == 0, "reference kernel call failed with CUDA error %d" % rc


def stream():
    return torch.cuda.current_stream().cuda_stream


def is_half(t):
    assert t.dtype in (torch.float32, torch.float16)
    return int(t.dtype == torch.float16)


def encode(x, gate, used, capacity):
    """The reference's moe_encode (src/op/dialect/cuda/moe.cc:351-395) with its TVM parts on the host side of this call:
    indices = argmax(gate), gates_s = the gate value at that index.  Returns gates_s, indices, locations, used_capacity
    after the call, elements per expert and the dispatched buffer."""
    S, M = x.shape
    E = gate.shape[1]
    idx = torch.argmax(gate, dim=1).to(torch.int32)
    gates_s = gate.gather(1, idx.long()[:, None])[:, 0].contiguous()
    loc = torch.zeros(S, dtype=torch.int32, device=x.device)
    cap_out = torch.zeros(E, dtype=torch.int32, device=x.device)
    elems = torch.zeros(E, dtype=torch.int64, device=x.device)
    disp = torch.empty((E, capacity, M), dtype=x.dtype, device=x.device)
    L = lib()
    ok(L.raf_ref_gen_location(ptr(idx), ptr(used), ptr(loc), ptr(cap_out), ptr(elems), capacity, S, E, M, stream()))
    ok(L.raf_ref_encode_forward(is_half(x), ptr(idx), ptr(loc), ptr(used), ptr(x), ptr(disp), S, M, capacity, E, stream()))
    return gates_s, idx, loc, cap_out, elems, disp


def lans(g, p, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, bias_correction=1, weight_decay=0.01,
         grad_averaging=1, mode=1, normalize_grad=True):
    """One in-place step of the reference's multi_tensor_lans_cuda<float> over lists of fp32 CUDA tensors (the gradient
    tensors are overwritten with the update, as in the reference)."""
    n = len(g)
    numels = np.array([t.numel() for t in g], dtype=np.int32)
    assert numels.min() > 0, "the reference's launcher never flushes its last launch after an empty tensor"
    dev = g[0].device
    q = torch.zeros(int(numels.sum()), dtype=torch.float32, device=dev)
    max_chunks = int(((numels + 65535) // 65536).max())
    scratch = torch.zeros(n * max_chunks + 4 * n, dtype=torch.float32, device=dev)
    ok(lib().raf_ref_lans(table(g), table(p), table(m), table(v), numels.ctypes.data, n, ptr(q), ptr(scratch), lr, beta1, beta2,
                          eps, bias_correction, weight_decay, grad_averaging, mode, int(normalize_grad), float(step), stream()))
