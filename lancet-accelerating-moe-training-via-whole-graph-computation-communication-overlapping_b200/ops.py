"""Host-side mirror of the reference's operator surface for the MoE hot path.

Function names, argument order and meaning follow the RAF op schemas
(scripts/src_codegen/def_schema.py:642-716 and :726-742 of the reference):
`moe_encode(data, gate, used_capacity, capacity_factor)`, `moe_decode(data, gate,
indices_locations)`, `moe_encode_dx(dy, indices_locations)`, `moe_encode_dg(dy,
indices_locations, n_experts)`, `moe_decode_dx(dy, gate, indices_locations, n_experts,
capacity)`, `moe_decode_dg(dy, data, indices_locations)`, `lans(tensor_list, step, ...)`.
torch supplies device memory and the current stream only; all arithmetic runs in the CUDA
library behind the C ABI.  Extra keyword arguments (k, gates dtype) extend the surface to the
top-2 gate; their defaults reproduce the reference ops.
"""
import ctypes

import torch

from . import _capi
from ._capi import check

_DT = {torch.float32: _capi.F32, torch.float16: _capi.F16, torch.bfloat16: _capi.BF16}
_workspaces = {}


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError("lancet_b200: unsupported dtype %s (float32, float16, bfloat16)" % t.dtype)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("lancet_b200 ops need CUDA tensors (there is no CPU path)")
        if t is not None and not t.is_contiguous():
            raise ValueError("lancet_b200 ops need contiguous tensors")


def workspace(device, nbytes, tag="default"):
    """A cached, 256-byte aligned scratch tensor per (device, tag), grown on demand."""
    key = (device, tag)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def moe_capacity(S, E, capacity_factor=1.0, k=1):
    return _capi.lib().lancet_moe_capacity(S, E, capacity_factor, k)


def moe_gate(gate, used_capacity, capacity, M, k=1, gates_dtype=torch.float32, flags=0):
    """Gating only: returns (gates_s [k,S], indices_locations [2k,S], capused [E], elements [E] uint64)."""
    _require_cuda(gate, used_capacity)
    S, E = gate.shape
    dev = gate.device
    gates_s = torch.empty((k, S), dtype=gates_dtype, device=dev)
    idx_loc = torch.empty((2 * k, S), dtype=torch.int32, device=dev)
    capused = torch.empty((E,), dtype=torch.int32, device=dev)
    elems = torch.empty((E,), dtype=torch.uint64, device=dev)
    L = _capi.lib()
    nws = L.lancet_moe_gate_workspace_bytes(S, E, k)
    ws = workspace(dev, nws, "gate")
    check(L.lancet_moe_gate(_ptr(gate), _dt(gate), S, E, k, _ptr(used_capacity), capacity, M, _ptr(gates_s),
                            _DT[gates_dtype], _ptr(idx_loc), _ptr(capused), _ptr(elems), _ptr(ws), ws.numel(), flags,
                            _stream(gate)))
    return gates_s, idx_loc, capused, elems


def moe_encode(data, gate, used_capacity, capacity_factor=1.0, k=1, gates_dtype=None, out=None, flags=0):
    """`raf.op.moe_encode`: returns (gates_s, indices_locations, used_capacity, elements_per_expert,
    dispatched [E,C,M]).  For k=1 gates_s has shape [S] and indices_locations [2,S] as in the reference."""
    _require_cuda(data, gate, used_capacity)
    S, M = data.shape
    E = gate.shape[1]
    if gate.shape[0] != S:
        raise ValueError("Input data and gate should have matching shape in dim 0.")
    dev = data.device
    gates_dtype = gates_dtype or torch.float32
    L = _capi.lib()
    C = L.lancet_moe_capacity(S, E, capacity_factor, k)
    gates_s = torch.empty((k, S), dtype=gates_dtype, device=dev)
    idx_loc = torch.empty((2 * k, S), dtype=torch.int32, device=dev)
    capused = torch.empty((E,), dtype=torch.int32, device=dev)
    elems = torch.empty((E,), dtype=torch.uint64, device=dev)
    disp = out if out is not None else torch.empty((E, C, M), dtype=data.dtype, device=dev)
    nws = L.lancet_moe_gate_workspace_bytes(S, E, k)
    ws = workspace(dev, nws, "gate")
    check(L.lancet_moe_encode(_ptr(data), _ptr(gate), _dt(gate), _ptr(used_capacity), capacity_factor, S, M, E, k,
                              _dt(data), _ptr(gates_s), _DT[gates_dtype], _ptr(idx_loc), _ptr(capused), _ptr(elems),
                              _ptr(disp), _ptr(ws), ws.numel(), flags, _stream(data)))
    if k == 1:
        gates_s = gates_s[0]
    return gates_s, idx_loc, capused, elems, disp


def moe_encode_fwd(indices_locations, data, n_experts, capacity, used_capacity=None, rows_hi=None, rows_lo=None,
                   out=None, flags=0):
    """Dispatch only (launch_encode_forward of the reference)."""
    _require_cuda(indices_locations, data)
    S, M = data.shape
    k = indices_locations.shape[0] // 2
    disp = out if out is not None else torch.empty((n_experts, capacity, M), dtype=data.dtype, device=data.device)
    check(_capi.lib().lancet_moe_encode_fwd(_ptr(indices_locations), k, _ptr(used_capacity), _ptr(rows_hi),
                                            _ptr(rows_lo), _ptr(data), _ptr(disp), S, M, capacity, n_experts,
                                            _dt(data), flags, _stream(data)))
    return disp


def moe_zero_tail(dispatched, used):
    E, C, M = dispatched.shape
    check(_capi.lib().lancet_moe_zero_tail(_ptr(dispatched), _ptr(used), M, C, E, _dt(dispatched), _stream(dispatched)))
    return dispatched


def _k_of(indices_locations):
    return indices_locations.shape[0] // 2


def moe_decode(data, gate, indices_locations, out=None):
    """`raf.op.moe_decode`: data [E,C,M] expert output, gate = gates_s, returns [S,M]."""
    _require_cuda(data, gate, indices_locations)
    E, C, M = data.shape
    S = indices_locations.shape[1]
    k = _k_of(indices_locations)
    res = out if out is not None else torch.empty((S, M), dtype=data.dtype, device=data.device)
    check(_capi.lib().lancet_moe_decode_fwd(_ptr(gate), _dt(gate), _ptr(indices_locations), k, _ptr(data), _ptr(res),
                                            S, M, C, E, _dt(data), _stream(data)))
    return res


def moe_encode_dx(dy, indices_locations):
    """`raf.op.moe_encode_dx`: dy [E,C,M] -> dx [S,M]."""
    _require_cuda(dy, indices_locations)
    E, C, M = dy.shape
    S = indices_locations.shape[1]
    dx = torch.empty((S, M), dtype=dy.dtype, device=dy.device)
    check(_capi.lib().lancet_moe_encode_bwd_data(_ptr(indices_locations), _k_of(indices_locations), _ptr(dy), _ptr(dx),
                                                 S, M, C, E, _dt(dy), _stream(dy)))
    return dx


def moe_encode_dg(dy, indices_locations, n_experts, gate=None):
    """`raf.op.moe_encode_dg`: dy = gradient of gates_s -> dgate [S,E] in dy's dtype (k=1).
    For k=2 the gate matrix is needed (Jacobian of the normalisation); dgate has gate's dtype."""
    _require_cuda(dy, indices_locations, gate)
    S = indices_locations.shape[1]
    k = _k_of(indices_locations)
    if k == 2 and gate is None:
        raise ValueError("moe_encode_dg with k=2 needs the gate matrix")
    out_dtype = gate.dtype if gate is not None else dy.dtype
    dgate = torch.empty((S, n_experts), dtype=out_dtype, device=dy.device)
    check(_capi.lib().lancet_moe_encode_bwd_gate(_ptr(dy), _dt(dy), _ptr(indices_locations), k, _ptr(gate),
                                                 _DT[out_dtype], _ptr(dgate), S, n_experts, _stream(dy)))
    return dgate


def moe_decode_dx(dy, gate, indices_locations, n_experts, capacity, rows_used=None):
    """`raf.op.moe_decode_dx`: dy [S,M], gate = gates_s -> d_expert [E,C,M]."""
    _require_cuda(dy, gate, indices_locations, rows_used)
    S, M = dy.shape
    out = torch.empty((n_experts, capacity, M), dtype=dy.dtype, device=dy.device)
    check(_capi.lib().lancet_moe_decode_bwd_data(_ptr(gate), _dt(gate), _ptr(indices_locations), _k_of(indices_locations),
                                                 _ptr(dy), _ptr(out), _ptr(rows_used), S, M, capacity, n_experts,
                                                 _dt(dy), _stream(dy)))
    return out


def moe_decode_dg(dy, data, indices_locations, gates_dtype=None):
    """`raf.op.moe_decode_dg`: dy [S,M], data [E,C,M] -> dgates_s [S] (k=1) or [k,S]."""
    _require_cuda(dy, data, indices_locations)
    E, C, M = data.shape
    S = dy.shape[0]
    k = _k_of(indices_locations)
    gates_dtype = gates_dtype or torch.float32
    out = torch.empty((k, S), dtype=gates_dtype, device=dy.device)
    check(_capi.lib().lancet_moe_decode_bwd_gate(_ptr(indices_locations), k, _ptr(dy), _ptr(data), _ptr(out),
                                                 _DT[gates_dtype], S, M, C, E, _dt(dy), _stream(dy)))
    return out[0] if k == 1 else out


class LansState:
    """Host tables of one LANS parameter group (built once, reused every step)."""

    def __init__(self, grads, params, exp_avg, exp_avg_sq):
        n = len(params)
        if not (len(grads) == len(exp_avg) == len(exp_avg_sq) == n):
            raise ValueError("lans: the four tensor lists must have the same length")
        _require_cuda(*grads, *params, *exp_avg, *exp_avg_sq)
        for t in list(grads) + list(params) + list(exp_avg) + list(exp_avg_sq):
            if t.dtype != torch.float32:
                raise TypeError("lans: only float32 tensors are supported")
        self.n = n
        self.device = params[0].device if n else torch.device("cuda")
        self.numels = (ctypes.c_int64 * max(n, 1))(*[p.numel() for p in params])
        mk = lambda ts: (ctypes.c_void_p * max(n, 1))(*[t.data_ptr() for t in ts])
        self.g, self.p, self.m, self.v = mk(grads), mk(params), mk(exp_avg), mk(exp_avg_sq)
        self.key = tuple(t.data_ptr() for t in list(grads) + list(params) + list(exp_avg) + list(exp_avg_sq))
        L = _capi.lib()
        self.ws_bytes = L.lancet_lans_workspace_bytes(n, self.numels) if n else 0
        self.ws = torch.empty(max(self.ws_bytes, 256), dtype=torch.uint8, device=self.device)
        self.ready = False


_lans_states = {}


def lans(tensor_list, step, learning_rate=1e-3, beta1=0.9, beta2=0.999, eps=1e-6, bias_correction=1,
         weight_decay=0.01, grad_averaging=1, mode=1, normalize_grad=True, state=None):
    """`raf.op.lans`: tensor_list = g_list + x_list + m_list + v_list (python/raf/optim/lans.py:265 of the
    reference); parameters, m and v are updated in place and the list is returned.  `step` is a host
    integer or float (1-based), or - as the reference's op receives it - a float32 scalar tensor on the
    device, which is then read by the kernels themselves: the call stays asynchronous."""
    n4 = len(tensor_list)
    if n4 % 4 != 0:
        raise ValueError("lans: tensor_list must hold 4 lists of equal length")
    n = n4 // 4
    if n == 0:
        return tensor_list
    g, p, m, v = (tensor_list[i * n:(i + 1) * n] for i in range(4))
    if state is None:
        key = tuple(t.data_ptr() for t in tensor_list)
        state = _lans_states.get(key)
        if state is None:
            state = LansState(g, p, m, v)
            _lans_states.clear()
            _lans_states[key] = state
    flags = _capi.LANS_TABLES_READY if state.ready else 0
    if isinstance(step, torch.Tensor) and step.is_cuda:
        if step.dtype != torch.float32 or step.numel() != 1:
            raise TypeError("lans: a device step must be a float32 scalar")
        check(_capi.lib().lancet_lans_dev_step(_ptr(state.ws), state.ws.numel(), state.n, state.numels, state.g, state.p,
                                               state.m, state.v, _capi.F32, _ptr(step), learning_rate, beta1, beta2, eps,
                                               int(bias_correction), weight_decay, int(grad_averaging), int(mode),
                                               int(bool(normalize_grad)), flags, _stream(p[0])))
        state.ready = True
        return tensor_list
    check(_capi.lib().lancet_lans(_ptr(state.ws), state.ws.numel(), state.n, state.numels, state.g, state.p, state.m,
                                  state.v, _capi.F32, int(step), learning_rate, beta1, beta2, eps, int(bias_correction),
                                  weight_decay, int(grad_averaging), int(mode), int(bool(normalize_grad)), flags,
                                  _stream(p[0])))
    state.ready = True
    return tensor_list


def gate_softmax(h, wg, out=None):
    """probs [S,E] float32 = softmax(h @ wg.T): the gate projection in front of `moe_encode` (Gate module of the
    reference, models/benchmark/pytorch/utils.py:565-573), one warp per token in a fixed order, so that a token's
    probabilities do not depend on which other tokens are in the call.  h [S,M] float32/float16/bfloat16, wg [E,M] float32."""
    _require_cuda(h, wg, out)
    S, M = h.shape
    E = wg.shape[0]
    if wg.dtype != torch.float32 or wg.shape[1] != M:
        raise TypeError("gate_softmax: wg must be float32 [E, M]")
    out = torch.empty((S, E), dtype=torch.float32, device=h.device) if out is None else out
    check(_capi.lib().lancet_gate_softmax(_ptr(h), _dt(h), _ptr(wg), _ptr(out), S, M, E, _stream(h)))
    return out


def gate_softmax_bwd(probs, dprobs, wg, dtype):
    """Returns (dlogits [S,E] float32, dh [S,M] in `dtype`) of `gate_softmax`; the weight gradient is dlogits.T @ h."""
    _require_cuda(probs, dprobs, wg)
    S, E = probs.shape
    M = wg.shape[1]
    if probs.dtype != torch.float32 or dprobs.dtype != torch.float32 or wg.dtype != torch.float32:
        raise TypeError("gate_softmax_bwd: probs, dprobs and wg must be float32")
    dlogits = torch.empty_like(probs)
    dh = torch.empty((S, M), dtype=dtype, device=probs.device)
    check(_capi.lib().lancet_gate_softmax_bwd(_ptr(probs), _ptr(dprobs), _ptr(wg), _ptr(dlogits), _ptr(dh), _DT[dtype], S, M, E,
                                              _stream(probs)))
    return dlogits, dh


LAYER_NORM_WIDTHS = (128, 256, 512, 768, 1024, 1536, 2048)


def layer_norm_fwd(x, weight, bias, eps=1e-5, out_dtype=torch.float32, out=None, mean=None, rstd=None):
    """`raf.op.layer_norm` over the last axis of float32 rows [rows, M]; returns (y in out_dtype, mean, rstd).  `out`, `mean`
    and `rstd` may be given (contiguous, of the right shapes) to have the results written in place."""
    _require_cuda(x, weight, bias)
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or bias.dtype != torch.float32:
        raise TypeError("layer_norm_fwd: rows, weight and bias must be float32")
    x = x.contiguous()
    rows, M = x.shape
    y = torch.empty((rows, M), dtype=out_dtype, device=x.device) if out is None else out
    mean = torch.empty((rows,), dtype=torch.float32, device=x.device) if mean is None else mean
    rstd = torch.empty((rows,), dtype=torch.float32, device=x.device) if rstd is None else rstd
    if not (y.is_contiguous() and mean.is_contiguous() and rstd.is_contiguous()) or y.shape != x.shape:
        raise ValueError("layer_norm_fwd: out, mean and rstd must be contiguous and shaped like the rows")
    check(_capi.lib().lancet_layer_norm_fwd(_ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _dt(y), _ptr(mean), _ptr(rstd), rows, M,
                                            float(eps), _stream(x)))
    return y, mean, rstd


def layer_norm_bwd(x, dy, weight, mean, rstd):
    """Returns (dx float32 [rows, M], dweight [M], dbias [M]) of `layer_norm_fwd`; dy in float32 or a 16-bit type."""
    _require_cuda(x, dy, weight, mean, rstd)
    x, dy = x.contiguous(), dy.contiguous()
    rows, M = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty((M,), dtype=torch.float32, device=x.device)
    db = torch.empty((M,), dtype=torch.float32, device=x.device)
    L = _capi.lib()
    ws = workspace(x.device, L.lancet_layer_norm_workspace_bytes(rows, M), "layer_norm")
    check(L.lancet_layer_norm_bwd(_ptr(x), _ptr(dy), _dt(dy), _ptr(weight), _ptr(mean), _ptr(rstd), _ptr(dx), _ptr(dw), _ptr(db), rows,
                                  M, _ptr(ws), ws.numel(), _stream(x)))
    return dx, dw, db


def softmax_xent_fwd(logits, target, vocab):
    """Row losses and log-sum-exp of a [rows, cols >= vocab] logits matrix (columns past `vocab` are padding); target int64
    [rows], negative = ignored.  Returns (loss_rows, lse_rows), float32."""
    _require_cuda(logits, target)
    if logits.dim() != 2 or logits.stride(1) != 1 or target.dtype != torch.int64 or not target.is_contiguous():
        raise TypeError("softmax_xent_fwd: logits must be a row-major matrix and target a contiguous int64 vector")
    rows = logits.shape[0]
    loss = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    check(_capi.lib().lancet_softmax_xent_fwd(_ptr(logits), logits.stride(0), _ptr(target), rows, vocab, _dt(logits), _ptr(loss),
                                              _ptr(lse), _stream(logits)))
    return loss, lse


def softmax_xent_bwd(logits, target, vocab, lse, grad_out, scale):
    """Gradient of sum(loss_rows) * grad_out * scale with respect to the logits, in the logits' type and shape; padded
    columns and ignored rows are zero.  grad_out: float32 scalar tensor on the device (or None for 1)."""
    _require_cuda(logits, target, lse)
    rows, cols = logits.shape
    dx = torch.empty((rows, cols), dtype=logits.dtype, device=logits.device)
    if grad_out is not None and (grad_out.dtype != torch.float32 or grad_out.numel() != 1 or not grad_out.is_cuda):
        raise TypeError("softmax_xent_bwd: grad_out must be a float32 scalar on the device")
    check(_capi.lib().lancet_softmax_xent_bwd(_ptr(logits), logits.stride(0), _ptr(target), rows, vocab, cols, _dt(logits), _ptr(lse),
                                              _ptr(grad_out) if grad_out is not None else None, float(scale), _ptr(dx),
                                              dx.stride(0), _stream(logits)))
    return dx


ACT = {None: 0, "none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3}
_gemm_status = {}


def gemm_status(device):
    """Device status word of the grouped GEMM (non-zero after a bounded wait gave up)."""
    st = _gemm_status.get(device)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _gemm_status[device] = st
    return st


def grouped_gemm_nt(a, b, bias=None, counts=None, act=None, out=None, preact=None, row_begin=None):
    """Expert FFN GEMM: out[g] = act(a[g] @ b[g % LE].T + bias[g % LE]).

    a [groups, C, K], b [LE, N, K] (the nn.Linear weight layout of Experts.forward,
    models/benchmark/pytorch/utils.py:546-562 of the reference), bias [LE, N], counts int32 [groups]
    (live rows per group; rows past them are neither computed nor written).  With row_begin (int32 [groups])
    only the rows [row_begin[g] rounded down to 128, counts[g]) of every group are computed (pipeline stages)."""
    _require_cuda(a, b, bias, counts, out, preact, row_begin)
    groups, C, K = a.shape
    LE, N, K2 = b.shape
    if K2 != K or groups % LE:
        raise ValueError("grouped_gemm_nt: shapes do not match")
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("grouped_gemm_nt: bfloat16 or float16 operands of one type")
    out = torch.empty((groups, C, N), dtype=a.dtype, device=a.device) if out is None else out
    st = gemm_status(a.device)
    check(_capi.lib().lancet_grouped_gemm_nt_window(_ptr(a), _ptr(b), _ptr(out), _ptr(bias), _ptr(preact), groups, LE, C, N,
                                                    K, _ptr(row_begin), _ptr(counts), ACT[act], _dt(a), _ptr(st),
                                                    _stream(a)))
    return out


def grouped_gemm_nn(a, b, counts=None, act=None, preact=None, out=None, row_begin=None):
    """Data gradient: out[g] = (a[g] @ b[g % LE]) * act'(preact[g]); a [groups, C, K], b [LE, K, N].
    row_begin as in grouped_gemm_nt."""
    _require_cuda(a, b, counts, out, preact, row_begin)
    groups, C, K = a.shape
    LE, K2, N = b.shape
    if K2 != K or groups % LE:
        raise ValueError("grouped_gemm_nn: shapes do not match")
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("grouped_gemm_nn: bfloat16 or float16 operands of one type")
    out = torch.empty((groups, C, N), dtype=a.dtype, device=a.device) if out is None else out
    st = gemm_status(a.device)
    check(_capi.lib().lancet_grouped_gemm_nn_window(_ptr(a), _ptr(b), _ptr(out), _ptr(preact), groups, LE, C, N, K,
                                                    _ptr(row_begin), _ptr(counts), ACT[act], _dt(a), _ptr(st), _stream(a)))
    return out


def sparse_expert_matmul_nt(data, weight, nelements_per_gpu, nelements_offset=0, nelements_stride=1, nelements_scale=1,
                            out=None):
    """`raf.op.sparse_expert_matmul_nt` (scripts/src_codegen/def_schema.py:711-718 of the reference):
    data [C, G, M], weight [N, M], nelements_per_gpu uint64 [G*stride] -> [C, G, N]; source block g has
    nelements_per_gpu[offset + g*stride] * scale / M live rows, the other rows of the output are zero."""
    _require_cuda(data, weight, nelements_per_gpu, out)
    C, G, M = data.shape
    N, M2 = weight.shape
    if M2 != M:
        raise ValueError("Input data and weight should have matching shape in dim 2 and 1, respectively.")
    if nelements_per_gpu.dim() != 1 or nelements_per_gpu.numel() // nelements_stride != G:
        raise ValueError("Input data and nelements should have matching shape in dim 1 and 0 after stride.")
    if data.dtype != weight.dtype or data.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("sparse_expert_matmul_nt: bfloat16 or float16 operands of one type")
    if nelements_per_gpu.dtype not in (torch.uint64, torch.int64):
        raise TypeError("sparse_expert_matmul_nt: nelements_per_gpu must be a 64-bit integer tensor")
    out = torch.empty((C, G, N), dtype=data.dtype, device=data.device) if out is None else out
    L = _capi.lib()
    nws = L.lancet_sparse_expert_matmul_nt_workspace_bytes(G)
    ws = workspace(data.device, nws, "sparse_expert_matmul_nt")
    check(L.lancet_sparse_expert_matmul_nt(_ptr(data), _ptr(weight), _ptr(out), _ptr(nelements_per_gpu), nelements_offset,
                                           nelements_stride, nelements_scale, C, G, M, N, _dt(data), _ptr(ws), nws,
                                           _stream(data)))
    return out


def grouped_gemm_tn(a, b, n_local_experts, counts=None, out=None):
    """Weight gradient: out[e] = sum_{g % LE == e} a[g, :n_g].T @ b[g, :n_g]; a [groups, C, Mout], b [groups, C, N]."""
    _require_cuda(a, b, counts, out)
    groups, C, Mout = a.shape
    N = b.shape[2]
    if b.shape[0] != groups or b.shape[1] != C or groups % n_local_experts:
        raise ValueError("grouped_gemm_tn: shapes do not match")
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("grouped_gemm_tn: bfloat16 or float16 operands of one type")
    out = torch.empty((n_local_experts, Mout, N), dtype=a.dtype, device=a.device) if out is None else out
    st = gemm_status(a.device)
    check(_capi.lib().lancet_grouped_gemm_tn(_ptr(a), _ptr(b), _ptr(out), groups, n_local_experts, C, Mout, N,
                                             _ptr(counts), _dt(a), _ptr(st), _stream(a)))
    return out


def _ptr_table(ts):
    return (ctypes.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


def moe_merge_masks(indices_locations, n_experts):
    """`raf.op.moe_merge_masks`: list of n [2,S] masks -> [2, n*S] with running per-expert offsets."""
    _require_cuda(*indices_locations)
    n, S = len(indices_locations), indices_locations[0].shape[1]
    dev = indices_locations[0].device
    out = torch.empty((2, n * S), dtype=torch.int32, device=dev)
    L = _capi.lib()
    ws = workspace(dev, L.lancet_moe_partition_workspace_bytes(n, n_experts), "partition")
    check(L.lancet_moe_merge_masks(_ptr_table(indices_locations), n, S, n_experts, _ptr(out), _ptr(ws), ws.numel(),
                                   _stream(out)))
    return out


def moe_redispatch(data, indices_locations):
    """`raf.op.moe_redispatch`: n partitioned [E,C,M] buffers -> one compacted [E,C,M]."""
    _require_cuda(*data, *indices_locations)
    n = len(data)
    E, C, M = data[0].shape
    S = indices_locations[0].shape[1]
    out = torch.empty_like(data[0])
    L = _capi.lib()
    ws = workspace(out.device, L.lancet_moe_partition_workspace_bytes(n, E), "partition")
    check(L.lancet_moe_redispatch(_ptr_table(data), _ptr_table(indices_locations), n, S, M, C, E, _dt(out), _ptr(out),
                                  _ptr(ws), ws.numel(), _stream(out)))
    return out


def moe_redispatch_expert_input(data, recv_cnts, local_expert_id, n_local_experts, recv_cnts_scale=1):
    """`raf.op.moe_redispatch_expert_input`: n post-exchange [C,G,M] inputs -> one compacted [C,G,M]."""
    _require_cuda(*data, *recv_cnts)
    C, G, M = data[0].shape
    out = torch.empty_like(data[0])
    check(_capi.lib().lancet_moe_redispatch_expert_input(_ptr_table(data), _ptr_table(recv_cnts), len(data), local_expert_id,
                                                         n_local_experts, C, G, M, recv_cnts_scale, _dt(out), _ptr(out),
                                                         _stream(out)))
    return out


def moe_encode_batch_prioritized(data, gate, n_partitions=1, partition_id=0, capacity_factor=1.0):
    """`raf.op.moe_encode_batch_prioritized`: data [S_orig, M] and gate [S_orig, E] of the whole batch;
    returns the tuple5 of `moe_encode` for partition `partition_id`."""
    _require_cuda(data, gate)
    S_orig, M = data.shape
    E = gate.shape[1]
    if S_orig % n_partitions:
        raise ValueError("S must be divisible by n_partitions")
    Sp = S_orig // n_partitions
    dev = data.device
    L = _capi.lib()
    C = L.lancet_moe_capacity(Sp, E, capacity_factor, 1)
    gates_s = torch.empty((Sp,), dtype=torch.float32, device=dev)
    idx_loc = torch.empty((2, Sp), dtype=torch.int32, device=dev)
    capused = torch.empty((E,), dtype=torch.int32, device=dev)
    elems = torch.empty((E,), dtype=torch.uint64, device=dev)
    disp = torch.empty((E, C, M), dtype=data.dtype, device=dev)
    ws = workspace(dev, L.lancet_moe_gate_bpr_workspace_bytes(S_orig, E), "bpr")
    check(L.lancet_moe_encode_bpr(_ptr(data), _ptr(gate), _dt(gate), n_partitions, partition_id, capacity_factor, S_orig, M,
                                  E, _dt(data), _ptr(gates_s), _capi.F32, _ptr(idx_loc), _ptr(capused), _ptr(elems),
                                  _ptr(disp), _ptr(ws), ws.numel(), _stream(data)))
    return gates_s, idx_loc, capused, elems, disp


def grouped_bias_grad(dy, n_local_experts, counts=None, out=None):
    """Bias gradient of an expert layer: out[e] = sum of the live rows of dy[g] over the groups g of expert e."""
    _require_cuda(dy, counts, out)
    groups, C, N = dy.shape
    out = torch.empty((n_local_experts, N), dtype=dy.dtype, device=dy.device) if out is None else out
    L = _capi.lib()
    ws = workspace(dy.device, L.lancet_grouped_bias_grad_workspace_bytes(n_local_experts, N), "bias_grad")
    check(L.lancet_grouped_bias_grad(_ptr(dy), _ptr(out), groups, n_local_experts, C, N, _ptr(counts), _dt(dy), _ptr(ws),
                                     ws.numel(), _stream(dy)))
    return out
