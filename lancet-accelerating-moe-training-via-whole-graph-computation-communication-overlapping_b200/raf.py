"""Drive the operators through the RAF-style registry of the library (declare -> allocate outputs ->
dispatch by dialect priority -> satisfy requests -> execute), the way the reference's interpreter
runs an op (src/impl/interpreter.cc:246-337).  torch supplies the output memory."""
import ctypes

import torch

from . import _capi
from ._capi import RafValue

_CODE = {torch.float32: (2, 32), torch.float16: (2, 16), torch.bfloat16: (4, 16), torch.int32: (0, 32),
         torch.int64: (0, 64), torch.uint64: (1, 64)}
_FROM = {v: k for k, v in _CODE.items()}


class RafError(RuntimeError):
    pass


def _tensor_value(t):
    v = RafValue()
    v.kind = 1
    v.data = t.data_ptr()
    v.dtype_code, v.dtype_bits = _CODE[t.dtype]
    v.ndim = t.dim()
    for i, s in enumerate(t.shape):
        v.shape[i] = s
    v.device_type = 2 if t.is_cuda else 1
    return v


def _flatten(args):
    out = []
    for a in args:
        if isinstance(a, torch.Tensor):
            if not a.is_contiguous():
                raise ValueError("tensors must be contiguous")
            out.append(_tensor_value(a))
        elif isinstance(a, (list, tuple)):
            v = RafValue()
            v.kind = 2
            v.ndim = len(a)
            out.append(v)
            out.extend(_flatten(a))
        elif isinstance(a, bool) or isinstance(a, int):
            v = RafValue()
            v.kind = 3
            v.scalar = float(int(a))
            out.append(v)
        elif isinstance(a, float):
            v = RafValue()
            v.kind = 4
            v.scalar = a
            out.append(v)
        else:
            raise TypeError("unsupported argument %r" % (a,))
    return out


def dialect_ops(base_op):
    buf = ctypes.create_string_buffer(1024)
    _capi.lib().lancet_raf_dialect_ops(base_op.encode(), buf, 1024)
    return [tuple(e.split(":")) for e in buf.value.decode().split(";") if e]


def declare(op, *args):
    """[(shape, dtype), ...] of the outputs of `op` for these arguments."""
    L = _capi.lib()
    vals = _flatten(args)
    arr = (RafValue * len(vals))(*vals)
    outs = (RafValue * 64)()
    n = ctypes.c_int(0)
    if L.lancet_raf_declare(op.encode(), arr, len(vals), outs, 64, ctypes.byref(n)):
        raise RafError(L.lancet_raf_last_error().decode())
    return [(tuple(outs[i].shape[j] for j in range(outs[i].ndim)), _FROM[(outs[i].dtype_code, outs[i].dtype_bits)])
            for i in range(n.value)]


def call(op, *args, device=None):
    """Run `op` through the registry; returns (list of output tensors, dialect op that ran)."""
    L = _capi.lib()
    vals = _flatten(args)
    arr = (RafValue * len(vals))(*vals)
    specs = declare(op, *args)
    if device is None:
        device = next(a.device for a in _iter_tensors(args) if a.is_cuda)
    if op == "raf.op.lans":
        outs_t = list(args[0])                       # in place: outputs alias the inputs
    else:
        outs_t = [torch.empty(shape, dtype=dt, device=device) for shape, dt in specs]
    ovals = [_tensor_value(t) for t in outs_t]
    oarr = (RafValue * max(1, len(ovals)))(*ovals)
    name = ctypes.create_string_buffer(128)
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    with torch.cuda.device(device):
        rc = L.lancet_raf_execute(op.encode(), arr, len(vals), oarr, len(ovals), name, 128, stream)
    if rc:
        raise RafError(L.lancet_raf_last_error().decode())
    return outs_t, name.value.decode()


def _iter_tensors(args):
    for a in args:
        if isinstance(a, torch.Tensor):
            yield a
        elif isinstance(a, (list, tuple)):
            yield from _iter_tensors(a)
