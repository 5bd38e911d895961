"""ctypes binding of the C ABI declared in include/lancet_b200.h.

The library is the product: there is no Python or CPU fallback.  `lib()` raises if the
shared object has not been built (run `python -m lancet_b200.build` or `__graft_entry__.build()`).
"""
import ctypes
import os
import re

from . import build as _build

_LIB = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_float = ctypes.c_float
c_size_t = ctypes.c_size_t
c_i64 = ctypes.c_int64

INCLUDE_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "include")
HEADER = os.path.join(INCLUDE_DIR, "lancet_b200.h")


class RafValue(ctypes.Structure):
    """lancet_raf_value_t of include/lancet_raf_shim.h"""
    _fields_ = [("kind", ctypes.c_int), ("data", ctypes.c_void_p), ("dtype_code", ctypes.c_int),
                ("dtype_bits", ctypes.c_int), ("ndim", ctypes.c_int), ("shape", ctypes.c_int64 * 6),
                ("scalar", ctypes.c_double), ("device_type", ctypes.c_int)]

# name -> (restype, argtypes).  Kept next to the header; tests check that both list the same names.
SIGNATURES = {
    "lancet_last_error": (ctypes.c_char_p, []),
    "lancet_version": (ctypes.c_char_p, []),
    "lancet_abi_version": (c_int, []),
    "lancet_launch_count": (ctypes.c_ulonglong, []),
    "lancet_profile_begin": (c_int, [ctypes.c_char_p]),
    "lancet_profile_end": (c_int, [ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_longlong)]),
    "lancet_moe_capacity": (c_int, [c_int, c_int, c_float, c_int]),
    "lancet_moe_gate_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "lancet_moe_gate": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
                                c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "lancet_moe_gate_chained_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lancet_moe_gate_chained": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                        c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int, c_void_p]),
    "lancet_moe_gate_static_max_bytes": (c_size_t, []),
    "lancet_moe_gate_static": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "lancet_moe_encode_fwd": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_void_p]),
    "lancet_moe_zero_tail": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "lancet_moe_encode": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int,
                                  c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_int,
                                  c_void_p]),
    "lancet_moe_decode_fwd": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      c_int, c_void_p]),
    "lancet_moe_encode_bwd_data": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p]),
    "lancet_moe_encode_bwd_gate": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                                           c_void_p]),
    "lancet_moe_decode_bwd_data": (c_int, [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                           c_int, c_int, c_int, c_void_p]),
    "lancet_moe_decode_bwd_gate": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                           c_int, c_int, c_void_p]),
    "lancet_moe_dispatch_chunked_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "lancet_moe_dispatch_chunked": (c_int, [c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                            c_void_p]),
    "lancet_moe_scatter_chunked": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p]),
    "lancet_moe_combine_chunked": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_void_p, c_void_p]),
    "lancet_symm_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p), ctypes.c_char_p]),
    "lancet_symm_open": (c_int, [ctypes.c_char_p, ctypes.POINTER(c_void_p)]),
    "lancet_symm_close": (c_int, [c_void_p]),
    "lancet_symm_free": (c_int, [c_void_p]),
    "lancet_p2p_barrier": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, ctypes.c_uint, ctypes.c_ulonglong, c_void_p,
                                   c_void_p]),
    "lancet_p2p_barrier_counted": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p, ctypes.c_ulonglong, c_void_p,
                                           c_void_p]),
    "lancet_p2p_status": (c_int, [c_void_p, c_void_p]),
    "lancet_moe_dispatch_chunked_p2p": (c_int, [c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int, c_int, c_int,
                                                c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_void_p, c_size_t,
                                                c_int, c_void_p]),
    "lancet_moe_combine_chunked_p2p": (c_int, [ctypes.POINTER(c_void_p), c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                               c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "lancet_comm_unique_id": (c_int, [ctypes.c_char_p]),
    "lancet_comm_init_rank": (c_int, [ctypes.c_char_p, c_int, c_int, ctypes.POINTER(c_void_p)]),
    "lancet_comm_destroy": (c_int, [c_void_p]),
    "lancet_all_to_all": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "lancet_all_to_all_p2p": (c_int, [c_void_p, ctypes.POINTER(c_void_p), c_size_t, c_int, c_int, c_void_p]),
    "lancet_all_to_allv_p2p": (c_int, [c_void_p, ctypes.POINTER(c_void_p), c_void_p, ctypes.POINTER(c_void_p), c_int,
                                       c_size_t, c_size_t, c_int, c_int, c_void_p]),
    "lancet_grouped_gemm_nt": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "lancet_grouped_gemm_nn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                       c_int, c_int, c_void_p, c_void_p]),
    "lancet_grouped_gemm_tn": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                       c_void_p, c_void_p]),
    "lancet_all_to_all_tuple": (c_int, [ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_size_t), c_int,
                                        c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "lancet_all_to_all_evenly": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "lancet_raf_last_error": (ctypes.c_char_p, []),
    "lancet_raf_declare": (c_int, [ctypes.c_char_p, ctypes.POINTER(RafValue), c_int, ctypes.POINTER(RafValue), c_int,
                                   ctypes.POINTER(c_int)]),
    "lancet_raf_execute": (c_int, [ctypes.c_char_p, ctypes.POINTER(RafValue), c_int, ctypes.POINTER(RafValue), c_int,
                                   ctypes.c_char_p, c_int, c_void_p]),
    "lancet_raf_set_communicator": (c_int, [c_void_p, c_int, c_int]),
    "lancet_raf_dialect_ops": (c_int, [ctypes.c_char_p, ctypes.c_char_p, c_int]),
    "lancet_moe_gate_bpr_workspace_bytes": (c_size_t, [c_int, c_int]),
    "lancet_moe_gate_bpr": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "lancet_moe_encode_bpr": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p,
                                      c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]),
    "lancet_moe_partition_workspace_bytes": (c_size_t, [c_int, c_int]),
    "lancet_moe_merge_masks": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "lancet_moe_redispatch": (c_int, [ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_void_p, c_void_p, c_size_t, c_void_p]),
    "lancet_moe_redispatch_expert_input": (c_int, [ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_int, c_int,
                                                   c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "lancet_moe_combine_bwd_p2p": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p]),
    "lancet_moe_combine_bwd_part_p2p": (c_int, [c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                c_void_p]),
    "lancet_grouped_gemm_nt_window": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                              c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "lancet_grouped_gemm_nn_window": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                              c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "lancet_moe_gate_chunked_p2p": (c_int, [c_void_p, c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                            c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), c_void_p,
                                            c_size_t, c_void_p]),
    "lancet_moe_dispatch_rows_p2p": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                             c_int, c_int, c_int, ctypes.POINTER(c_void_p), c_void_p]),
    "lancet_moe_stage_windows": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "lancet_sparse_expert_matmul_nt_workspace_bytes": (c_size_t, [c_int]),
    "lancet_sparse_expert_matmul_nt": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                               c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "lancet_all_to_allv": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_void_p, c_void_p]),
    "lancet_grouped_bias_grad_workspace_bytes": (c_size_t, [c_int, c_int]),
    "lancet_grouped_bias_grad": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_size_t,
                                         c_void_p]),
    "lancet_lans_workspace_bytes": (c_size_t, [c_int, ctypes.POINTER(c_i64)]),
    "lancet_lans": (c_int, [c_void_p, c_size_t, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_void_p),
                            ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int, c_int,
                            c_float, c_float, c_float, c_float, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p]),
    "lancet_moe_gate_chunks_p2p": (c_int, [c_void_p, c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_int, c_void_p, c_void_p, c_void_p, c_void_p, ctypes.POINTER(c_void_p), c_void_p,
                                           c_size_t, c_void_p]),
    "lancet_moe_stage_window": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                        c_void_p, c_void_p]),
    "lancet_gate_softmax": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "lancet_gate_softmax_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_void_p]),
    "lancet_set_cta_limits": (c_int, [c_int, c_int]),
    "lancet_set_gemm_paired": (c_int, [c_int]),
    "lancet_set_chained_launch": (c_int, [c_int]),
    "lancet_layer_norm_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, ctypes.c_float,
                                      c_void_p]),
    "lancet_layer_norm_workspace_bytes": (ctypes.c_size_t, [c_int, c_int]),
    "lancet_layer_norm_bwd": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                      c_int, c_void_p, ctypes.c_size_t, c_void_p]),
    "lancet_softmax_xent_fwd": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "lancet_softmax_xent_bwd": (c_int, [c_void_p, ctypes.c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                        ctypes.c_float, c_void_p, ctypes.c_longlong, c_void_p]),
    "lancet_peer_copy": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "lancet_lans_dev_step": (c_int, [c_void_p, c_size_t, c_int, ctypes.POINTER(c_i64), ctypes.POINTER(c_void_p),
                                     ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p), c_int,
                                     c_void_p, c_float, c_float, c_float, c_float, c_int, c_float, c_int, c_int, c_int, c_int,
                                     c_void_p]),
}

F32, F16, BF16 = 0, 1, 2
OK = 0
ENCODE_GLOBAL_LOC, ENCODE_NO_ZERO = 1, 2
GATE_GLOBAL_LOC = 1
LANS_TABLES_READY = 1
P2P_NO_REMOTE_ZERO = 1
ERR_TIMEOUT = 4


class LancetError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("lancet_b200 error %d: %s" % (code, text))
        self.code = code


def header_symbols():
    """Names of all functions declared in include/*.h."""
    names = set()
    for fn in sorted(os.listdir(INCLUDE_DIR)):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(INCLUDE_DIR, fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(lancet_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def lib_path():
    return _build.LIB_PATH


def lib():
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(
                "lancet_b200: %s is missing. Build it with `python -m lancet_b200.build`; there is no fallback path."
                % path)
        handle = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def check(status):
    if status != OK:
        raise LancetError(status, lib().lancet_last_error().decode("utf-8", "replace"))
