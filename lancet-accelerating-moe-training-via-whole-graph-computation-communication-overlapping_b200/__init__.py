"""lancet_b200: B200-native MoE dispatch/combine, all-to-all, expert GEMM and LANS behind the
operator surface of the reference (RAF `moe_encode`, `moe_decode`, `_all_to_all`, `lans`)."""
from . import _capi, build, raf  # noqa: F401
from ._capi import LancetError  # noqa: F401
from .pipeline import ChunkedMoE  # noqa: F401
from .layer import MoELayer  # noqa: F401
from .autograd import LayerNorm, MoE, softmax_cross_entropy  # noqa: F401
from .collective import Communicator, SymmAllToAll  # noqa: F401
from .dist import DistChunkedMoE, LocalFabric, ProcessFabric, tensor_from_ptr  # noqa: F401
from .ops import (  # noqa: F401
    LansState, gate_softmax, gate_softmax_bwd, gemm_status, grouped_bias_grad, grouped_gemm_nn, grouped_gemm_nt, grouped_gemm_tn, sparse_expert_matmul_nt, lans, moe_capacity, moe_decode, moe_decode_dg, moe_decode_dx, moe_encode, moe_encode_dg,
    moe_encode_batch_prioritized, moe_encode_dx, moe_encode_fwd, moe_gate, moe_merge_masks, moe_redispatch, moe_redispatch_expert_input,
    layer_norm_bwd, layer_norm_fwd, moe_zero_tail, softmax_xent_bwd, softmax_xent_fwd, workspace,
)
