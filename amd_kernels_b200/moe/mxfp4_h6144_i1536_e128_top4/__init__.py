"""MXFP4 routed MoE H6144 I1536 E128 top4 on B200 -- the TP2 sibling of the i768 package, the public names of the
reference's ``amd_kernels.moe.mxfp4_h6144_i1536_e128_top4`` (its __init__.py:11-18). The kernels are the i768 package's
sources built a second time with the intermediate size 1536 (``libb200moe_i1536.so``: 24 W13 tiles and 6 K-tiles in GEMM2 per
expert instead of 12 and 3); the host side is the same code, which takes the shape from the weights it is given. Only
``MoeWeights`` / ``SharedWeights`` differ: their ``from_row_major`` insist on this package's shapes."""
from ..mxfp4_h6144_i768_e128_top4 import chain as _chain
from ..mxfp4_h6144_i768_e128_top4 import shared_expert as _shared
from ..mxfp4_h6144_i768_e128_top4.chain import mxfp4_moe, warm_up_mxfp4_moe, route, mxfp4_moe_experts
from ..mxfp4_h6144_i768_e128_top4.prepared_input import MoeInput, MoeInputCompact, prepare_mxfp4_moe, gather_mxfp4_moe
from ..mxfp4_h6144_i768_e128_top4.shared_expert import set_dbo_query
from ..mxfp4_h6144_i768_e128_top4.tail import slots4_add_rmsnorm_mxfp8

H, I, E, TOPK = 6144, 1536, 128, 4  # noqa: E741
SWIGLU_OAI = (1.702, 7.0, 1.0)  # alpha, limit, beta (up + beta)
SHARED_FULL = False  # SharedWeights takes the TP2 shard [2 * 1536, 6144] / [6144, 1536], not the full 3072-wide expert


class MoeWeights(_chain.MoeWeights):
    """``MoeWeights`` of the i1536 shape: w13 [E, 3072, 3072] u8, w2 [E, 6144, 768] u8 and their e8m0 scales."""
    INTERMEDIATE = I


class SharedWeights(_shared.SharedWeights):
    """``SharedWeights`` of the i1536 shape: w13 e4m3 [3072, 6144], w2 e4m3 [6144, 1536] and their e8m0 scales."""
    INTERMEDIATE = I


def unsupported_reason(w13, w13_scale, w2, w2_scale, shared_w13, shared_s13, shared_w2, shared_s2, swiglu=SWIGLU_OAI,
                       **kwargs):
    """None when ``MoeWeights.from_row_major`` (with ``SharedWeights``) takes these checkpoint-layout tensors, else the
    reason (reference __init__.py:24-45 of the i1536 package; the full, unsharded shared expert is not taken here)."""
    return _chain.unsupported_reason(w13, w13_scale, w2, w2_scale, shared_w13, shared_s13, shared_w2, shared_s2, swiglu,
                                     inter=I, **kwargs)


__all__ = ["MoeWeights", "SharedWeights", "mxfp4_moe", "warm_up_mxfp4_moe", "MoeInput", "MoeInputCompact",
           "prepare_mxfp4_moe", "gather_mxfp4_moe", "set_dbo_query", "unsupported_reason", "route", "mxfp4_moe_experts",
           "slots4_add_rmsnorm_mxfp8", "SHARED_FULL"]
