"""MXFP4 routed MoE H6144 I768 E128 top4 on B200 — the public names of the reference's
``amd_kernels.moe.mxfp4_h6144_i768_e128_top4`` (its __init__.py:11-16) for the routed experts and the MXFP8 shared expert."""
from .chain import MoeWeights, mxfp4_moe, warm_up_mxfp4_moe, unsupported_reason, route, mxfp4_moe_experts
from .shared_expert import SharedWeights, set_dbo_query
from .tail import slots4_add_rmsnorm_mxfp8
from .prepared_input import MoeInput, MoeInputCompact, prepare_mxfp4_moe, gather_mxfp4_moe

__all__ = ["MoeWeights", "SharedWeights", "mxfp4_moe", "warm_up_mxfp4_moe", "unsupported_reason", "route",
           "mxfp4_moe_experts", "MoeInput", "MoeInputCompact", "prepare_mxfp4_moe", "gather_mxfp4_moe", "set_dbo_query",
           "slots4_add_rmsnorm_mxfp8"]

H, I, E, TOPK = 6144, 768, 128, 4  # noqa: E741
SWIGLU_OAI = (1.702, 7.0, 1.0)  # alpha, limit, beta (up + beta)
