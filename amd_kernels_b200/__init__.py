"""B200-native kernels behind the amd_kernels entry points. Only the routed MXFP4 MoE block is provided:
``amd_kernels_b200.moe.mxfp4_h6144_i768_e128_top4`` mirrors ``amd_kernels.moe.mxfp4_h6144_i768_e128_top4``."""
