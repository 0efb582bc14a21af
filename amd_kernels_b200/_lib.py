"""ctypes binding of libb200moe.so (the C ABI declared in include/b200_moe.h). There is no fallback: when the library
is missing or does not load, every entry point of the package raises."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200moe.so")


def lib_path(inter: int = 768) -> str:
    """The library built for intermediate size ``inter``: 768 (the i768 package) or 1536 (its TP2 sibling shape)."""
    return LIB_PATH if inter == 768 else os.path.join(HERE, f"libb200moe_i{inter}.so")


E_ARG, E_ALIGN, E_DRIVER, E_TOO_LARGE = -1, -2, -3, -4
DEV_TIMEOUT, DEV_BAD_INDEX = 1, 2
ROUTE_SIGMOID_BIAS, ROUTE_SOFTMAX = 0, 1


class Weights(Structure):
    """struct b200moe_weights"""
    _fields_ = [("w13t", c_void_p), ("w2t", c_void_p), ("bias", c_void_p),
                ("num_experts", c_int), ("route_mode", c_int), ("route_scale", c_float), ("gate", c_void_p),
                ("gate_split", c_void_p)]


_P = c_void_p
SIGNATURES = {
    "b200moe_version": (c_int, []),
    "b200moe_arch": (c_char_p, []),
    "b200moe_max_sorted_rows": (c_int64, [c_int64, c_int, c_int]),
    "b200moe_block_rows": (c_int, [c_int64]),
    "b200moe_preshuffle_w13": (c_int, [_P, _P, c_int, _P, _P]),
    "b200moe_preshuffle_w2": (c_int, [_P, _P, c_int, _P, _P]),
    "b200moe_router_splits": (c_int, [c_int64]),
    "b200moe_router_gemm": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P]),
    "b200moe_router_split_gate": (c_int, [_P, c_int, _P, _P]),
    "b200moe_router_gemm_tc": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P, _P]),
    "b200moe_route_topk": (c_int, [_P, c_int64, c_int64, c_int, _P, c_int64, c_int, c_int, c_float, _P, _P, _P]),
    "b200moe_quant_mxfp4": (c_int, [_P, c_int64, c_int, _P, _P, _P]),
    "b200moe_permute_scratch_bytes": (c_size_t, [c_int64, c_int]),
    "b200moe_permute": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P, _P, _P, _P, _P]),
    "b200moe_permute_live": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P, _P, _P, _P, _P, _P]),
    "b200moe_ep_dest": (c_int, [_P, c_int64, c_int, c_int, c_int, _P, _P, _P]),
    "b200moe_ep_offsets": (c_int, [_P, c_int, c_int, _P, _P, _P, _P]),
    "b200moe_ep_sync": (c_int, [_P, _P, _P, c_int, c_int, _P, _P, _P]),
    "b200moe_permute_static": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P, _P, _P, _P]),
    "b200moe_route_sort": (c_int, [_P, _P, c_int64, c_int, c_int, c_float, c_int, _P, _P, _P, _P, _P, _P, _P, _P]),
    "b200moe_dispatch_rows": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_int, c_int64, _P, _P, _P]),
    "b200moe_quant_dispatch": (c_int, [_P, _P, _P, c_int64, c_int, c_int64, _P, _P, _P, _P]),
    "b200moe_gemm12": (c_int, [_P, _P, c_int, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int64, _P, _P, _P, _P, _P, _P]),
    "b200moe_quant_push": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, c_int64,
                                   _P, _P]),
    "b200moe_gemm1_swiglu_quant": (c_int, [_P, c_int, _P, _P, _P, _P, c_int64, c_int, _P, _P, _P, _P, _P]),
    "b200moe_gemm1_pair_supported": (c_int, []),
    "b200moe_gemm1_swiglu_quant_pair": (c_int, [_P, c_int, _P, _P, _P, _P, c_int64, _P, _P, _P, _P]),
    "b200moe_gemm1_swiglu_quant_wide": (c_int, [_P, c_int, _P, _P, _P, _P, c_int64, _P, _P, _P, _P]),
    "b200moe_gemm1_swiglu_quant_gather": (c_int, [_P, c_int, _P, _P, c_int64, c_int, _P, _P, _P, c_int64, _P, _P, _P, _P]),
    "b200moe_gemm1_swiglu_quant_gather_range": (c_int, [_P, c_int, _P, _P, c_int64, c_int, _P, _P, _P, c_int64, _P, _P, _P,
                                                        c_int, _P, _P]),
    "b200moe_block_chunks": (c_int, [_P, c_int, c_int, _P, _P]),
    "b200moe_gemm2_weighted": (c_int, [_P, c_int, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int64, _P, _P, _P]),
    "b200moe_gemm2_weighted_peer": (c_int, [_P, c_int, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int64, _P, _P, _P, c_int,
                                            c_int64, _P, _P]),
    "b200moe_gemm2_weighted_peer_range": (c_int, [_P, c_int, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int64, _P, _P, _P,
                                                  c_int, c_int64, _P, c_int, _P, _P]),
    "b200moe_gemm1_simt": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int64, _P, _P, _P]),
    "b200moe_gemm2_simt": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_int64, _P, _P]),
    "b200moe_reduce_slots": (c_int, [_P, _P, c_int64, _P, _P]),
    "b200moe_reduce_rows": (c_int, [_P, _P, _P, c_int64, _P, _P]),
    "b200moe_preshuffle_shared": (c_int, [_P, _P, _P, _P, _P, _P, _P]),
    "b200moe_shared_block_rows": (c_int, [c_int64]),
    "b200moe_shared_quant": (c_int, [_P, c_int64, c_int, _P, _P, _P]),
    "b200moe_shared_workspace_bytes": (c_size_t, [c_int64]),
    "b200moe_shared_expert": (c_int, [_P, _P, _P, c_int64, _P, c_size_t, _P, _P, _P]),
    "b200moe_shared_quant_rows": (c_int, [_P, c_int64, _P, _P, _P]),
    "b200moe_shared_expert_quantized": (c_int, [_P, _P, _P, _P, c_int64, _P, c_size_t, _P, _P, _P]),
    "b200moe_scales_to_atoms": (c_int, [_P, c_int64, c_int, c_int, _P, _P]),
    "b200moe_sidecar_pack": (c_int, [_P, _P, _P, _P, c_int64, _P, _P]),
    "b200moe_sidecar_unpack": (c_int, [_P, _P, _P, _P, c_int64, _P, _P]),
    "b200moe_router_gemm_quant": (c_int, [_P, _P, c_int64, c_int, c_int, _P, _P, _P, _P, _P, _P]),
    "b200moe_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "b200moe_workspace_bytes_x": (c_size_t, [c_int64, c_int]),
    "b200moe_forward_x": (c_int, [POINTER(Weights), _P, c_int64, _P, c_size_t, _P, _P, _P, _P]),
    "b200moe_set_wait_limit_ns": (c_int, [c_uint64]),
    "b200moe_route_sort_partials": (c_int, [_P, c_int64, c_int64, c_int, _P, c_int64, c_int, c_int, c_float, c_int, _P, _P,
                                            _P, _P, _P, _P, _P, _P]),
    "b200moe_reduce_slots_add_rmsnorm_quant": (c_int, [_P, _P, _P, _P, c_float, c_int64, _P, _P, _P, _P, _P]),
    "b200moe_forward": (c_int, [POINTER(Weights), _P, _P, c_int64, _P, c_size_t, _P, _P, _P, _P]),
    "b200moe_forward_host": (c_int, [POINTER(Weights), _P, _P, c_int64, _P, _P, _P, c_size_t, _P, _P, _P, _P, _P]),
}

_libs: dict = {}


def load(inter: int = 768) -> ctypes.CDLL:
    """The loaded library (for intermediate size ``inter``) with typed entry points. Raises RuntimeError when it is absent
    or unloadable."""
    if inter not in _libs:
        path = lib_path(inter)
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with `python -m amd_kernels_b200.build` "
                               "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise RuntimeError(f"cannot load {path}: {exc}") from exc
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _libs[inter] = lib
    return _libs[inter]


def check(code: int, what: str) -> None:
    """Turns a non-zero status of an entry point into an exception (ValueError for rejected arguments)."""
    if code == 0:
        return
    if code in (E_ARG, E_ALIGN):
        raise ValueError(f"{what}: rejected argument ({'alignment' if code == E_ALIGN else 'size, pointer or block height'})")
    if code == E_TOO_LARGE:
        raise ValueError(f"{what}: more tokens than the allocation-free entry point supports")
    if code == E_DRIVER:
        raise RuntimeError(f"{what}: the CUDA driver cannot encode tensor maps")
    raise RuntimeError(f"{what}: CUDA error {code}")
