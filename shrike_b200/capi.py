"""ctypes declarations of the C ABI in include/shrike_b200.h.

Loading the library never falls back to anything: if the shared object is
missing or a symbol is absent the import raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libshrike_b200.so"

DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
ACT_SILU, ACT_GELU_TANH, ACT_CLAMPED_SWIGLU = 0, 1, 2
ROUTER_SOFTMAX, ROUTER_SIGMOID = 0, 1
IO_PENDING, IO_READY, IO_FAILED = 0, 1, 2
SLOT_MISS = 0xFFFFFFFF
MAX_DECODE_TOKENS = 64
STATIC_ROUTER_MAX_ROWS = 64
EP_MAX_WORLD = 16
EP_HANDLE_BYTES = 64

OK, EINVAL, ENOMEM, ERANGE, EIO, ETIMEDOUT = 0, 22, 12, 34, 5, 110


class MoEConfig(C.Structure):
    _fields_ = [
        ("d", C.c_uint32), ("f", C.c_uint32), ("num_experts", C.c_uint32), ("top_k", C.c_uint32),
        ("weight_bits", C.c_uint32), ("group_size", C.c_uint32), ("meta_dtype", C.c_uint32),
        ("act_dtype", C.c_uint32), ("activation", C.c_uint32), ("expert_bias", C.c_uint32),
        ("router_kind", C.c_uint32), ("routed_scaling", C.c_float),
        ("router_weight_bits", C.c_uint32), ("round_route_weights_f16", C.c_uint32),
        ("has_shared", C.c_uint32), ("shared_gated", C.c_uint32), ("shared_f", C.c_uint32),
        ("max_tokens", C.c_uint32), ("y_dtype", C.c_uint32),
    ]


class ExpertOffsets(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in (
        "gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b",
        "down_w", "down_s", "down_b", "gate_ab", "up_ab", "down_ab")]


class RouterOperands(C.Structure):
    _fields_ = [
        ("weights", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p),
        ("effective_scale", C.c_void_p), ("per_expert_scale", C.c_void_p),
        ("logit_bias", C.c_void_p), ("shared_gate", C.c_void_p),
    ]


class SharedExpert(C.Structure):
    _fields_ = [("block", C.c_void_p), ("offsets", ExpertOffsets)]


class StackLayer(C.Structure):
    _fields_ = [("moe", C.c_void_p), ("pool", C.c_void_p), ("routed_offsets", C.POINTER(ExpertOffsets)),
                ("residency_table_row", C.c_void_p), ("router", C.POINTER(RouterOperands)),
                ("shared", C.POINTER(SharedExpert))]


_P = C.c_void_p
_U32, _U64, _INT = C.c_uint32, C.c_uint64, C.c_int

# name -> (restype, argtypes); every symbol include/shrike_b200.h declares
SIGNATURES = {
    "shrike_moe_create": (_INT, [C.POINTER(MoEConfig), _INT, C.POINTER(_P)]),
    "shrike_moe_destroy": (None, [_P]),
    "shrike_last_error": (C.c_char_p, [_P]),
    "shrike_moe_status": (_INT, [_P, _P]),
    "shrike_expert_offsets_make": (_INT, [C.POINTER(MoEConfig), _INT, C.POINTER(ExpertOffsets), C.POINTER(_U64)]),
    "shrike_pool_create": (_INT, [_P, _U32, _U64, _U32, C.POINTER(_P)]),
    "shrike_pool_destroy": (None, [_P]),
    "shrike_pool_upload": (_INT, [_P, _U32, _P, _U64, _P]),
    "shrike_pool_download": (_INT, [_P, _U32, _P, _U64, _P]),
    "shrike_pool_cell_address": (_INT, [_P, _U32, C.POINTER(_P)]),
    "shrike_pool_fill_synthetic": (_INT, [_P, _P, _U32, _U32, _U64, _U32, _U32, _INT, _P]),
    "shrike_residency_create": (_INT, [_P, _U32, C.POINTER(_P)]),
    "shrike_residency_set": (_INT, [_P, _U32, _U32, _U32, _U32, _P]),
    "shrike_residency_set_layer_identity": (_INT, [_P, _U32, _U32, _P]),
    "shrike_encode_router": (_INT, [_P, _P, C.POINTER(RouterOperands), _P, _U32, _U32, _P, _P, _P]),
    "shrike_encode_router_static": (_INT, [C.POINTER(MoEConfig), _P, C.POINTER(RouterOperands), _P, _U32, _U32, _P, _P,
                                           _P, C.c_char_p, C.c_size_t]),
    "shrike_encode_residency_classification": (_INT, [_P, _P, _P, _P, _U32, _P, _P, _P, _P]),
    "shrike_encode_decode_plan": (_INT, [_P, _P, _P, _P, _P, _U32, _P]),
    "shrike_encode_phase1": (_INT, [_P, _P, _P, C.POINTER(ExpertOffsets), C.POINTER(SharedExpert), _U32]),
    "shrike_encode_phase2_reduce": (_INT, [_P, _P, _P, C.POINTER(ExpertOffsets), _P, C.POINTER(SharedExpert), _P,
                                           _U32, _P, _P]),
    "shrike_encode_moe_decode": (_INT, [_P, _P, _P, C.POINTER(ExpertOffsets), _P, _P, _P, _U32,
                                        C.POINTER(SharedExpert), _P, _P, _P, _P]),
    "shrike_encode_route_decode": (_INT, [_P, _P, C.POINTER(RouterOperands), _P, _P, _P, _U32, _U32, _P, _P, _P, _P,
                                          _P, _P]),
    "shrike_encode_decode_layer": (_INT, [_P, _P, _P, C.POINTER(ExpertOffsets), _P, C.POINTER(RouterOperands),
                                          C.POINTER(SharedExpert), _P, _U32, _P, _P, _P, _P, _P]),
    "shrike_encode_moe_prefill": (_INT, [_P, _P, _P, C.POINTER(ExpertOffsets), _P, _P, _P, _P, _U32,
                                         C.POINTER(SharedExpert), _P, _P, _P]),
    "shrike_encode_group_pairs": (_INT, [_P, _P, _P, _P, _U32, _P, _P, _P]),
    "shrike_ep_encode_dispatch": (_INT, [_P, _P, _P, _P, _P, _U32, _U32, _U32, _U32, _P, _P, _P, _P, _P]),
    "shrike_ep_encode_local_slots": (_INT, [_P, _P, _P, _P, _U32, _P]),
    "shrike_ep_encode_combine": (_INT, [_P, _P, _P, _P, _P, _U32, _U32, _U32, _P, _P]),
    "shrike_ep_create": (_INT, [_P, _P, _U32, _U32, _U32, C.POINTER(_P)]),
    "shrike_ep_destroy": (None, [_P]),
    "shrike_ep_export": (_INT, [_P, _P]),
    "shrike_ep_connect": (_INT, [_P, _P]),
    "shrike_dequant_affine_rows": (_INT, [_P, _P, _P, _P, _U32, _U32, _U32, _U32, _U32, _P]),
    "shrike_ep_buffer": (_INT, [_P, C.POINTER(_P), C.POINTER(_U64)]),
    "shrike_ep_connect_pointers": (_INT, [_P, C.POINTER(_P)]),
    "shrike_ep_set_wait_polls": (_INT, [_P, _U32]),
    "shrike_ep_forward": (_INT, [_P, _P, _P, C.POINTER(ExpertOffsets), _P, C.POINTER(RouterOperands),
                                 C.POINTER(SharedExpert), _P, _U32, _P, _P]),
    "shrike_ep_status": (_INT, [_P, _P]),
    "shrike_ep_last_counts": (_INT, [_P, C.POINTER(_U32), C.POINTER(_U32), C.POINTER(_U64)]),
    "shrike_decode_stack_create": (_INT, [C.POINTER(StackLayer), _U32, _U32, C.POINTER(_P)]),
    "shrike_decode_stack_destroy": (None, [_P]),
    "shrike_decode_stack_forward_host": (_INT, [_P, _P, _P, _U32, _P]),
    "shrike_moe_layer_forward_host": (_INT, [_P, _P, _P, C.POINTER(ExpertOffsets), _P,
                                             C.POINTER(RouterOperands), C.POINTER(SharedExpert),
                                             _P, _U32, _P, _P, _P]),
}

_lib = None


def load() -> C.CDLL:
    """Loads libshrike_b200.so and binds every declared symbol (raises if any is missing)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise OSError(
            f"{LIB_PATH} is missing: build it with `python -m shrike_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
