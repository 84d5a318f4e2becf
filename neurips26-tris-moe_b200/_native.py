"""ctypes binding of ``csrc/libtrismoe_b200.so`` (the C ABI of ``include/trismoe_b200.h``).

Loading fails loudly: the library is the product, there is nothing to fall back to.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libtrismoe_b200.so")

TRIS_OK = 0
STATUS_NAMES = {
    0: "TRIS_OK", 1: "TRIS_ERR_INVALID_ARG", 2: "TRIS_ERR_UNSUPPORTED", 3: "TRIS_ERR_CUDA",
    4: "TRIS_ERR_CORRUPT", 5: "TRIS_ERR_WORKSPACE", 6: "TRIS_ERR_TIMEOUT",
}

_vp = C.c_void_p
_i32 = C.c_int32


class TrisProjView(C.Structure):
    _fields_ = [
        ("num_experts", _i32), ("out_features", _i32), ("rank", _i32), ("num_groups", _i32),
        ("sign2_rows", _i32), ("gmap_sparse_rows", _i32), ("gr_max_words", _i32), ("use_block_gr", _i32),
        ("qweight1", _vp), ("qweight2_sparse", _vp), ("qweight2_sparse_prefix", _vp),
        ("q_gmap_sparse", _vp), ("q_gmap_sparse_prefix", _vp),
        ("q_gmap_gr_words", _vp), ("q_gmap_gr_offsets", _vp), ("q_gmap_gr_meta", _vp),
        ("c_map", _vp), ("g_idx", _vp), ("col_pack3", _vp), ("row_pack3", _vp),
        ("output_scale", _vp), ("bias", _vp),
        ("gr_index", _vp), ("gr_substreams", _i32), ("packed_row_group", _vp), ("gmap_slot", _vp), ("expert_slot", _vp),
        ("tile_records", _vp), ("tile_desc", _vp), ("col_records", _vp),
        ("col_record_bytes", _i32), ("max_record_bytes", _i32), ("max_sal_words", _i32), ("reserved0", _i32),
    ]


class TrisPageJob(C.Structure):
    _fields_ = [("host_src", _vp), ("dst", _vp), ("bytes_per_expert", C.c_int64)]


ABI_VERSION = 4  # TRIS_B200_ABI_VERSION of include/trismoe_b200.h


class TrisRouteView(C.Structure):
    _fields_ = [
        ("expert_ids", _vp), ("segment_offsets", _vp), ("num_segments_dev", _vp),
        ("num_segments", _i32), ("num_rows", _i32), ("max_rows_per_segment", _i32),
        ("row_gather", _vp), ("status_dev", _vp), ("flags", _i32), ("hidden_row_stride", _i32),
        ("out_row_scatter", _vp), ("hidden_col_scale", _vp),
    ]


class TrisPacked4View(C.Structure):
    _fields_ = [
        ("qweight", _vp), ("qzeros", _vp), ("scales", _vp),
        ("n_off", _vp), ("z_off", _vp), ("kw_off", _vp), ("g_off", _vp),
        ("n_count", _vp), ("k_count", _vp), ("g_count", _vp),
        ("q_ld", _i32), ("z_ld", _i32), ("s_ld", _i32),
        ("n", _i32), ("k", _i32), ("num_groups", _i32), ("group_size", _i32), ("num_experts", _i32),
    ]


class TrisMoeLayerView(C.Structure):
    _fields_ = [
        ("hidden_size", _i32), ("intermediate_size", _i32), ("num_experts", _i32), ("top_k", _i32),
        ("norm_topk_prob", _i32),
        ("router_weight", _vp), ("shared_gate", _vp), ("shared_up", _vp), ("shared_down", _vp),
        ("gate", TrisProjView), ("up", TrisProjView), ("down", TrisProjView),
        ("packed_gate", _vp), ("packed_up", _vp), ("packed_down", _vp),
    ]


# name -> (restype, argtypes); also the list of symbols include/trismoe_b200.h declares.
_P = C.POINTER
SIGNATURES = {
    "tris_abi_version": (C.c_int, []),
    "tris_compact3_kernel_abi_version": (C.c_int, []),
    "tris_status_string": (C.c_char_p, [C.c_int]),
    "tris_last_error": (C.c_char_p, []),
    "tris_set_programmatic_launch": (C.c_int, [_i32]),
    "tris_block_gr_encode_host": (C.c_int, [_vp, _i32, _i32, _i32, _vp, C.c_int64, _vp, _vp, _P(C.c_int64)]),
    "tris_block_gr_encode_host_k": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _i32, _vp, C.c_int64, _vp, _vp, _P(C.c_int64)]),
    "tris_block_gr_index_bytes": (C.c_size_t, [_i32, _i32, _i32, _i32]),
    "tris_block_gr_build_index": (C.c_int, [_P(TrisProjView), _vp, _i32, _vp, _vp]),
    "tris_block_gr_decode": (C.c_int, [_P(TrisProjView), _vp, _vp]),
    "tris_build_row_groups": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _vp, _vp]),
    "tris_compact3_dequantize": (C.c_int, [_P(TrisProjView), _vp, _vp]),
    "tris_tile_record_count": (C.c_int64, [_P(TrisProjView)]),
    "tris_col_record_bytes": (C.c_int64, [_P(TrisProjView), _i32]),
    "tris_tile_records_plan": (C.c_int, [_P(TrisProjView), _vp, _vp, _vp]),
    "tris_tile_records_build": (C.c_int, [_P(TrisProjView), _vp, _vp, _vp, _i32, _vp]),
    "tris_build_grouped_route": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tris_build_grouped_route_ex": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "tris_ep_pack_rows": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp]),
    "tris_ep_signal_increment": (C.c_int, []),
    "tris_ep_enable_peer_access": (C.c_int, [_i32]),
    "tris_ep_open_peer_memory": (C.c_int, [_vp, _P(_vp)]),
    "tris_ep_close_peer_memory": (C.c_int, [_vp]),
    "tris_ep_dispatch_peer": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp]),
    "tris_ep_return_peer": (C.c_int, [_vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "tris_ep_wait": (C.c_int, [_vp, _vp, _i32, _vp, _vp]),
    "tris_router_topk": (C.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "tris_input_projections": (C.c_int, [_vp, _i32, _i32, _vp, _vp, _i32, _vp, _i32, _vp, _vp, _i32, _vp, _vp]),
    "tris_packed4_dequantize": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "tris_packed4_grouped_forward": (C.c_int, [_P(TrisPacked4View), _P(TrisRouteView), _vp, _i32, _i32, _vp, _i32, _i32, _i32, _vp]),
    "tris_shared_hidden_forward": (C.c_int, [_vp, _vp, _i32, _vp, _i32, _vp, _i32, _vp, _i32, _vp]),
    "tris_grouped_forward": (C.c_int, [_P(TrisProjView), _P(TrisRouteView), _vp, _vp, _vp]),
    "tris_grouped_pair_forward": (C.c_int, [_P(TrisProjView), _P(TrisProjView), _P(TrisRouteView), _vp, _vp, _vp, _vp, _i32, _vp]),
    "tris_grouped_hidden_layout": (C.c_int, [_P(TrisProjView), _P(TrisProjView), _i32, _i32, _i32]),
    "tris_set_grouped_tc_min_rows": (C.c_int, [_i32]),
    "tris_set_grouped_row_split_max": (C.c_int, [_i32]),
    "tris_combine_routed": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _vp, _vp]),
    "tris_page_experts": (C.c_int, [_vp, _i32, _vp, _vp, _i32, _i32, _vp, _vp]),
    "tris_moe_layer_workspace_bytes": (C.c_size_t, [_P(TrisMoeLayerView), _i32]),
    "tris_moe_layer_last_status": (C.c_int, [_vp, _i32, _vp, _P(_i32)]),
    "tris_moe_layer_forward": (C.c_int, [_P(TrisMoeLayerView), _vp, _vp, _i32, _vp, _vp, _vp, C.c_size_t, _vp]),
    "tris_moe_layer_forward_static": (C.c_int, [_P(TrisMoeLayerView), _vp, _vp, _i32, _vp, _vp, _vp]),
}
STATIC_SCRATCH_BYTES = 8 << 20

_lib = None


def load():
    """Returns the loaded library, raising RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
            "(the trismoe_b200 kernels have no CPU or PyTorch fallback)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the header and the library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.tris_compact3_kernel_abi_version() != 2:
        raise RuntimeError("trismoe_b200: compact3 payload ABI mismatch")
    if lib.tris_abi_version() != ABI_VERSION:
        raise RuntimeError(f"trismoe_b200: the library has struct/entry-point ABI {lib.tris_abi_version()}, this "
                           f"package was written for {ABI_VERSION}; rebuild it (python build.py --force)")
    _lib = lib
    return lib


def check(status: int, what: str = "") -> None:
    """Raises RuntimeError for a non-zero status (the TORCH_CHECK of the reference extension)."""
    if status == TRIS_OK:
        return
    lib = load()
    msg = lib.tris_last_error().decode("utf-8", "replace")
    name = STATUS_NAMES.get(status, str(status))
    raise RuntimeError(f"trismoe_b200 {what} failed with {name}: {msg}")


def require_cuda(tensor, what: str) -> None:
    if tensor.device.type != "cuda":
        raise RuntimeError(f"trismoe_b200 {what}: tensors must live on a CUDA device (no CPU path exists)")
