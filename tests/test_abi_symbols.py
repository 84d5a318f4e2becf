"""CPU test: the shared library loads without a GPU and exports every symbol that
include/trismoe_b200.h declares; argument validation works without touching a device."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "trismoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tris_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    import trismoe_b200 as tm

    names = _declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert set(names) == set(tm._native.SIGNATURES), "ctypes table and header disagree"
    assert lib.tris_abi_version() == tm._native.ABI_VERSION == 4
    assert lib.tris_compact3_kernel_abi_version() == 2


def test_status_strings_and_host_validation(lib):
    import trismoe_b200 as tm

    assert lib.tris_status_string(0) == b"ok"
    assert b"corrupt" in lib.tris_status_string(4)
    # null pointers are rejected on the host, before any CUDA call
    st = lib.tris_grouped_forward(None, None, None, None, None)
    assert st == 1
    assert b"null" in lib.tris_last_error()
    view = tm._native.TrisProjView()
    st = lib.tris_block_gr_decode(C.byref(view), None, None)
    assert st == 1
    n = C.c_int64(0)
    st = lib.tris_block_gr_encode_host(None, 1, 1, 0, None, 0, None, None, C.byref(n))
    assert st == 1


def test_struct_sizes_match_c_layout(lib):
    """ctypes mirrors of the ABI structs: natural alignment, no packing surprises."""
    import trismoe_b200 as tm

    assert C.sizeof(tm._native.TrisProjView) == 224  # static_assert in csrc/common.cuh
    assert tm._native.TrisProjView.tile_records.offset == 184
    assert C.sizeof(tm._native.TrisRouteView) == 80
    assert C.sizeof(tm._native.TrisPacked4View) == 112
    assert tm._native.TrisRouteView.row_gather.offset == 40
    assert tm._native.TrisRouteView.out_row_scatter.offset == 64


def test_cpu_tensors_are_rejected_loudly(lib):
    import pytest
    import torch
    import trismoe_b200 as tm

    with pytest.raises(RuntimeError, match="CUDA"):
        tm.compute_shared_hidden(torch.zeros(2, 8, dtype=torch.float16), torch.zeros(4, 8, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="CUDA"):
        tm.build_grouped_route(torch.zeros(2, 2, dtype=torch.long), 4)
