"""trismoe_b200: B200 (sm_100a) grouped-expert dequant-GEMM runtime for TriS-MoE payloads.

The package mirrors the Python surface of the reference's grouped path
(``auto_gptq/nn_modules/qlinear/qlinear_cuda.py`` and
``auto_gptq/modeling_tris_moe`` in the TriS-MoE tree) on top of a C-ABI CUDA library
(``csrc/libtrismoe_b200.so``, declared in ``include/trismoe_b200.h``).  There is no CPU or
PyTorch fallback: every compute entry point raises if the library or a GPU is missing.
"""
from . import _native  # noqa: F401
from .formats import (  # noqa: F401
    block_gr_encode,
    build_compact3_packed_payload,
    dense_gmap_words,
    pack_bool_matrix,
    pack_bool_vector,
    pack_half4_words,
    stack_expert_payloads,
)
from .qlinear_grouped import (  # noqa: F401
    HIDDEN_LANE_ORDER,
    HIDDEN_PAIR_INTERLEAVED,
    HIDDEN_ROW_MAJOR,
    TRIS_COMPACT3_KERNEL_ABI_VERSION,
    ExpertSharedMatrix,
    build_grouped_precomputed_payload,
    build_grouped_route,
    compute_shared_hidden,
    decode_block_gr_gmap,
    dequantize_grouped_payload,
    dequantize_packed_4bit,
    prepare_grouped_payload,
    run_grouped_structured_expert_forward,
    run_grouped_structured_expert_pair_forward,
)
from .moe_block import TrisQwen2SparseMoeBlock, TrisSparseMoeBlock  # noqa: F401
from .compact3_linear import (  # noqa: F401
    Compact3Linear,
    run_compact3_gate_up_forward,
    run_compact3_qkv_forward,
)
from .ns_compensation import (  # noqa: F401
    Packed4Linear,
    build_grouped_ns_compensation_payload,
    run_grouped_ns_c1_forward,
    run_grouped_ns_compensation_forward,
)
from . import clocks, envflags, expert_parallel, synth  # noqa: F401

__all__ = [
    "Packed4Linear",
    "build_grouped_ns_compensation_payload",
    "run_grouped_ns_c1_forward",
    "run_grouped_ns_compensation_forward",
    "Compact3Linear",
    "run_compact3_gate_up_forward",
    "run_compact3_qkv_forward",
    "HIDDEN_LANE_ORDER",
    "HIDDEN_PAIR_INTERLEAVED",
    "HIDDEN_ROW_MAJOR",
    "TRIS_COMPACT3_KERNEL_ABI_VERSION",
    "ExpertSharedMatrix",
    "TrisQwen2SparseMoeBlock",
    "TrisSparseMoeBlock",
    "block_gr_encode",
    "build_compact3_packed_payload",
    "build_grouped_precomputed_payload",
    "build_grouped_route",
    "compute_shared_hidden",
    "decode_block_gr_gmap",
    "dense_gmap_words",
    "dequantize_grouped_payload",
    "dequantize_packed_4bit",
    "pack_bool_matrix",
    "pack_bool_vector",
    "pack_half4_words",
    "prepare_grouped_payload",
    "run_grouped_structured_expert_forward",
    "run_grouped_structured_expert_pair_forward",
    "stack_expert_payloads",
]
