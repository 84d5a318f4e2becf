"""Environment switches of the TriS-MoE runtime that this package honours, with the reference's
names and truth rules (values 0 / false / no / off / empty mean off):

``TRIS_GROUPED_EXPERTS`` (also ``OLMOE_GROUPED_EXPERTS``; ``modeling_olmoe.py:634-639``, default on)
    The reference switches between its grouped kernels and a per-expert Python loop.  There is no
    per-expert path here; off makes :class:`TrisSparseMoeBlock` compose the block from the individual
    grouped operators (``forward_grouped_ops``) instead of the single fused launch sequence.
``TRIS_DEPLOYMENT_ONLY`` (also ``OLMOE_DEPLOYMENT_ONLY``; ``qlinear_cuda.py:269-283``, default off)
    The grouped wrappers raise ``RuntimeError`` where they would return ``None`` ("kernel
    unavailable"), because a deployment-only checkpoint has nothing to fall back to.
``TRIS_COMPACT3_BLOCK_GR`` (``qlinear_cuda.py:235-240``, default on)
    One block Golomb-Rice policy for every payload: off keeps the sparse g_map planes as the
    format the kernels read, even when block-GR streams are present.
``TRIS_GROUPED_QGMAP_CPU_STAGING`` (also ``OLMOE_`` / ``MIXTRAL_``; ``grouped_payload_sidecar.py:147-152``,
    default off)  The host asks for the streaming mode (bitmaps paged from pinned host memory).
"""
from __future__ import annotations

import os

_OFF = {"0", "false", "no", "off", ""}


def _env_flag_enabled(*names: str, default: bool = False) -> bool:
    for name in names:
        value = os.environ.get(name)
        if value is None:
            continue
        return str(value).strip().lower() not in _OFF
    return default


def grouped_experts_enabled() -> bool:
    return _env_flag_enabled("OLMOE_GROUPED_EXPERTS", "TRIS_GROUPED_EXPERTS", default=True)


def deployment_only_enabled() -> bool:
    return _env_flag_enabled("OLMOE_DEPLOYMENT_ONLY", "TRIS_DEPLOYMENT_ONLY")


def compact3_block_gr_enabled() -> bool:
    value = os.environ.get("TRIS_COMPACT3_BLOCK_GR")
    if value is None or value == "":
        return True
    return str(value).strip().lower() not in {"0", "false", "no", "off"}


def grouped_qgmap_cpu_staging_enabled() -> bool:
    return _env_flag_enabled("MIXTRAL_GROUPED_QGMAP_CPU_STAGING", "OLMOE_GROUPED_QGMAP_CPU_STAGING",
                             "TRIS_GROUPED_QGMAP_CPU_STAGING")


def return_or_raise_none(label: str, reason: str):
    """``_return_or_raise_none`` (qlinear_cuda.py:279-283): ``None`` normally, an error when the
    process runs deployment-only."""
    if deployment_only_enabled():
        raise RuntimeError(f"[TriSMoE deployment-only] {label}: {reason}")
    return None
