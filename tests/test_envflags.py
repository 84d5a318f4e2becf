"""CPU tests of the environment switches (names and truth rules of the TriS-MoE reference:
qlinear_cuda.py:235-240, 269-283; modeling_olmoe.py:634-639; grouped_payload_sidecar.py:138-152)."""
import pytest
import torch


@pytest.fixture
def clean_env(monkeypatch):
    for name in ("TRIS_GROUPED_EXPERTS", "OLMOE_GROUPED_EXPERTS", "TRIS_DEPLOYMENT_ONLY", "OLMOE_DEPLOYMENT_ONLY",
                 "TRIS_COMPACT3_BLOCK_GR", "TRIS_GROUPED_QGMAP_CPU_STAGING", "OLMOE_GROUPED_QGMAP_CPU_STAGING",
                 "MIXTRAL_GROUPED_QGMAP_CPU_STAGING"):
        monkeypatch.delenv(name, raising=False)
    return monkeypatch


def test_defaults_and_truth_rules(lib, clean_env):
    from trismoe_b200 import envflags as ef

    assert ef.grouped_experts_enabled() and ef.compact3_block_gr_enabled()
    assert not ef.deployment_only_enabled() and not ef.grouped_qgmap_cpu_staging_enabled()
    for off in ("0", "false", "No", " OFF "):
        clean_env.setenv("TRIS_GROUPED_EXPERTS", off)
        clean_env.setenv("TRIS_COMPACT3_BLOCK_GR", off)
        assert not ef.grouped_experts_enabled() and not ef.compact3_block_gr_enabled()
    clean_env.setenv("TRIS_GROUPED_EXPERTS", "")          # set but empty: off for this flag ...
    clean_env.setenv("TRIS_COMPACT3_BLOCK_GR", "")        # ... default (on) for this one, as in the reference
    assert not ef.grouped_experts_enabled() and ef.compact3_block_gr_enabled()
    clean_env.setenv("OLMOE_GROUPED_EXPERTS", "1")        # the family-specific name is looked at first
    assert ef.grouped_experts_enabled()
    clean_env.setenv("TRIS_DEPLOYMENT_ONLY", "1")
    clean_env.setenv("TRIS_GROUPED_QGMAP_CPU_STAGING", "yes")
    assert ef.deployment_only_enabled() and ef.grouped_qgmap_cpu_staging_enabled()


def test_deployment_only_turns_none_into_an_error(lib, clean_env):
    from trismoe_b200 import envflags as ef

    assert ef.return_or_raise_none("label", "why") is None
    clean_env.setenv("TRIS_DEPLOYMENT_ONLY", "1")
    with pytest.raises(RuntimeError, match="deployment-only.*label.*why"):
        ef.return_or_raise_none("label", "why")


def test_block_gr_switch_selects_the_sparse_planes(lib, clean_env):
    from trismoe_b200 import qlinear_grouped as q, synth

    shape = synth.LayerShape(64, 96, 3, 2, rank=32, group_size=32)
    both = synth.synth_layer(shape, seed=1, keep_sparse_gmap=True)["gate"]
    gr_only = synth.synth_layer(shape, seed=1, keep_sparse_gmap=False)["gate"]
    assert q._use_block_gr(both) and q._use_block_gr(gr_only)
    clean_env.setenv("TRIS_COMPACT3_BLOCK_GR", "0")
    assert not q._use_block_gr(both)       # sparse planes are there: use them
    has_sparse = isinstance(gr_only.get("q_gmap_sparse"), torch.Tensor) and gr_only["q_gmap_sparse"].numel() > 0
    assert q._use_block_gr(gr_only) == (not has_sparse)  # nothing else to read: the streams stay
