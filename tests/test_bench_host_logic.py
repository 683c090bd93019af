"""Host-side arithmetic of bench.py: the byte and operation counts the rooflines divide by, and the choice of how many
steps one graph launch replays.  No GPU is touched."""
import argparse

import bench


def cfg(config_id):
    return dict(bench.CONFIGS[config_id])


def test_algorithmic_bytes_of_the_non_fused_pipeline():
    c = cfg(2)
    sb = bench.stage_bytes(c, "float16")
    tiles = 64 * 14 * 14
    assert sb["input_transform"] == 64 * 56 * 56 * 64 * 2 + 36 * tiles * 64 * 2
    assert sb["gemm"] == 2 * 36 * tiles * 64 * 2 + 36 * 64 * 64 * 2
    assert sb["output_transform"] == 36 * tiles * 64 * 2 + 64 * 56 * 56 * 64 * 2
    assert sb["weight_input_transform"] == sb["weight_transform"] + sb["input_transform"]
    total = bench.algorithmic_bytes(c, "float16", 0)
    assert total == sb["weight_transform"] + sb["input_transform"] + sb["gemm"] + sb["output_transform"]
    # with the contraction and the output transform as one kernel the products are neither written nor read back
    assert total - bench.algorithmic_bytes(c, "float16", 2) == 2 * 36 * tiles * 64 * 2
    # float32 transform-domain tensors double every transform-domain term
    sb32 = bench.stage_bytes(c, "float32")
    assert sb32["gemm"] == 2 * sb["gemm"]


def test_operation_counts():
    assert bench.direct_flops(cfg(2)) == 2.0 * 64 * 56 * 56 * 64 * 64 * 9
    assert bench.direct_flops(cfg(4)) == 2.0 * 256 * 14 * 14 * 256 * 256 * 9
    # a training step is the forward pass and its two adjoints
    assert bench.direct_flops(cfg(5)) == 3 * 2.0 * 256 * 56 * 56 * 64 * 64 * 9
    # the comparison records run the layers of cfg 2 and cfg 3
    for layer, base in ((12, 2), (13, 3)):
        assert bench.direct_flops(cfg(layer)) == bench.direct_flops(cfg(base))
        assert all(cfg(layer)[key] == cfg(base)[key] for key in ("n", "h", "w", "c", "k", "dtype"))


def test_fully_fused_byte_counts_are_input_plus_output():
    c = cfg(3)
    assert bench.algorithmic_bytes(c, None) == 2 * 128 * 28 * 28 * 128 * 2 + 9 * 128 * 128 * 2 + 4 * 128
    assert bench.moved_bytes_fused_winograd(c) > 4 * bench.algorithmic_bytes(c, None)
    c = cfg(4)
    assert bench.algorithmic_bytes(c, None) == 2 * 256 * 14 * 14 * 256 + 9 * 256 * 256 + 8 * 256


def test_steps_per_graph_keeps_the_step_count_exact():
    def args(**kw):
        base = dict(no_graph=False, steps_per_graph=0, rotation=4, steps=2000)
        base.update(kw)
        return argparse.Namespace(**base)
    assert bench.headline_steps_per_graph(args()) == 4
    assert bench.headline_steps_per_graph(args(steps=20)) == 4
    assert bench.headline_steps_per_graph(args(steps=21)) == 1          # 21 steps cannot be made of graphs of four
    assert bench.headline_steps_per_graph(args(steps_per_graph=1)) == 1  # asked for
    assert bench.headline_steps_per_graph(args(steps_per_graph=3)) == 4  # neither 1 nor the rotation: the default rule
    assert bench.headline_steps_per_graph(args(no_graph=True)) == 1


def test_ncu_traffic_table_names_existing_configurations():
    for (config_id, dtype, fused) in bench.NCU_TRAFFIC:
        assert config_id in bench.CONFIGS and isinstance(fused, bool)
        assert dtype in ("float16", "bfloat16", "float32", "int8")
        assert bench.NCU_TRAFFIC[(config_id, dtype, fused)] > 0
