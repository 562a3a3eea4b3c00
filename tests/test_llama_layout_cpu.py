"""Host-side facts of the Llama model description: the reference's 7B configuration
(benchmarks/train_llama7b_dp_pp_lowbit.py:222-231), its parameter count, and the split of
layers over pipeline stages (same rule as the reference, :127-131)."""

from bitscom_b200.models.llama import LlamaConfig, stage_layers


def test_llama7b_configuration_and_parameter_count():
    cfg = LlamaConfig.llama7b()
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size) == (32000, 4096, 11008)
    assert (cfg.num_layers, cfg.num_heads, cfg.head_dim) == (32, 32, 128)
    assert cfg.tie_embeddings and cfg.rope_theta == 1e4
    assert cfg.params_per_layer() == 4 * 4096 * 4096 + 3 * 4096 * 11008 + 2 * 4096
    # 6.61 G: 32 layers + one tied embedding + the final norm
    assert cfg.total_params() == 32 * cfg.params_per_layer() + 32000 * 4096 + 4096
    assert 6.6e9 < cfg.total_params() < 6.62e9


def test_stage_layers_cover_every_layer_once():
    assert [stage_layers(32, s, 4) for s in range(4)] == [(0, 8), (8, 16), (16, 24), (24, 32)]
    assert [stage_layers(5, s, 2) for s in range(2)] == [(0, 3), (3, 5)]
    for layers in (1, 5, 32, 33):
        for stages in (1, 2, 3, 4, 8):
            if stages > layers:
                continue
            ranges = [stage_layers(layers, s, stages) for s in range(stages)]
            assert ranges[0][0] == 0 and ranges[-1][1] == layers
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [hi - lo for lo, hi in ranges]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
