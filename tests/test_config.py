"""Configuration and registry (no GPU)."""
import json

import pytest

from gemmars_b200.config import ConfigError, known_architectures, load_config, load_stop_ids, resolve_architecture
from gemmars_b200.models.qwen3 import Qwen3Config, build_plan
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_key_of_both_tiny_configs():
    a, b = Qwen3Config.from_dict(TINY_A), Qwen3Config.from_dict(TINY_B)
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads) == (2, 64, 4, 2)
    assert (a.dim_per_head, a.intermediate_size, a.vocab_size) == (16, 192, 512)
    assert a.rope_theta == 10000.0 and a.rms_norm_eps == 1e-6 and a.tie_word_embeddings and not a.attention_bias
    assert a.eos_token_id == [7] and a.max_position_embeddings == 256 and a.layer_window(0) is None
    assert (b.num_hidden_layers, b.hidden_size, b.dim_per_head) == (3, 96, 32)
    assert b.attention_bias and not b.tie_word_embeddings and b.eos_token_id == [3, 11]
    assert [b.layer_window(i) for i in range(3)] == [40, None, 40]
    for x, y in zip(TINY_A.items(), TINY_B.items()):
        if x[0] in ("architectures", "model_type"):
            continue
        assert x[1] != y[1], f"the tiny configurations share {x[0]}"


def test_defaults_and_head_dim():
    raw = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "rope_theta", "rms_norm_eps", "eos_token_id")}
    c = Qwen3Config.from_dict(raw)
    assert c.dim_per_head == 64 // 4          # hidden / heads when absent
    assert c.rope_theta == 10_000_000.0       # the reference's value when absent
    assert c.rms_norm_eps == 1e-6 and c.eos_token_id == []
    assert Qwen3Config.from_dict(TINY_C).rotary_dim == 24


def test_rope_parameters_and_text_config():
    raw = dict(TINY_A, rope_parameters={"rope_theta": 5e5, "partial_rotary_factor": 0.5})
    c = Qwen3Config.from_dict(raw)
    assert c.rope_theta == 5e5 and c.rotary_dim == 8
    nested = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "text_config": dict(TINY_B)}
    assert Qwen3Config.from_dict(nested).hidden_size == 96


def test_errors_name_every_key():
    raw = dict(TINY_A)
    del raw["vocab_size"]
    raw["hidden_size"] = "64"
    raw["tie_word_embeddings"] = 1
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    msg = str(e.value)
    assert "vocab_size: missing" in msg and "hidden_size" in msg and "tie_word_embeddings" in msg


@pytest.mark.parametrize("patch, word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"num_hidden_layers": 0}, "positive"),
    ({"partial_rotary_factor": 0.2}, "even"),
    ({"use_sliding_window": True}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "length mismatch"),
    ({"layer_types": ["full_attention", "linear_attention"]}, "unknown layer type"),
    # options that change the logits and have no implementation are refused, with the key named
    ({"use_sliding_window": True, "sliding_window": 8}, "layer_types is absent"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"rope_parameters": {"rope_theta": 1e6, "rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rope_scaling": 4}, "rope_scaling"),
])
def test_validation(patch, word):
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(dict(TINY_A, **patch))
    assert word in str(e.value)


def test_null_and_default_rope_scaling_are_accepted():
    for v in (None, {"rope_type": "default"}, {"type": "default"}):
        assert Qwen3Config.from_dict(dict(TINY_A, rope_scaling=v)).rope_theta == TINY_A["rope_theta"]
    ok = Qwen3Config.from_dict(dict(TINY_A, rope_parameters={"rope_theta": 5e5, "rope_type": "default"}))
    assert ok.rope_theta == 5e5 and ok.rope_scaling is None


def test_registry():
    assert {"Qwen3ForCausalLM", "qwen3"} <= set(known_architectures())
    assert resolve_architecture({"model_type": "qwen3"}).config_class is Qwen3Config
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_class is Qwen3Config
    with pytest.raises(ConfigError) as e:
        resolve_architecture({"architectures": ["GemmaForCausalLM"], "model_type": "gemma"})
    assert "unsupported architecture 'gemma'" in str(e.value) and "qwen3" in str(e.value)
    with pytest.raises(ConfigError):
        resolve_architecture({})


def test_load_config_and_stop_ids(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Qwen3ForCausalLM" and cfg.vocab_size == 1000
    assert load_stop_ids(str(tmp_path)) == [3, 11]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 5}))
    assert load_stop_ids(str(tmp_path)) == [5]          # generation_config.json first
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nothing"))


def test_plan_is_data():
    cfg = Qwen3Config.from_dict(TINY_B)
    plan = build_plan(cfg)
    assert len(plan.layers) == 3 and [e.layer for e in plan.schedule] == [0, 1, 2]
    assert plan.layers[0].block == "prenorm" and set(plan.layers[0].parts) == {"mixer_norm", "mixer", "ffn_norm", "ffn"}
    m = plan.layers[0].parts["mixer"]
    assert m.kind == "attention" and m.params["window"] == 40 and plan.layers[1].parts["mixer"].params["window"] is None
    assert m.params["num_heads"] == 6 and m.params["num_kv_heads"] == 3 and m.params["head_dim"] == 32
    assert m.params["position"].kind == "rotary" and m.params["position"].params["theta"] == 1e6
    assert m.tensors["q_bias"] == "model.layers.0.self_attn.q_proj.bias"
    assert plan.head.tensors["weight"] == "lm_head.weight"
    tied = build_plan(Qwen3Config.from_dict(TINY_A))
    assert tied.head.tensors["weight"] == "model.embed_tokens.weight"
    # a checkpoint without a head is tied too, and another prefix is found by probing
    names = {"model.language_model.embed_tokens.weight"}
    p2 = build_plan(cfg, names)
    assert p2.head.tensors["weight"] == "model.language_model.embed_tokens.weight"
    assert p2.layers[2].parts["ffn"].tensors["down"] == "model.language_model.layers.2.mlp.down_proj.weight"


def test_schedule_validation():
    from gemmars_b200.parts.plan import ScheduleEntry
    plan = build_plan(Qwen3Config.from_dict(TINY_A))
    plan.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1)]
    plan.validate()
    plan.schedule = [ScheduleEntry(0, cache_of=1), ScheduleEntry(1)]
    with pytest.raises(ValueError):
        plan.validate()
    plan.schedule = [ScheduleEntry(5)]
    with pytest.raises(ValueError):
        plan.validate()


def test_measurement_shapes_are_configurations():
    """The layer sizes the measurements are taken at read as configurations of the architecture."""
    from gemmars_b200.tuning import SHAPES, main
    for name, (label, raw) in SHAPES.items():
        cfg = Qwen3Config.from_dict(raw)
        assert cfg.dim_per_head == 128 and label.startswith("Qwen3-")
    assert SHAPES["4b"][1]["tie_word_embeddings"] and not SHAPES["32b"][1]["tie_word_embeddings"]
    with pytest.raises(SystemExit):
        main(["no-such-command"])
