"""Configuration and registry (no GPU).  Cases follow the reference's own unit tests
(tests/unit/config.test.ts:56-139): sizes, defaults, required keys."""
import json

import pytest

from binfer_b200.config import (ConfigError, Qwen3Config, load_config, parse_config,
                                register_architecture, registered_architectures)
import helpers as H


def test_parses_sizes_and_options():
    c = Qwen3Config.from_dict(H.TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.vocab_size) == (3, 96, 6, 1, 32, 160, 300)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings


def test_defaults_as_in_the_reference():
    c = Qwen3Config.from_dict(dict(architectures=["Qwen3ForCausalLM"], hidden_size=64,
                                   num_attention_heads=4, intermediate_size=128,
                                   num_hidden_layers=2, vocab_size=100))
    assert c.head_dim == 16 and c.num_key_value_heads == 4
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0
    assert c.max_position_embeddings == 4096 and c.tie_word_embeddings is False
    assert c.eos_token_id == (2,) and c.qk_norm


def test_camel_case_keys_are_accepted():
    c = Qwen3Config.from_dict(dict(architectures=["Qwen3ForCausalLM"], hiddenSize=64,
                                   numAttentionHeads=4, intermediateSize=128,
                                   numHiddenLayers=2, vocabSize=100, ropeTheta=5.0))
    assert c.hidden_size == 64 and c.rope_theta == 5.0


@pytest.mark.parametrize("key", ["hidden_size", "num_attention_heads", "intermediate_size",
                                 "num_hidden_layers", "vocab_size"])
def test_missing_required_key(key):
    raw = dict(H.TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=f"Missing required config key: {key}"):
        Qwen3Config.from_dict(raw)


@pytest.mark.parametrize("change,match", [
    (dict(num_key_value_heads=3), "multiple of"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(attention_bias=True), "attention_bias"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 4.0}), "rope_scaling"),
    (dict(head_dim=15), "head_dim"),
    (dict(layer_types=["full_attention"]), "layer_types"),
    (dict(use_sliding_window=True, sliding_window=None, max_window_layers=0), "sliding_window"),
])
def test_refuses_what_the_engine_cannot_do(change, match):
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict({**H.TINY_A, **change})


def test_windows_per_layer():
    c = Qwen3Config.from_dict(H.TINY_W)
    assert c.layer_windows() == [None, 24, 24, None]
    c2 = Qwen3Config.from_dict({**H.TINY_A, "use_sliding_window": True, "sliding_window": 8,
                                "max_window_layers": 1})
    assert c2.layer_windows() == [None, 8]
    c3 = Qwen3Config.from_dict({**H.TINY_A, "sliding_window": 8})     # not switched on
    assert c3.layer_windows() == [None, None]
    # layer_types that name sliding layers, but the switch is off: every layer attends fully
    c4 = Qwen3Config.from_dict({**H.TINY_W, "use_sliding_window": False})
    assert c4.layer_windows() == [None] * 4
    assert all(l.mixer.window is None for l in c4.to_spec().layers)
    import qwen3_plain as P
    assert P.read_config({**H.TINY_W, "use_sliding_window": False})["windows"] == [None] * 4
    assert P.read_config(H.TINY_W)["windows"] == [None, 24, 24, None]


def test_spec_is_chosen_layer_by_layer():
    spec = Qwen3Config.from_dict(H.TINY_W).to_spec()
    assert [l.mixer.window for l in spec.layers] == [None, 24, 24, None]
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    assert spec.layers[0].mixer.position.theta == 50000.0
    assert spec.layers[0].norm.eps == 3e-6 and spec.final_norm.eps == 3e-6


def test_round_trip_through_config_json(tmp_path):
    c = Qwen3Config.from_dict(H.TINY_W)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c


def test_registry():
    assert "Qwen3ForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError, match="registered"):
        parse_config({"architectures": ["NoSuchModel"]})
    register_architecture("ToyForTest", lambda raw: ("toy", raw["x"]))
    assert parse_config({"architectures": ["ToyForTest"], "x": 3}) == ("toy", 3)


def test_memory_arithmetic():
    c = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096,
        num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
        vocab_size=151936))
    assert c.kv_bytes_per_token(2) == 147456
    assert abs(c.num_parameters() - 8.19e9) < 0.01e9


def test_position_encoding_with_tensors_of_its_own_is_part_of_the_checkpoint():
    """A position encoding is chosen by its spec's kind like every part; one that names
    tensors adds them, under the mixer's prefix, to what a checkpoint must hold; an unknown
    kind is refused with the list of known ones.  (No GPU: only the list of tensors.)"""
    from dataclasses import dataclass

    from binfer_b200.config import (AttentionSpec, GatedMLPSpec, LayerSpec, ModelSpec, NameLayout,
                                    NormSpec, RopeSpec, ScheduleEntry)
    from binfer_b200.parts import PositionEncoding, param_specs_for, register_position
    from binfer_b200.weights import ParamSpec

    @dataclass(frozen=True)
    class TableSpec:
        kind: str = "test_cpu_position_table"
        entries: int = 5

    class Table(PositionEncoding):
        def __init__(self, spec, head_dim, env):
            self.spec, self.head_dim = spec, head_dim

        def param_specs(self, prefix):
            return [ParamSpec(prefix + "position_table.weight", (self.spec.entries, self.head_dim))]

    register_position("test_cpu_position_table", Table)
    norm = NormSpec(eps=1e-6)

    def model(position):
        attn = AttentionSpec(num_heads=2, num_kv_heads=1, head_dim=16, position=position)
        layers = (LayerSpec(mixer=attn, ffn=GatedMLPSpec(intermediate_size=24), norm=norm),)
        return ModelSpec(architecture="ToyForCausalLM", hidden_size=32, vocab_size=11, layers=layers,
                         schedule=(ScheduleEntry(0),), final_norm=norm, tie_word_embeddings=True,
                         names=NameLayout())

    specs = {s.name: s.shape for s in param_specs_for(model(TableSpec()))}
    assert specs["model.layers.0.self_attn.position_table.weight"] == (5, 16)
    plain = {s.name for s in param_specs_for(model(RopeSpec(theta=1e4)))}
    assert not any("position_table" in n for n in plain)
    assert set(specs) - plain == {"model.layers.0.self_attn.position_table.weight"}

    @dataclass(frozen=True)
    class Unknown:
        kind: str = "test_no_such_position"

    with pytest.raises(KeyError, match="position encoding.*test_no_such_position"):
        param_specs_for(model(Unknown()))
