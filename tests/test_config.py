"""Configuration and registry (CPU)."""
import json

import pytest

from helpers import TINY_A, TINY_B
from tq_kv_b200.config import (Architecture, ConfigError, ModelSpec, Qwen2Config, named_shape, read_config_json,
                               register_architecture, registered_architectures, resolve, shape_names,
                               spec_from_config_dict, unregister_architecture)


def test_typed_fields_and_defaults():
    c = Qwen2Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 96, 3, 1)
    assert c.head_dim == 32 and c.intermediate_size == 200 and c.vocab_size == 1000
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings
    d = dict(TINY_A)
    del d["head_dim"], d["num_key_value_heads"]
    c = Qwen2Config.from_dict(d)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4      # defaults follow the reference


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size",
                                 "intermediate_size", "rms_norm_eps", "rope_theta", "max_position_embeddings"])
def test_missing_key_is_an_error(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


def test_wrong_type_and_inconsistent_sizes():
    with pytest.raises(ConfigError, match="hidden_size"):
        Qwen2Config.from_dict({**TINY_A, "hidden_size": "64"})
    with pytest.raises(ConfigError, match="multiple"):
        Qwen2Config.from_dict({**TINY_A, "num_key_value_heads": 3})
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict({**TINY_A, "use_sliding_window": True, "sliding_window": None})
    with pytest.raises(ConfigError, match="hidden_act"):
        Qwen2Config.from_dict({**TINY_A, "hidden_act": "gelu"})


def test_window_rule():
    c = Qwen2Config.from_dict(TINY_B)
    assert [c.layer_window(i) for i in range(3)] == [None, 16, 16]
    c = Qwen2Config.from_dict(TINY_A)
    assert [c.layer_window(i) for i in range(2)] == [None, None]


def test_round_trip_through_json(tmp_path):
    c = Qwen2Config.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert Qwen2Config.from_dict(read_config_json(str(tmp_path))) == c
    with pytest.raises(ConfigError, match="Cannot read config.json"):
        read_config_json(str(tmp_path / "nope"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="Invalid config.json"):
        read_config_json(str(tmp_path))


def test_registry_resolves_by_name_and_lists_known_names():
    assert "Qwen2ForCausalLM" in registered_architectures()
    assert resolve(TINY_A).name == "Qwen2ForCausalLM"
    assert resolve({"model_type": "qwen2"}).name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        resolve({"architectures": ["NoSuchModel"]})


def test_another_architecture_registers_without_touching_the_package():
    class ToyConfig:
        @classmethod
        def from_dict(cls, d):
            return Qwen2Config.from_dict({**TINY_A, "num_hidden_layers": d["depth"]})

    def build(cfg):
        from tq_kv_b200.config import build_qwen2_spec
        return build_qwen2_spec(cfg)

    register_architecture(Architecture("ToyForCausalLM", "toy", ToyConfig, build))
    try:
        arch, cfg, spec = spec_from_config_dict({"architectures": ["ToyForCausalLM"], "depth": 5})
        assert arch.name == "ToyForCausalLM" and len(spec.layers) == 5
    finally:
        unregister_architecture("ToyForCausalLM")


def test_spec_is_parts_chosen_layer_by_layer():
    _, _, spec = spec_from_config_dict(TINY_B)
    assert isinstance(spec, ModelSpec) and len(spec.layers) == 3 and len(spec.schedule) == 3
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 16, 16]
    assert spec.layers[0].mixer.kind == "gqa_attention" and spec.layers[0].feed_forward.kind == "swiglu"
    assert spec.head.params["tied_to"] is None
    _, _, spec_a = spec_from_config_dict(TINY_A)
    assert spec_a.head.params["tied_to"] == "model.embed_tokens.weight"


def test_schedule_validation():
    from dataclasses import replace
    from tq_kv_b200.config import ScheduleEntry
    _, _, spec = spec_from_config_dict(TINY_A)
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_of=1))).validate()
    with pytest.raises(ConfigError):
        replace(spec, schedule=(ScheduleEntry(0, cache_of=0),)).validate()
    with pytest.raises(ConfigError):
        replace(spec, schedule=(ScheduleEntry(7),)).validate()


def test_named_shapes_are_valid_configs():
    assert {"tiny-a", "tiny-b", "qwen2.5-7b", "qwen2.5-0.5b", "qwen2.5-32b"} <= set(shape_names())
    for n in shape_names():
        Qwen2Config.from_dict(named_shape(n))
    with pytest.raises(KeyError):
        named_shape("nope")


def test_head_sizes_the_kernels_do_not_take_are_refused_where_the_config_is_read():
    from helpers import TINY_A
    from tq_kv_b200.config import ConfigError, Qwen2Config
    for hd in (8, 24, 40, 272):
        with pytest.raises(ConfigError, match="head_dim"):
            Qwen2Config.from_dict({**TINY_A, "head_dim": hd})
    for hd in (16, 48, 112, 256):
        assert Qwen2Config.from_dict({**TINY_A, "head_dim": hd}).head_dim == hd


def test_a_layer_names_its_parts_and_a_missing_one_is_named_in_the_error():
    from dataclasses import replace
    from helpers import TINY_A
    from tq_kv_b200.config import ConfigError, PartSpec, Qwen2Config, build_qwen2_spec
    layer = build_qwen2_spec(Qwen2Config.from_dict(TINY_A)).layers[0]
    assert list(layer.parts()) == ["mixer_norm", "mixer", "feed_forward_norm", "feed_forward"]
    more = replace(layer, extra_parts={"after": PartSpec("rms_norm", {"width": 64, "eps": 1e-6}, "x.")})
    assert more.part("after").weights_prefix == "x." and len(more.parts()) == 5
    with pytest.raises(ConfigError, match="needs a part named 'gate'"):
        layer.part("gate")
    with pytest.raises(ConfigError, match="twice"):
        replace(layer, extra_parts={"mixer": layer.mixer}).parts()
