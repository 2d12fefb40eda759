"""Configuration and registry (CPU)."""
import json

import pytest

from llm_rs_b200.config import (ConfigError, Qwen3Config, architecture_names, load_config, resolve_architecture)
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_config_json():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim,
            c.intermediate_size, c.vocab_size) == (3, 96, 8, 2, 32, 224, 384)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and not c.tie_word_embeddings
    assert c.q_width == 256 and c.kv_width == 64 and c.eos_token_ids == (382, 383)


def test_defaults_follow_the_reference():
    c = Qwen3Config.from_dict(dict(vocab_size=10, hidden_size=32, num_hidden_layers=1, num_attention_heads=2,
                                   intermediate_size=8, architectures=["Qwen3ForCausalLM"]))
    assert c.num_key_value_heads == 2 and c.head_dim == 16
    assert c.max_position_embeddings == 2048 and c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-5
    assert c.tie_word_embeddings is False and c.eos_token_ids == (2,)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "intermediate_size"])
def test_required_keys(key):
    raw = dict(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=f"{key} missing from config"):
        Qwen3Config.from_dict(raw)


@pytest.mark.parametrize("patch,msg", [
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": "big"}, "integer"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
])
def test_refusals(patch, msg):
    with pytest.raises(ConfigError, match=msg):
        Qwen3Config.from_dict({**TINY_A, **patch})


def test_rope_parameters_object():
    """Newer files of the architecture keep the rotation's base inside ``rope_parameters`` and have no
    top-level ``rope_theta``; reading only the top-level key would rotate with the default 10000."""
    raw = {k: v for k, v in TINY_B.items() if k != "rope_theta"}
    raw["rope_parameters"] = {"rope_theta": 1000000.0, "rope_type": "default"}
    assert Qwen3Config.from_dict(raw).rope_theta == 1e6
    assert Qwen3Config.from_dict({**raw, "rope_theta": 1000000.0}).rope_theta == 1e6
    with pytest.raises(ConfigError, match="disagree"):
        Qwen3Config.from_dict({**raw, "rope_theta": 10000.0})
    with pytest.raises(ConfigError, match="rope_parameters"):
        Qwen3Config.from_dict({**raw, "rope_parameters": {"rope_theta": 1e6, "rope_type": "yarn", "factor": 4.0}})
    with pytest.raises(ConfigError, match="rope_parameters"):
        Qwen3Config.from_dict({**raw, "rope_parameters": "linear"})
    # rope_scaling with a base of its own is read the same way
    assert Qwen3Config.from_dict({**TINY_A, "rope_scaling": {"type": "default"}}).rope_theta == 10000.0


def test_end_token_absent_null_or_list():
    base = {k: v for k, v in TINY_A.items() if k != "eos_token_id"}
    assert Qwen3Config.from_dict(base).eos_token_ids == (2,)          # llm-core/src/backends/candle.rs:711-722
    none = Qwen3Config.from_dict({**base, "eos_token_id": None})
    assert none.eos_token_ids == ()
    assert Qwen3Config.from_dict(json.loads(json.dumps(none.to_dict()))) == none


def test_config_json_has_no_null_values():
    for raw in (TINY_A, TINY_B, TINY_C):
        d = Qwen3Config.from_dict(raw).to_dict()
        assert all(v is not None for v in d.values()), d


def test_window_layers_and_unrotated_layers():
    c = Qwen3Config.from_dict(TINY_C)
    assert c.layer_windows == (0, 0, 24, 24)
    assert c.no_rope_layers == (False, False, False, True)
    c2 = Qwen3Config.from_dict({**TINY_A, "sliding_window": 8,
                                "layer_types": ["sliding_attention", "full_attention"]})
    assert c2.layer_windows == (8, 0)


def test_round_trip_through_config_json():
    for raw in (TINY_A, TINY_B, TINY_C):
        c = Qwen3Config.from_dict(raw)
        assert Qwen3Config.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_registry_by_name(tmp_path):
    assert "Qwen3ForCausalLM" in architecture_names()
    assert resolve_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_cls is Qwen3Config
    assert resolve_architecture({"model_type": "qwen3"}).config_cls is Qwen3Config
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="failed to parse"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    entry, cfg = load_config(str(tmp_path))
    assert entry.name == "Qwen3ForCausalLM" and cfg.hidden_size == 64


def test_spec_has_no_architecture_constants():
    """The spec is data derived from the configuration: per-layer windows, positions, scopes."""
    from llm_rs_b200.models.qwen3 import build_spec
    spec = build_spec(Qwen3Config.from_dict(TINY_C))
    spec.validate()
    assert [l.mixer.params["window"] for l in spec.layers] == [0, 0, 24, 24]
    assert [l.mixer.params["position"].kind for l in spec.layers] == ["rope_half"] * 3 + ["none"]
    assert spec.layers[1].mixer.params["bias"] is True
    assert [s.layer for s in spec.run_order] == [0, 1, 2, 3]


def test_parts_take_their_tensor_names_from_the_spec():
    """The parts know roles; which tensor plays a role is the architecture's data. The same parts with another
    name map (and other scopes) ask the loader for other tensors."""
    import dataclasses
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel, PartSpec
    spec = build_spec(Qwen3Config.from_dict(TINY_A))
    names = {s.name for s in DecoderModel(spec).weight_specs()}
    assert "model.layers.0.self_attn.q_proj.weight" in names and "model.layers.1.mlp.down_proj.weight" in names
    other = []
    for l in spec.layers:
        mixer = PartSpec(l.mixer.kind, {**l.mixer.params, "names": {"q": "wq", "k": "wk", "v": "wv", "o": "wo",
                                                                    "q_norm": "qn", "k_norm": "kn"}})
        ffn = PartSpec(l.feed_forward.kind, {**l.feed_forward.params, "names": {"gate": "w1", "up": "w3", "down": "w2"}})
        other.append(dataclasses.replace(l, mixer=mixer, feed_forward=ffn, mixer_scope="attention.",
                                         feed_forward_scope="feed_forward.", prefix=l.prefix.replace("model.layers", "blocks")))
    renamed = dataclasses.replace(
        spec, layers=tuple(other),
        embedding=PartSpec("token_embedding", {**spec.embedding.params, "name": "tok.weight"}),
        lm_head=PartSpec("linear_head", {**spec.lm_head.params, "tied_to": "tok.weight"}))
    names = {s.name for s in DecoderModel(renamed).weight_specs() if s.load}
    assert {"tok.weight", "blocks.0.attention.wq.weight", "blocks.1.attention.qn.weight",
            "blocks.1.feed_forward.w2.weight"} <= names
    assert not any("q_proj" in n or "mlp" in n or "embed_tokens" in n for n in names)
    with pytest.raises(ValueError, match="names may rename"):
        DecoderModel(dataclasses.replace(spec, layers=(spec.layers[0], dataclasses.replace(spec.layers[1], mixer=PartSpec(
            "gqa_attention", {**spec.layers[1].mixer.params, "names": {"query": "x"}})))))


@pytest.mark.parametrize("head_dim", [8, 24, 272, 512])
def test_head_sizes_the_kernels_do_not_take_are_refused_when_the_model_is_built(head_dim):
    """Head sizes come in steps of 16 up to 256; anything else is refused with a clear error when the model is put
    together, not by a kernel at the first step."""
    from llm_rs_b200.models.qwen3 import build_spec
    from llm_rs_b200.parts import DecoderModel
    spec = build_spec(Qwen3Config.from_dict({**TINY_A, "head_dim": head_dim}))
    with pytest.raises(ValueError, match=f"head_dim {head_dim} is not supported"):
        DecoderModel(spec)
