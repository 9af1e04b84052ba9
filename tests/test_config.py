"""Configuration and registry (no GPU)."""
import pytest

from gibbs_b200.config import ConfigError, Lfm2Config, detect, known_architectures, parse_config
from helpers import TINY_A, TINY_B


def base(**over):
    d = dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8,
             vocab_size=65536, intermediate_size=12288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
             block_multiple_of=256, conv_L_cache=3, full_attn_idxs=[2, 5, 8, 10, 12, 14], norm_eps=1e-5,
             rope_theta=1000000.0, architectures=["Lfm2ForCausalLM"])
    d.update(over)
    return d


def test_feed_forward_width_rule():
    # arch/families/lfm2.json5:36-40
    assert Lfm2Config.from_dict(base()).ffn_dim == 8192
    assert Lfm2Config.from_dict(base(hidden_size=1536, num_attention_heads=24, intermediate_size=10240)).ffn_dim == 6912
    assert Lfm2Config.from_dict(base(intermediate_size=10752)).ffn_dim == 7168
    assert Lfm2Config.from_dict(TINY_B).ffn_dim == 256
    assert Lfm2Config.from_dict(base(block_auto_adjust_ff_dim=False)).ffn_dim == 12288
    assert Lfm2Config.from_dict(base(block_ffn_dim_multiplier=0)).ffn_dim == 12288 * 2 // 3
    cfg = base()
    del cfg["intermediate_size"]
    cfg["block_ff_dim"] = 6000
    assert Lfm2Config.from_dict(cfg).intermediate_size == 6000
    del cfg["block_ff_dim"]
    assert Lfm2Config.from_dict(cfg).intermediate_size == 4 * 2048


def test_defaults_and_aliases():
    c = Lfm2Config.from_dict(base())
    assert c.head_dim == 64 and c.attention_layers == (2, 5, 8, 10, 12, 14) and len(c.conv_layers) == 10
    assert c.max_position_embeddings == 2048 and not c.conv_bias and not c.attention_bias
    cfg = base(num_heads=16, rms_norm_eps=1e-6, rope_parameters={"rope_theta": 5e5}, tie_word_embeddings=False)
    for k in ("num_attention_heads", "norm_eps", "rope_theta", "num_key_value_heads"):
        del cfg[k]
    c = Lfm2Config.from_dict(cfg)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (16, 16, 128)
    assert c.norm_eps == 1e-6 and c.rope_theta == 5e5 and c.tie_embedding is False
    assert Lfm2Config.from_dict(base(norm_eps=3e-6, rms_norm_eps=1e-6)).norm_eps == 3e-6


def test_layer_kinds_from_tensor_names_when_config_is_silent():
    cfg = base(num_hidden_layers=3)
    del cfg["full_attn_idxs"]
    with pytest.raises(ConfigError, match="layer_types"):
        Lfm2Config.from_dict(cfg)
    names = ["model.layers.0.conv.in_proj.weight", "model.layers.2.conv.in_proj.weight", "lm_head.weight",
             "model.layers.1.self_attn.q_proj.bias"]
    c = Lfm2Config.from_dict(cfg, names)
    assert c.layer_types == ("conv", "full_attention", "conv")
    assert c.tie_embedding is False and c.attention_bias is True and c.conv_bias is False


@pytest.mark.parametrize("over,msg", [
    (dict(conv_L_cache=1), "conv_L_cache"),
    (dict(num_key_value_heads=5), "multiple"),
    (dict(head_dim=63), "even"),
    (dict(layer_types=["conv"] * 3), "layer_types"),
    (dict(layer_types=["conv"] * 15 + ["mamba"]), "unknown layer_types"),
    (dict(full_attn_idxs=[99]), "full_attn_idxs"),
    (dict(norm_eps=0.0), "norm_eps"),
])
def test_refusals(over, msg):
    cfg = base(**over)
    if "layer_types" in over:
        del cfg["full_attn_idxs"]
    with pytest.raises(ConfigError, match=msg):
        Lfm2Config.from_dict(cfg)


def test_missing_required_key():
    for key in ("hidden_size", "num_hidden_layers", "conv_L_cache", "vocab_size"):
        cfg = base()
        del cfg[key]
        with pytest.raises(ConfigError, match=key):
            Lfm2Config.from_dict(cfg)


def test_round_trip_through_config_json():
    for raw in (TINY_A, TINY_B, base()):
        c = Lfm2Config.from_dict(raw)
        assert Lfm2Config.from_dict(c.to_dict()) == c


def test_registry():
    assert "Lfm2ForCausalLM" in known_architectures()
    assert detect({"architectures": ["Lfm2ForCausalLM"]}).name == "Lfm2ForCausalLM"
    assert detect({"model_type": "lfm2"}).name == "Lfm2ForCausalLM"
    assert detect({"architectures": ["Nope"]}, forced="lfm2").name == "Lfm2ForCausalLM"
    with pytest.raises(KeyError, match="known"):
        detect({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    assert isinstance(parse_config(TINY_A), Lfm2Config)


def test_plan_is_data():
    plan = Lfm2Config.from_dict(TINY_B).plan()
    kinds = [l.mixer.kind for l in plan.layers]
    assert kinds == ["gqa_attention", "gated_short_conv", "gqa_attention", "gated_short_conv", "gated_short_conv",
                     "gqa_attention"]
    assert [e.layer for e in plan.order] == list(range(6))
    assert plan.head.tensors["weight"] == "lm_head.weight"
    assert Lfm2Config.from_dict(TINY_A).plan().head.tensors["weight"] == "model.embed_tokens.weight"
    att = plan.layers[0].mixer
    assert att.params["heads"] == 3 and att.params["kv_heads"] == 1 and att.params["head_dim"] == 32
    assert att.tensors["q_norm.weight"] == "model.layers.0.self_attn.q_layernorm.weight"
    assert "q_proj.bias" in att.tensors and "conv.bias" in plan.layers[1].mixer.tensors
