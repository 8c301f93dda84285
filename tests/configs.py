"""Tiny LFM2 configurations of the tests.  They differ in every size and option."""

# 4 layers [conv, attn, conv, attn], hidden 64, 4 heads / 2 kv heads, head 16, ff 128 given
# directly, vocab 256, 3 taps, no bias, theta 1e4, eps 1e-5, tied head, layers by `layer_types`.
TINY_A = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 4,
    "num_attention_heads": 4, "num_key_value_heads": 2,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "conv_L_cache": 3, "conv_bias": False, "block_ff_dim": 128, "block_auto_adjust_ff_dim": False,
    "norm_eps": 1e-5, "rope_theta": 10000.0, "tie_embedding": True,
}

# 6 layers, attention at [0, 2, 5], hidden 96, 4 heads / 1 kv head (MQA), head 24 (not a power
# of two, not a multiple of 16), ff 384 -> 256 by the 2/3 rule at multiple_of 32, vocab 503 (odd),
# 4 taps, conv bias, theta 1e6, eps 1e-6, untied head, layers by `full_attn_idxs`.
TINY_B = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 503, "hidden_size": 96, "num_hidden_layers": 6,
    "num_attention_heads": 4, "num_key_value_heads": 1,
    "full_attn_idxs": [0, 2, 5],
    "conv_L_cache": 4, "conv_bias": True, "block_ff_dim": 384, "block_auto_adjust_ff_dim": True,
    "block_multiple_of": 32, "norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_embedding": False,
}

# 5 layers ending in a conv layer, hidden 192, 6 heads / 3 kv heads, head 32, ff 200 (no power of
# two), vocab 1000, 2 taps (one value of history), eps 1e-5.
TINY_C = {
    "architectures": ["Lfm2ForCausalLM"], "model_type": "lfm2",
    "vocab_size": 1000, "hidden_size": 192, "num_hidden_layers": 5,
    "num_attention_heads": 6, "num_key_value_heads": 3,
    "layer_types": ["full_attention", "conv", "full_attention", "conv", "conv"],
    "conv_L_cache": 2, "conv_bias": False, "intermediate_size": 200,
    "norm_eps": 1e-5, "rope_theta": 500000.0, "tie_word_embeddings": True,
}

# name -> (config, seed, init style).  "fan_in" draws N(0, 1/fan_in) with norm weights 1 + 0.1 N(0,1)
# so that logits and attention are far from flat; "normal" is N(0, 0.02) with norm weights 1.
TINY = {
    "a": (TINY_A, 0, "fan_in"),
    "b": (TINY_B, 1, "fan_in"),
    "c": (TINY_C, 2, "fan_in"),
    "a_normal": (TINY_A, 0, "normal"),
}
