"""The two tiny configurations the tests run on; they differ in every size and option."""

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "eos_token_id": 2, "bos_token_id": 1,
}
TINY_A_INIT = dict(seed=0, std=0.02, norm_jitter=0.1)

TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "intermediate_size": 160, "vocab_size": 320, "rope_theta": 100000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "eos_token_id": [7, 9],
}
TINY_B_INIT = dict(seed=1, std=0.03, norm_jitter=0.2)

# The production head layout in small: head size 64, three query heads per kv head, an intermediate size that is a
# multiple of 64, a vocabulary that is no power of two.  It sends the engine tests through the same kernel
# instantiations as the SmolLM2 sizes.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 384, "num_attention_heads": 6, "num_key_value_heads": 2,
    "intermediate_size": 448, "vocab_size": 1000, "rope_theta": 50000.0, "rms_norm_eps": 2e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 2048,
}
TINY_C_INIT = dict(seed=2, std=0.05, norm_jitter=0.3)
