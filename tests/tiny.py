"""The tiny Qwen3 configurations of the tests. They differ in every size and option: layers, width,
query and key/value heads (and so the group size), head size (16, 24 with heads * head_dim != width,
64 for the tensor-core kernels, 32), intermediate size, vocabulary (no power of two in B and C),
rope_theta, rms_norm_eps, q/k/v biases, tied or separate output matrix, context, and a sliding
window on some layers (C, E, F). F and G have the sizes that send their single-token steps through the
persistent kernel."""

A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=256, hidden_size=64,
         intermediate_size=192, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
         rope_theta=10000.0, rms_norm_eps=1e-6, attention_bias=False, tie_word_embeddings=True,
         max_position_embeddings=128)

B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=503, hidden_size=96,
         intermediate_size=160, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=24,
         rope_theta=1000000.0, rms_norm_eps=1e-5, attention_bias=True, tie_word_embeddings=False,
         max_position_embeddings=256)

# head_dim 64 takes the tensor-core attention kernels in bfloat16; one KV head (group of 5); windows on two layers
C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=311, hidden_size=80,
         intermediate_size=136, num_hidden_layers=4, num_attention_heads=5, num_key_value_heads=1, head_dim=64,
         rope_theta=50000.0, rms_norm_eps=3e-6, attention_bias=True, tie_word_embeddings=True,
         max_position_embeddings=512, sliding_window=40,
         layer_types=["full_attention", "sliding_attention", "full_attention", "sliding_attention"])

# head_dim 128, the benchmark's head size, with a group of 2; long context for the long-decoding test
D = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=640, hidden_size=128,
         intermediate_size=200, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
         rope_theta=1000000.0, rms_norm_eps=1e-6, attention_bias=False, tie_word_embeddings=False,
         max_position_embeddings=1024)

# head_dim 64 with a group of 4 (a divisor of 128): prompts of this one run the tensor-memory attention kernel and
# the q/k/v product with its fused epilogue at head size 64, with biases, and with a window on the middle layer
E = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=777, hidden_size=192,
         intermediate_size=264, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
         rope_theta=100000.0, rms_norm_eps=2e-6, attention_bias=True, tie_word_embeddings=False,
         max_position_embeddings=512, sliding_window=48,
         layer_types=["full_attention", "sliding_attention", "full_attention"])

# Sizes that the persistent single-token kernel takes (width a multiple of 128, head size 64, intermediate a multiple
# of 32): decode steps of up to 16 sequences of this one run through it, with biases, a group of 2 and a window on the
# middle layer
F = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=333, hidden_size=128,
         intermediate_size=96, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
         rope_theta=500000.0, rms_norm_eps=1e-5, attention_bias=True, tie_word_embeddings=False,
         max_position_embeddings=512, sliding_window=70,
         layer_types=["full_attention", "sliding_attention", "full_attention"])

# The same kernel at head size 128 with a group of 3, no biases, no window, a wider intermediate
G = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=410, hidden_size=256,
         intermediate_size=160, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=128,
         rope_theta=20000.0, rms_norm_eps=3e-6, attention_bias=False, tie_word_embeddings=True,
         max_position_embeddings=1024)

CONFIGS = {"A": A, "B": B, "C": C, "D": D, "E": E, "F": F, "G": G}
SEEDS = {"A": 11, "B": 22, "C": 33, "D": 44, "E": 55, "F": 66, "G": 77}
