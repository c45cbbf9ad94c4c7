"""Two tiny configurations of the architecture that differ in every size and option, a third with
other head sizes and a fourth with the head size of the tensor-memory attention kernel; model
folders are made in temporary folders."""
import torch

from qwen_decoder_b200.config import Qwen2Config
from qwen_decoder_b200.weights import write_random_model

TINY_A = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=64, intermediate_size=176, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, vocab_size=512, max_position_embeddings=256,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, rope_pairing="adjacent")
TINY_B = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=128, intermediate_size=352, num_hidden_layers=3,
    num_attention_heads=4, num_key_value_heads=1, vocab_size=1000, max_position_embeddings=512,
    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
# head size not hidden/heads, 6 heads in groups of 3, odd vocabulary, adjacent rotary pairs as in A
# (B and D leave the key out and get the default, half-split pairs)
TINY_C = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=72, intermediate_size=200, num_hidden_layers=2,
    num_attention_heads=6, num_key_value_heads=2, head_dim=48, vocab_size=777,
    max_position_embeddings=384, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
    rope_pairing="adjacent")

# head size 64 in groups of 2: the sizes the tcgen05 attention kernel and the 128-row tiles take
TINY_D = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=96, intermediate_size=264, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=300,
    max_position_embeddings=640, rope_theta=20000.0, rms_norm_eps=2e-6, tie_word_embeddings=True)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3}


def make_folder(name: str, path: str) -> str:
    cfg = Qwen2Config.from_dict(TINY[name])
    return write_random_model(cfg, path, SEEDS[name], dtype=torch.bfloat16)
