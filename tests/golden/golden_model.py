"""The tiny model behind the committed reference logits: sizes of tiny configuration A and
weights from a small explicit generator (no library random numbers), so that the script that
made the golden file and the test that reads it build identical tensors everywhere.

Every matrix element is k * 2^-12 with k an integer in [-163, 163] \\ {0}: exactly representable in
float16 and never a float16 subnormal (the reference's fp16_to_float decodes subnormals as about
zero, common.cpp:211-213).  Norm scales are 1 + k * 2^-7, biases k * 2^-12, stored in float32 as the
reference expects (common.cpp:104-112).
"""
import numpy as np

CONFIG = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=64, intermediate_size=176, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, vocab_size=512, max_position_embeddings=64,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, rope_pairing="adjacent")
TOKENS = [5, 17, 3, 250, 99, 511, 0, 42, 42, 7, 300, 128]


def _ints(n: int, seed: int, lo: int, hi: int) -> np.ndarray:
    """n integers in [lo, hi] from a 64-bit linear congruential generator."""
    out = np.empty(n, dtype=np.int64)
    x = (seed * 2654435761 + 12345) % (1 << 64)
    span = hi - lo + 1
    for i in range(n):
        x = (x * 6364136223846793005 + 1442695040888963407) % (1 << 64)
        out[i] = lo + (x >> 33) % span
    return out


def _matrix(shape, seed):
    k = _ints(int(np.prod(shape)), seed, -163, 163)
    k[k == 0] = 1
    return (k.astype(np.float64) / 4096.0).reshape(shape)


def weights():
    """{HF tensor name: float64 array}."""
    c = CONFIG
    D, F, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    H, G = c["num_attention_heads"], c["num_key_value_heads"]
    d = D // H
    w = {"model.embed_tokens.weight": _matrix((V, D), 1), "lm_head.weight": _matrix((V, D), 2),
         "model.norm.weight": 1.0 + _ints(D, 3, -20, 20) / 128.0}
    for l in range(c["num_hidden_layers"]):
        p, s = f"model.layers.{l}.", 100 * (l + 1)
        w[p + "input_layernorm.weight"] = 1.0 + _ints(D, s + 1, -20, 20) / 128.0
        w[p + "post_attention_layernorm.weight"] = 1.0 + _ints(D, s + 2, -20, 20) / 128.0
        w[p + "self_attn.q_proj.weight"] = _matrix((H * d, D), s + 3)
        w[p + "self_attn.k_proj.weight"] = _matrix((G * d, D), s + 4)
        w[p + "self_attn.v_proj.weight"] = _matrix((G * d, D), s + 5)
        w[p + "self_attn.o_proj.weight"] = _matrix((D, H * d), s + 6)
        w[p + "self_attn.q_proj.bias"] = _matrix((H * d,), s + 7)
        w[p + "self_attn.k_proj.bias"] = _matrix((G * d,), s + 8)
        w[p + "self_attn.v_proj.bias"] = _matrix((G * d,), s + 9)
        w[p + "mlp.gate_proj.weight"] = _matrix((F, D), s + 10)
        w[p + "mlp.up_proj.weight"] = _matrix((F, D), s + 11)
        w[p + "mlp.down_proj.weight"] = _matrix((D, F), s + 12)
    return w
