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


# ---------------------------------------------------------------------------------------------------
# A second model, for what the first cannot pin: half-split rotary pairs, an eps other than 1e-6, one
# key/value head, other sizes.  The reference's CPU forward knows adjacent pairs and eps = 1e-6 only
# (cpu_decoder.cpp:135-157, :51), so it is given an *equivalent* model:
#
# * pairing: rotating pairs (p, p + d/2) of q and k is rotating adjacent pairs (2p, 2p+1) of the same
#   vectors with their elements reordered, and a score q.k does not change when q and k are reordered
#   alike.  So the rows of Wq, Wk (and bq, bk) are reordered per head: row p -> 2p, row p + d/2 -> 2p + 1.
# * eps: with the embedding, o_proj and down_proj scaled by c the whole residual sum is scaled by c, and
#   rmsnorm(c x; eps0) = x / sqrt(mean(x^2) + eps0 / c^2) * w = rmsnorm(x; eps0 / c^2).  With eps0 = 1e-6
#   and c^2 = 0.1 that is eps = 1e-5.  The output matrix is a tensor of its own and stays as it is.
#
# The tensors handed to the reference ("reference side") come from the explicit generator, exactly
# representable in float16; the model they stand for (what tests/plain_model.py computes with
# rope_pairing "half" and eps 1e-5) is derived from them in float64.
CONFIG_B = dict(
    architectures=["Qwen2ForCausalLM"], hidden_size=96, intermediate_size=208, num_hidden_layers=3,
    num_attention_heads=3, num_key_value_heads=1, vocab_size=300, max_position_embeddings=64,
    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, rope_pairing="half")
TOKENS_B = [7, 299, 0, 13, 13, 150, 42, 8, 271, 99, 3, 64, 200, 1]
REFERENCE_EPS = 1e-6          # gpu_kernels.cu:63, cpu_decoder.cpp:51


def _interleave_rows(a, n_heads, d):
    """Per head: rows (0 .. d/2-1 | d/2 .. d-1) -> (0, d/2, 1, d/2 + 1, ...): the half-split pair (p, p + d/2)
    lands on the adjacent pair (2p, 2p + 1)."""
    shape = a.shape
    a = a.reshape((n_heads, 2, d // 2) + shape[1:])
    return np.swapaxes(a, 1, 2).reshape(shape)


def _deinterleave_rows(a, n_heads, d):
    shape = a.shape
    a = a.reshape((n_heads, d // 2, 2) + shape[1:])
    return np.swapaxes(a, 1, 2).reshape(shape)


def weights_b_reference():
    """{HF-style tensor name: float64 array} of the model as the reference is given it (adjacent pairs,
    eps 1e-6); config for it: CONFIG_B with rope_pairing "adjacent" and rms_norm_eps 1e-6."""
    c = CONFIG_B
    D, F, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    H, G = c["num_attention_heads"], c["num_key_value_heads"]
    d = D // H
    w = {"model.embed_tokens.weight": _matrix((V, D), 1001), "lm_head.weight": _matrix((V, D), 1002),
         "model.norm.weight": 1.0 + _ints(D, 1003, -20, 20) / 128.0}
    for l in range(c["num_hidden_layers"]):
        p, s = f"model.layers.{l}.", 1000 + 100 * (l + 1)
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


def weights_b():
    """{HF tensor name: float64 array} of the model with half-split pairs and eps 1e-5 that
    ``weights_b_reference`` stands for."""
    c = CONFIG_B
    H, G = c["num_attention_heads"], c["num_key_value_heads"]
    d = c["hidden_size"] // H
    scale = np.sqrt(REFERENCE_EPS / c["rms_norm_eps"])        # the reference side's residual sum is scale * ours
    w = dict(weights_b_reference())
    w["model.embed_tokens.weight"] = w["model.embed_tokens.weight"] / scale
    for l in range(c["num_hidden_layers"]):
        p = f"model.layers.{l}."
        w[p + "self_attn.o_proj.weight"] = w[p + "self_attn.o_proj.weight"] / scale
        w[p + "mlp.down_proj.weight"] = w[p + "mlp.down_proj.weight"] / scale
        for name, n in (("q", H), ("k", G)):
            for kind in ("weight", "bias"):
                key = f"{p}self_attn.{name}_proj.{kind}"
                w[key] = _deinterleave_rows(w[key], n, d)
    return w
