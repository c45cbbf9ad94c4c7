"""A plain, slow implementation of the Qwen2.5 dense decoder: whole sequences, no
cache, one function per part, float64, on whatever device its weights lie (the CPU unless
a test moves them: float64 has no reduced-precision mode on any device).  It is written from the formulas of
the reference project nature-li/qwen-decoder (each function cites file:line there) and
shares no code with the engine: it reads a model folder with the ``safetensors``
package and ``json``.

``tests/golden/`` holds logits made by the reference's own CPU forward
(cpu_decoder.cpp, compiled unmodified) for a tiny random model; ``test_plain_model.py``
checks this file against them.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# ----------------------------------------------------------------------- folder
def read_folder(model_dir: str):
    """(config dict, {name: float64 tensor}) of a model folder."""
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt", device="cpu") as sf:
        for k in sf.keys():
            tensors[k] = sf.get_tensor(k).to(F64)
    return cfg, tensors


def head_dim_of(cfg) -> int:
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


# ------------------------------------------------------------------------ parts
def embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x[t, :] = table[tokens[t], :]  (gpu_kernels.cu:18-29; cpu_decoder.cpp:118-119)."""
    return table[torch.as_tensor(list(tokens), dtype=torch.long, device=table.device)]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum(x^2); out = x * (1 / sqrt(ss / dim + eps)) * w  (cpu_decoder.cpp:48-53;
    gpu_kernels.cu:41-65, where eps is the literal 1e-6 at :63)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(ss / x.shape[-1] + eps)) * w


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, i] = sum_j x[t, j] * w[i, j] (+ b[i])  (cpu_decoder.cpp:55-62; bias added after the
    product, cpu_decoder.cpp:131-133, gpu_kernels.cu:70-79)."""
    y = x @ w.t()
    return y + b if b is not None else y


def rope(x: torch.Tensor, positions: torch.Tensor, n_heads: int, head_dim: int, base: float,
         pairing: str = "adjacent") -> torch.Tensor:
    """Per head, pair p: theta = 1 / base^(2p / head_dim); angle = theta * pos;
    (x0, x1) -> (x0 cos - x1 sin, x0 sin + x1 cos)  (cpu_decoder.cpp:135-157;
    gpu_kernels.cu:94-100).  The reference pairs adjacent elements (2p, 2p+1); ``half``
    pairs (p, p + head_dim/2), the convention of this architecture's safetensors checkpoints."""
    T = x.shape[0]
    x = x.reshape(T, n_heads, head_dim).clone()
    p = torch.arange(head_dim // 2, dtype=F64, device=x.device)
    theta = 1.0 / torch.pow(torch.tensor(base, dtype=F64, device=x.device), 2.0 * p / head_dim)
    ang = positions.to(device=x.device, dtype=F64)[:, None] * theta[None, :]          # [T, d/2]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if pairing == "adjacent":
        x0, x1 = x[..., 0::2].clone(), x[..., 1::2].clone()
        x[..., 0::2] = x0 * c - x1 * s
        x[..., 1::2] = x0 * s + x1 * c
    elif pairing == "half":
        h = head_dim // 2
        x0, x1 = x[..., :h].clone(), x[..., h:].clone()
        x[..., :h] = x0 * c - x1 * s
        x[..., h:] = x0 * s + x1 * c
    else:
        raise ValueError(pairing)
    return x.reshape(T, n_heads * head_dim)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_heads: int, n_kv_heads: int,
              head_dim: int, window: Optional[int] = None) -> torch.Tensor:
    """Query at position t reads keys 0..t of kv head h / (H / G): score = (q . k) / sqrt(d),
    softmax with the maximum subtracted, weighted sum of v  (cpu_decoder.cpp:160-193;
    gpu_kernels.cu:222-311).  ``window`` (not in the reference) keeps keys t-window+1..t."""
    T = q.shape[0]
    kv_mul = n_heads // n_kv_heads
    scale = 1.0 / math.sqrt(head_dim)
    q = q.reshape(T, n_heads, head_dim)
    k = k.reshape(T, n_kv_heads, head_dim)
    v = v.reshape(T, n_kv_heads, head_dim)
    out = torch.zeros(T, n_heads, head_dim, dtype=F64, device=q.device)
    idx = torch.arange(T, device=q.device)
    for h in range(n_heads):
        g = h // kv_mul
        scores = (q[:, h, :] @ k[:, g, :].t()) * scale                  # [T, T]
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask = mask | (idx[None, :] < idx[:, None] - window + 1)
        scores = scores.masked_fill(mask, float("-inf"))
        scores = scores - scores.max(dim=-1, keepdim=True).values
        e = scores.exp()
        out[:, h, :] = (e / e.sum(dim=-1, keepdim=True)) @ v[:, g, :]
    return out.reshape(T, n_heads * head_dim)


def silu(x: torch.Tensor) -> torch.Tensor:
    """x * 1 / (1 + exp(-x))  (cpu_decoder.cpp:64; gpu_kernels.cu:157-158)."""
    return x * (1.0 / (1.0 + torch.exp(-x)))


def swiglu_ffn(x, w_gate, w_up, w_down) -> torch.Tensor:
    """hb = x W1^T, hb2 = x W3^T, hb = silu(hb) * hb2, out = hb W2^T  (cpu_decoder.cpp:204-211;
    W1 = gate, W3 = up, W2 = down: common.cpp:160-172)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def attention_block(x, w: Dict[str, torch.Tensor], prefix: str, cfg, positions, window=None) -> torch.Tensor:
    """q, k, v projections with bias, rotation of q and k, attention, output projection
    (cpu_decoder.cpp:125-198)."""
    H, G, d = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim_of(cfg)
    bias = lambda n: w.get(f"{prefix}self_attn.{n}_proj.bias")
    q = linear(x, w[f"{prefix}self_attn.q_proj.weight"], bias("q"))
    k = linear(x, w[f"{prefix}self_attn.k_proj.weight"], bias("k"))
    v = linear(x, w[f"{prefix}self_attn.v_proj.weight"], bias("v"))
    pairing = cfg.get("rope_pairing", "half")      # the configuration's default; the reference's is "adjacent"
    q = rope(q, positions, H, d, cfg["rope_theta"], pairing)
    k = rope(k, positions, G, d, cfg["rope_theta"], pairing)
    a = attention(q, k, v, H, G, d, window)
    return linear(a, w[f"{prefix}self_attn.o_proj.weight"])


def decoder_layer(x, w, prefix: str, cfg, positions) -> torch.Tensor:
    """x += attention(norm(x)); x += ffn(norm(x))  (cpu_decoder.cpp:121-212)."""
    eps = cfg["rms_norm_eps"]
    x = x + attention_block(rmsnorm(x, w[f"{prefix}input_layernorm.weight"], eps), w, prefix, cfg, positions)
    h = rmsnorm(x, w[f"{prefix}post_attention_layernorm.weight"], eps)
    return x + swiglu_ffn(h, w[f"{prefix}mlp.gate_proj.weight"], w[f"{prefix}mlp.up_proj.weight"],
                          w[f"{prefix}mlp.down_proj.weight"])


def forward(cfg, w: Dict[str, torch.Tensor], tokens: Sequence[int],
            rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [len(tokens), vocab] of one whole sequence from position 0
    (cpu_decoder.cpp:111-220; final norm :216, output projection :219; with
    ``tie_word_embeddings`` the output matrix is the embedding table).  With ``rows`` only the
    logits at those positions, [len(rows), vocab] (a large vocabulary times a long sequence is
    more than a test needs)."""
    x = embedding(w["model.embed_tokens.weight"], tokens)
    positions = torch.arange(len(tokens), device=x.device)
    for l in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, f"model.layers.{l}.", cfg, positions)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long, device=x.device)]
    x = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(x, head)


# --------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor) -> int:
    """First maximum wins (common.cpp:564-574)."""
    best, idx = logits[0], 0
    for i in range(1, logits.numel()):
        if logits[i] > best:
            best, idx = logits[i], i
    return idx


def sample_topk(logits: torch.Tensor, k: int, temperature: float, r: float):
    """The reference's sampler with the uniform draw ``r`` given (common.cpp:576-629):
    temperature 0 -> argmax; else keep logits >= the k-th largest (all if k <= 0 or k >= V),
    p_i = exp((l_i - max) / T) / sum, return the first i with r <= p_0 + ... + p_i.
    Returns (token, margin): margin is how far r * sum is from the nearest step of the running sum,
    so that a test can skip draws that float32 rounding could decide either way."""
    if temperature == 0.0:
        return argmax(logits), float("inf")
    l = logits.to(F64)
    V = l.numel()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < k < V:
        threshold = torch.sort(l, descending=True).values[k - 1]
        keep = l >= threshold
    p = torch.where(keep, torch.exp((l - l.max()) / temperature), torch.zeros_like(l))
    cum = torch.cumsum(p / p.sum(), 0)
    hit = torch.nonzero(cum >= r)
    tok = int(hit[0]) if hit.numel() else V - 1
    margin = float((cum - r).abs().min())
    return tok, margin


def greedy_generate(cfg, w, prompt: Sequence[int], n_new: int) -> List[int]:
    """Feed the prompt, then each sampled token in turn, taking the argmax every time; the
    margin between the two best logits comes back too (a test may stop at a near tie)."""
    seq = list(prompt)
    out, margins = [], []
    for _ in range(n_new):
        logits = forward(cfg, w, seq)[-1]
        top2 = torch.topk(logits, 2).values
        tok = int(torch.argmax(logits))
        out.append(tok)
        margins.append(float(top2[0] - top2[1]))
        seq.append(tok)
    return out, margins
