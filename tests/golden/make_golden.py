#!/usr/bin/env python3
"""Makes tests/golden/reference_cpu_logits.npy and reference_cpu_logits_b.npy: logits of the reference
project's own CPU forward (nature-li/qwen-decoder, cpu_decoder.cpp:111-220, compiled unmodified from its
source tree) for the two tiny models of golden_model.py, one row per token fed at positions 0, 1, 2, ...
The second model reaches the reference as an equivalent model with adjacent rotary pairs and eps 1e-6
(golden_model.weights_b_reference), and so pins half-split pairs, another eps, one key/value head and
an output matrix of its own on the reference's code.

Usage: python tests/golden/make_golden.py [path to the reference source tree]

How: (1) the weights are written as a GGUF v3 file the reference's loader reads
(gguf_loader.cpp:107-156: header, typed metadata, tensor infos, data aligned to 32 bytes; tensor names
and types of common.cpp:113-176; metadata keys of common.cpp:65-71 and 231-251; dims innermost first,
common.cpp:76); (2) cpu_decoder.cpp does not compile on its own (it uses ``config`` and ``tokenizer``
without declaring them), so a wrapper translation unit declares the two at file scope and includes it;
(3) the wrapper calls CPUDecoder::forward(token, pos) and dumps get_logits().
"""
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import golden_model  # noqa: E402

U32, F32, STRING, ARRAY = 4, 6, 8, 9
GGML_F32, GGML_F16 = 0, 1


def gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, c: dict, w: dict) -> None:
    L = c["num_hidden_layers"]
    kv = [
        ("qwen2.embedding_length", U32, c["hidden_size"]), ("qwen2.feed_forward_length", U32, c["intermediate_size"]),
        ("qwen2.block_count", U32, L), ("qwen2.attention.head_count", U32, c["num_attention_heads"]),
        ("qwen2.attention.head_count_kv", U32, c["num_key_value_heads"]),
        ("qwen2.context_length", U32, c["max_position_embeddings"]), ("qwen2.rope.freq_base", F32, c["rope_theta"]),
        ("tokenizer.ggml.bos_token_id", U32, 1), ("tokenizer.ggml.eos_token_id", U32, 2),
    ]
    names = {"token_embd.weight": "model.embed_tokens.weight", "output.weight": "lm_head.weight",
             "output_norm.weight": "model.norm.weight"}
    for l in range(L):
        p = f"model.layers.{l}."
        for g, h in [("attn_norm.weight", "input_layernorm.weight"), ("attn_q.weight", "self_attn.q_proj.weight"),
                     ("attn_k.weight", "self_attn.k_proj.weight"), ("attn_v.weight", "self_attn.v_proj.weight"),
                     ("attn_output.weight", "self_attn.o_proj.weight"), ("attn_q.bias", "self_attn.q_proj.bias"),
                     ("attn_k.bias", "self_attn.k_proj.bias"), ("attn_v.bias", "self_attn.v_proj.bias"),
                     ("ffn_norm.weight", "post_attention_layernorm.weight"), ("ffn_gate.weight", "mlp.gate_proj.weight"),
                     ("ffn_up.weight", "mlp.up_proj.weight"), ("ffn_down.weight", "mlp.down_proj.weight")]:
            names[f"blk.{l}.{g}"] = p + h
    blobs, infos, off = [], [], 0
    for gname, hname in names.items():
        a = w[hname]
        if a.ndim == 2:
            data, t = a.astype(np.float16), GGML_F16
            assert np.array_equal(data.astype(np.float64), a), hname      # exactly representable
        else:
            data, t = a.astype(np.float32), GGML_F32
        raw = data.tobytes()
        infos.append((gname, list(reversed(a.shape)), t, off))
        blobs.append(raw + b"\0" * ((32 - len(raw) % 32) % 32))
        off += len(blobs[-1])
    out = struct.pack("<IIQQ", 0x46554747, 3, len(infos), len(kv) + 1)
    for k, t, v in kv:
        out += gstr(k) + struct.pack("<I", t) + (struct.pack("<I", v) if t == U32 else struct.pack("<f", v))
    out += gstr("tokenizer.ggml.tokens") + struct.pack("<IIQ", ARRAY, STRING, c["vocab_size"])
    out += b"".join(gstr(f"t{i}") for i in range(c["vocab_size"]))
    for n, dims, t, o in infos:
        out += gstr(n) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", t, o)
    out += b"\0" * ((32 - len(out) % 32) % 32)
    with open(path, "wb") as f:
        f.write(out + b"".join(blobs))


WRAPPER = r'''
#include "cpu_decoder.h"
static Config config;
static Tokenizer tokenizer;
#include "cpu_decoder.cpp"
#include <cstdio>
#include <cstdlib>
int main(int argc, char** argv) {
  CPUDecoder dec(argv[1]);
  FILE* out = fopen(argv[2], "wb");
  int vocab = atoi(argv[3]);
  for (int i = 4; i < argc; i++) {
    dec.forward(atoi(argv[i]), i - 4);
    fwrite(dec.get_logits(), sizeof(float), vocab, out);
  }
  fclose(out);
  return 0;
}
'''


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QWEN_DECODER_REF")
    if not ref or not os.path.isfile(os.path.join(ref, "cpu_decoder.cpp")):
        sys.exit("usage: make_golden.py <folder of the reference's sources>   (or QWEN_DECODER_REF=<folder>)")
    with tempfile.TemporaryDirectory() as tmp:
        gguf, wrap, exe, raw = (os.path.join(tmp, n) for n in ("m.gguf", "wrap.cpp", "golden", "out.bin"))
        open(wrap, "w").write(WRAPPER)
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-ffp-contract=off", f"-I{ref}", "-I/usr/local/cuda/include",
                               wrap, os.path.join(ref, "common.cpp"), os.path.join(ref, "gguf_loader.cpp"),
                               "-o", exe])
        for out_name, config, weights, tokens in (
                ("reference_cpu_logits.npy", golden_model.CONFIG, golden_model.weights(), golden_model.TOKENS),
                ("reference_cpu_logits_b.npy", golden_model.CONFIG_B, golden_model.weights_b_reference(),
                 golden_model.TOKENS_B)):
            write_gguf(gguf, config, weights)
            V = config["vocab_size"]
            subprocess.check_call([exe, gguf, raw, str(V)] + [str(t) for t in tokens])
            logits = np.fromfile(raw, dtype="<f4").reshape(len(tokens), V)
            np.save(os.path.join(HERE, out_name), logits)
            print("wrote", out_name, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
