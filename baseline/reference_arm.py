"""The reference arm of bench.py: nature-li/qwen-decoder's own ``gpu_decoder_main``, unmodified, run as the
program it is (gpu_main.cu:12-71) on a model file written here.

The reference is a CMake project of executables, not a Python package: pip cannot install it, and its
CMakeLists.txt as a whole needs Drogon, gRPC and MPI (CMakeLists.txt:17-30).  The one target that the
benchmark needs, ``gpu_decoder_main`` (CMakeLists.txt:125-134), is nine source files and cuBLAS; it is
compiled from an untouched copy of the source tree under ``baseline/_ref/src`` with one nvcc command
(architecture 100 as CMakeLists.txt:9 sets it) into ``baseline/_ref/gpu_decoder_main``.

What it runs on: a GGUF v3 file (gguf_loader.cpp:107-156) with random float16 weights N(0, 0.02) at the
benchmark's layer sizes, float32 norms and biases (common.cpp:104-172), and a vocabulary whose first 256
entries are the single characters that the tokenizer maps bytes to (common.cpp:297-318), without merges:
a prompt line of n characters becomes exactly n tokens (common.cpp:393-470).  The program wraps each
line in its chat template (common.cpp:556-562) and puts a BOS token in front (decoder.cpp:20-22), so a
line is made ``TEMPLATE_TOKENS + 1`` characters shorter than the wanted prompt.  It decodes greedily
(gpu_main.cu:45-48) for 256 tokens and prints one line per step with the wall time since the step
before (decoder.cpp:178-185); a decode step's time is the ``between`` of the line after it.
"""
from __future__ import annotations

import os
import re
import shutil
import struct
import subprocess
import sys
import time
from typing import Dict, List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
SRC_DIR = os.path.join(REF_DIR, "src")
BINARY = os.path.join(REF_DIR, "gpu_decoder_main")
SOURCES = ["gpu_kernels.cu", "gpu_decoder.cu", "gpu_main.cu", "decoder.cpp", "common.cpp", "gguf_loader.cpp",
           "scheduler.cpp", "kv_cache.cpp", "prefix_cache.cpp"]          # CMakeLists.txt:125-134
TEMPLATE = ("<|im_start|>system\nYou are a helpful assistant.<|im_end|>\n<|im_start|>user\n", "<|im_end|>\n<|im_start|>assistant\n")
TEMPLATE_TOKENS = len(TEMPLATE[0].encode()) + len(TEMPLATE[1].encode())     # one token per byte with this vocabulary
NEW_TOKENS = 256                                                          # fixed in gpu_main.cu:48

U32, I32, F32, STRING, ARRAY = 4, 5, 6, 8, 9          # gguf_loader.h:21-35
GGML_F32, GGML_F16 = 0, 1


class Unavailable(RuntimeError):
    """The reference cannot be built or run here; the message is the one-line reason."""


def find_sources() -> Optional[str]:
    for cand in (SRC_DIR, os.environ.get("QWEN_DECODER_REF"), "/root/reference"):
        if cand and all(os.path.isfile(os.path.join(cand, f)) for f in SOURCES):
            return cand
    return None


def ensure_binary(verbose: bool = True) -> str:
    """The built program; compiled first if it is not there (needs the source tree and nvcc)."""
    if os.path.isfile(BINARY) and os.access(BINARY, os.X_OK):
        return BINARY
    src = find_sources()
    if src is None:
        raise Unavailable("no copy of the reference's sources (baseline/_ref/src) and no built gpu_decoder_main")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise Unavailable("nvcc not found to build the reference's gpu_decoder_main")
    os.makedirs(REF_DIR, exist_ok=True)
    if os.path.abspath(src) != os.path.abspath(SRC_DIR):
        # an untouched copy travels with the repository's folder to machines that have no source tree
        shutil.copytree(src, SRC_DIR, dirs_exist_ok=True)
        src = SRC_DIR
    cmd = [nvcc, "-std=c++17", "-O3", "-arch=sm_100", "-diag-suppress", "997", f"-I{src}"] + \
        [os.path.join(src, f) for f in SOURCES] + ["-lcublas", "-o", BINARY]
    if verbose:
        print("[reference] building gpu_decoder_main ...", file=sys.stderr, flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise Unavailable("nvcc failed on the reference's gpu_decoder_main: " + proc.stderr.strip().splitlines()[-1][:200])
    return BINARY


# ------------------------------------------------------------------------------------------ the model file
def byte_characters() -> List[str]:
    """The character the reference's tokenizer turns each byte into (common.cpp:297-318): printable
    bytes (33-126, 161-172, 174-255) stand for themselves, the others become code points 256, 257, ...
    in byte order."""
    own = list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256))
    table, n = {}, 0
    for b in own:
        table[b] = chr(b)
    for b in range(256):
        if b not in table:
            table[b] = chr(256 + n)
            n += 1
    return [table[b] for b in range(256)]


def _gstr(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, cfg: Dict, seed: int = 0, context_length: int = 4096, device: str = "cuda:0") -> int:
    """Write random weights of ``cfg`` (config.json keys) as a GGUF file the reference loads; returns bytes.
    Tensors are made one at a time (on ``device`` when that is a GPU: the generator is fast there)."""
    import torch
    D, F, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    H, G, V = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["vocab_size"]
    d = D // H
    dev = torch.device(device if (not device.startswith("cuda") or torch.cuda.is_available()) else "cpu")
    kv = [("qwen2.embedding_length", U32, D), ("qwen2.feed_forward_length", U32, F), ("qwen2.block_count", U32, L),
          ("qwen2.attention.head_count", U32, H), ("qwen2.attention.head_count_kv", U32, G),
          ("qwen2.context_length", U32, context_length), ("qwen2.rope.freq_base", F32, float(cfg["rope_theta"])),
          # no token the greedy decoding may stop on by accident more often than any other: the last ids
          ("tokenizer.ggml.bos_token_id", U32, V - 1), ("tokenizer.ggml.eos_token_id", U32, V - 2)]
    tensors = [("token_embd.weight", (V, D), "w"), ("output.weight", (V, D), "w"), ("output_norm.weight", (D,), "n")]
    for l in range(L):
        b = f"blk.{l}."
        tensors += [(b + "attn_norm.weight", (D,), "n"), (b + "attn_q.weight", (H * d, D), "w"),
                    (b + "attn_k.weight", (G * d, D), "w"), (b + "attn_v.weight", (G * d, D), "w"),
                    (b + "attn_output.weight", (D, H * d), "w"), (b + "attn_q.bias", (H * d,), "b"),
                    (b + "attn_k.bias", (G * d,), "b"), (b + "attn_v.bias", (G * d,), "b"),
                    (b + "ffn_norm.weight", (D,), "n"), (b + "ffn_gate.weight", (F, D), "w"),
                    (b + "ffn_up.weight", (F, D), "w"), (b + "ffn_down.weight", (D, F), "w")]
    infos, off = [], 0
    for name, shape, kind in tensors:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * (2 if kind == "w" else 4)
        infos.append((name, list(reversed(shape)), GGML_F16 if kind == "w" else GGML_F32, off))    # dims innermost first
        off += (nbytes + 31) // 32 * 32
    vocab = byte_characters() + [f"[{i}]" for i in range(256, V)]
    head = struct.pack("<IIQQ", 0x46554747, 3, len(infos), len(kv) + 2)
    for k, t, v in kv:
        head += _gstr(k) + struct.pack("<I", t) + (struct.pack("<I", v) if t == U32 else struct.pack("<f", v))
    head += _gstr("tokenizer.ggml.tokens") + struct.pack("<IIQ", ARRAY, STRING, V) + b"".join(_gstr(s) for s in vocab)
    # every token an ordinary one (type 1): the encoder reads this array for every id (common.cpp:399-403)
    head += _gstr("tokenizer.ggml.token_type") + struct.pack("<IIQ", ARRAY, I32, V) + struct.pack("<i", 1) * V
    for n, dims, t, o in infos:
        head += _gstr(n) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", x) for x in dims) + struct.pack("<IQ", t, o)
    head += b"\0" * ((32 - len(head) % 32) % 32)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    written = len(head)
    with open(path, "wb") as f:
        f.write(head)
        for (name, shape, kind), (_, _, _, o) in zip(tensors, infos):
            t = torch.empty(shape, dtype=torch.float32, device=dev)
            if kind == "n":
                t.normal_(0.0, 0.1, generator=gen).add_(1.0)
            else:
                t.normal_(0.0, 0.02, generator=gen)
            raw = (t.half() if kind == "w" else t).cpu().numpy().tobytes()
            if name == "output.weight" and cfg.get("tie_word_embeddings"):
                raw = tied_raw                      # the reference has no tied output: the same matrix twice
            if name == "token_embd.weight":
                tied_raw = raw
            pad = (32 - len(raw) % 32) % 32
            f.write(raw + b"\0" * pad)
            written += len(raw) + pad
    return written


# ------------------------------------------------------------------------------------------ the run
STEP_LINE = re.compile(r"between ([0-9.]+), step (\d+): total_tokens=(\d+) n_decode=(\d+) n_prefill=(\d+) prefill_tokens=(\d+)")
TOTAL_LINE = re.compile(r"total: (\d+) tokens in ([0-9.]+)s")


def parse(stdout: str, stderr: str, batch: int) -> Dict:
    """Per-step records of the program's own lines: a step's wall time is the ``between`` printed by the
    step after it (decoder.cpp:178-185 prints the time since the line before)."""
    steps = [(float(m[1]), int(m[2]), int(m[3]), int(m[4]), int(m[5]), int(m[6])) for m in STEP_LINE.finditer(stdout)]
    decode_ms, prefill = [], []
    for cur, nxt in zip(steps, steps[1:]):
        ms = nxt[0]
        if cur[4] == 0 and cur[3] == batch and nxt[4] == 0:          # all requests decode, in this step and the next
            decode_ms.append(ms)
        elif cur[5] > 0:
            prefill.append((cur[5], cur[3], ms))
    out = {"n_steps": len(steps), "decode_ms": decode_ms, "prefill_steps": prefill}
    m = TOTAL_LINE.search(stderr)
    if m:
        out["total_tokens"], out["total_s"] = int(m[1]), float(m[2])
    return out


def run(model_path: str, batch: int, prompt_tokens: int, max_prefill_step: int = 4096, timeout_s: float = 900.0,
        log_path: Optional[str] = None) -> Dict:
    """``gpu_decoder_main model batch 4096 max_prefill_step max_total 0`` with ``batch`` prompt lines on its
    standard input; returns ``parse``'s record.  Killed (its own process only) after ``timeout_s``."""
    exe = ensure_binary()
    n_chars = prompt_tokens - TEMPLATE_TOKENS - 1
    if n_chars < 1:
        raise Unavailable(f"a prompt of {prompt_tokens} tokens is shorter than the program's chat template")
    import random
    rng = random.Random(1)
    letters = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789"
    lines = ["".join(rng.choice(letters) for _ in range(n_chars)) for _ in range(batch)]
    stdin = "\n".join(lines) + "\n\n"
    cmd = [exe, model_path, str(batch), "4096", str(max_prefill_step), str(max_prefill_step + batch), "0"]
    t0 = time.time()
    # bytes, not text: the program prints the decoded output of random weights, which is no valid UTF-8
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE)
    text = lambda b: b.decode("utf-8", errors="replace")
    try:
        out, err = (text(b) for b in proc.communicate(stdin.encode(), timeout=timeout_s))
    except subprocess.TimeoutExpired:
        proc.kill()
        out, err = (text(b) for b in proc.communicate())
        if log_path:
            open(log_path, "w").write(out[-20000:] + "\n---- stderr ----\n" + err[-5000:])
        raise Unavailable(f"the reference's gpu_decoder_main did not finish batch {batch} within {timeout_s:.0f} s")
    if log_path:
        # the step lines and the totals; the echoed prompts and outputs are left out
        keep = [ln[ln.find("between"):] if "between" in ln else ln for ln in out.splitlines()
                if "between" in ln or ln.startswith("BlockPool")]
        open(log_path, "w").write("\n".join(keep) + "\n---- stderr ----\n" + err[-5000:])
    if proc.returncode != 0:
        last = (err.strip().splitlines() or ["no message"])[-1][:200]
        raise Unavailable(f"the reference's gpu_decoder_main exited with {proc.returncode}: {last}")
    rec = parse(out, err, batch)
    rec["seconds"] = time.time() - t0
    return rec
