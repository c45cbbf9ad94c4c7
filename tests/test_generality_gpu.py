"""Parts chosen layer by layer, the order of layers as data, and parts defined outside the
framework: a toy architecture with windowed and full attention layers, a schedule that names a
layer twice and lets a run read another run's cache, and a toy mixer with per-request state of
its own -- all registered here, without a change to the framework's files."""
import json
import os
import random
from dataclasses import dataclass, field

import numpy as np
import pytest
import torch

import plain_model
import trace_tools
from qwen_decoder_b200.cache import FixedState
from qwen_decoder_b200.config import (LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture,
                                      register_part, unregister_architecture, unregister_part)
from qwen_decoder_b200.parts import FeedForward, Mixer, PositionEncoding
from qwen_decoder_b200.weights import TensorSpec, write_random_model

pytestmark = pytest.mark.gpu
TOL = {"float32": 1e-5, "bfloat16": 3e-2}


# ------------------------------------------------------------ a toy configuration class
@dataclass(frozen=True)
class ToyConfig:
    architecture: str
    hidden_size: int = 48
    intermediate_size: int = 112
    num_heads: int = 3
    num_kv_heads: int = 1
    head_dim: int = 16
    vocab_size: int = 331
    max_positions: int = 256
    eps: float = 2e-6
    rope_base: float = 777.0
    window: int = 20
    kinds: tuple = ()
    schedule: tuple = ()
    routed_layers: tuple = ()        # layers whose feed-forward is the toy routed one
    num_experts: int = 3
    expert_size: int = 40
    gain_period: float = 9.0
    block: str = "pre_norm"
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, d):
        d = dict(d)
        arch = d.pop("architectures")[0]
        d["kinds"] = tuple(d.get("kinds", ()))
        d["schedule"] = tuple(tuple(x) for x in d.get("schedule", ()))
        d["routed_layers"] = tuple(d.get("routed_layers", ()))
        return cls(architecture=arch, **d)

    def to_dict(self):
        d = {k: getattr(self, k) for k in self.__dataclass_fields__ if k not in ("architecture", "eos_token_ids")}
        d["architectures"] = [self.architecture]
        d["kinds"] = list(self.kinds)
        d["schedule"] = [list(x) for x in self.schedule]
        d["routed_layers"] = list(self.routed_layers)
        return d


def describe_toy(c: ToyConfig) -> ModelSpec:
    norm = {"size": c.hidden_size, "eps": c.eps}
    layers = []
    for i, kind in enumerate(c.kinds):
        if kind in ("ema", "ema_gain", "ema_dev"):
            mixer = PartSpec("toy_ema_device" if kind == "ema_dev" else "toy_ema",
                             {"hidden_size": c.hidden_size, "prefix": "mix.",
                              "position": "gain" if kind == "ema_gain" else None})
        else:
            mixer = PartSpec("gq_attention", {
                "hidden_size": c.hidden_size, "num_heads": c.num_heads, "num_kv_heads": c.num_kv_heads,
                "head_dim": c.head_dim, "qkv_bias": True, "out_bias": False, "position": "rope",
                "window": c.window if kind == "window" else None, "prefix": "self_attn."})
        layers.append(LayerSpec(
            prefix=f"model.layers.{i}.", block=c.block, mixer=mixer,
            feed_forward=PartSpec("toy_routed", {"hidden_size": c.hidden_size, "expert_size": c.expert_size,
                                                 "num_experts": c.num_experts, "prefix": "moe."})
            if i in c.routed_layers else
            PartSpec("swiglu", {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size,
                                "prefix": "mlp."}),
            norms={"input": PartSpec("rmsnorm", dict(norm, prefix="input_layernorm.")),
                   "post_mixer": PartSpec("rmsnorm", dict(norm, prefix="post_attention_layernorm."))}))
    sched = [ScheduleEntry(l, None if src < 0 else src) for l, src in c.schedule] or \
        [ScheduleEntry(i) for i in range(len(layers))]
    return ModelSpec(
        hidden_size=c.hidden_size, vocab_size=c.vocab_size, max_positions=c.max_positions,
        embedding_tensor="model.embed_tokens.weight",
        positions={"rope": PartSpec("rotary", {"head_dim": c.head_dim, "rotary_dim": c.head_dim,
                                               "base": c.rope_base, "pairing": "adjacent"}),
                   "gain": PartSpec("toy_gain", {"period": c.gain_period})},
        layers=layers, schedule=sched, final_norm=PartSpec("rmsnorm", dict(norm, prefix="")),
        final_norm_prefix="model.norm.", lm_head_tensor="lm_head.weight")


# ------------------------------------------------------------ another arrangement of the same parts
from qwen_decoder_b200.parts.block import PreNormBlock  # noqa: E402


class ToyParallelBlock(PreNormBlock):
    """x += mixer(norm1(x)) + feed_forward(norm2(x)), both branches from the same x: the parts and tensor
    names of the pre-norm block in another order.  It inherits ``native_params`` and changes nothing there:
    native code that restates the pre-norm order must not take it."""

    def forward(self, stream, ctx, cache):
        h1 = self.input_norm.forward(stream, self.dtype)          # adds what is pending, normalises
        h2 = self.post_mixer_norm.forward(stream, self.dtype)     # nothing pending: the same x
        a = self.mixer.forward(h1, ctx, cache)
        f = self.feed_forward.forward(h2, ctx)
        stream.push(a)
        stream.push(f)


# ------------------------------------------------------------ a toy mixer with its own state
class ToyEma(Mixer):
    """y_t = (s_t) W^T with s_t = 0.75 s_{t-1} + 0.25 x_t, s kept per request between steps.
    Written as a loop over requests on the host, so it says so: its model runs every step eagerly."""

    needs_host_metadata = True

    def __init__(self, hidden_size, prefix="mix.", position=None):
        self.hidden_size, self.prefix, self.position = hidden_size, prefix, position

    def cache_need(self):
        return FixedState((self.hidden_size,), torch.float32)

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}proj.weight", (self.hidden_size, self.hidden_size))]

    def bind(self, source, dtype, device):
        self.w = source.get(f"{self.prefix}proj.weight").to(device=device, dtype=torch.float32)
        self.dtype = dtype

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        for r in range(ctx.num_requests):
            a, b = ctx.host_cu_tokens[r], ctx.host_cu_tokens[r + 1]
            s = cache.state[ctx.host_state_slots[r]]
            rows = []
            for t in range(a, b):
                xt = x[t].float()
                if self.position is not None:        # another position encoding: a gain by position
                    xt = xt * self.position.table[ctx.host_start_pos[r] + (t - a)]
                s = 0.75 * s + 0.25 * xt
                rows.append(s)
            if cache.write:
                cache.state[ctx.host_state_slots[r]] = s
            out[a:b] = (torch.stack(rows) @ self.w.t()).to(x.dtype)
        return out


class ToyEmaDevice(ToyEma):
    """The same mixer computed from the step's device tensors alone (no loop over requests on the host):
    decode steps of its model replay as CUDA graphs like any other model's."""

    needs_host_metadata = False

    def forward(self, x, ctx, cache):
        T, R = ctx.num_tokens, ctx.num_requests
        slots = ctx.state_slots.long()
        cu = ctx.cu_tokens.long()
        s = cache.state[slots]                                   # [R, D]
        rows = torch.zeros((T + 1, x.shape[1]), dtype=torch.float32, device=x.device)   # row T: for nobody
        xf = x.float()
        for j in range(ctx.max_portion):                        # token j of every request that has one
            idx = cu[:-1] + j
            valid = idx < cu[1:]
            xt = xf[idx.clamp(max=T - 1)]
            if self.position is not None:
                xt = xt * self.position.table[(ctx.start_pos.long() + j).clamp(max=self.position.table.numel() - 1)][:, None]
            s = torch.where(valid[:, None], 0.75 * s + 0.25 * xt, s)
            rows.index_put_((torch.where(valid, idx, torch.full_like(idx, T)),), s)
        if cache.write:
            cache.state.index_put_((slots,), s)
        return (rows[:T] @ self.w.t()).to(x.dtype)


# ------------------------------------------------------------ another position encoding
def gain_table(n, period):
    return 1.0 + 0.5 * torch.sin(torch.arange(n, dtype=torch.float64) / period)


class ToyGain(PositionEncoding):
    """Not a rotation: a table of gains by position that the toy mixer multiplies its input with."""

    def __init__(self, period):
        self.period = period
        self.table = None

    def prepare(self, max_positions, device):
        self.table = gain_table(max_positions, self.period).to(torch.float32).to(device)


# ------------------------------------------------------------ a toy feed-forward with routing
class ToyRouted(FeedForward):
    """Every token goes to the expert with the largest router logit (float32): y = relu(x W1_e^T) W2_e^T."""

    def __init__(self, hidden_size, expert_size, num_experts, prefix="moe."):
        self.D, self.E, self.n, self.prefix = hidden_size, expert_size, num_experts, prefix

    def tensor_specs(self):
        specs = [TensorSpec(f"{self.prefix}router.weight", (self.n, self.D))]
        for e in range(self.n):
            specs += [TensorSpec(f"{self.prefix}experts.{e}.w1.weight", (self.E, self.D)),
                      TensorSpec(f"{self.prefix}experts.{e}.w2.weight", (self.D, self.E))]
        return specs

    def bind(self, source, dtype, device):
        get = lambda n: source.get(self.prefix + n).to(device=device, dtype=torch.float32)
        self.router = get("router.weight")
        self.w1 = [get(f"experts.{e}.w1.weight") for e in range(self.n)]
        self.w2 = [get(f"experts.{e}.w2.weight") for e in range(self.n)]

    def forward(self, x, ctx):
        xf = x.float()
        choice = (xf @ self.router.t()).argmax(-1)
        out = torch.zeros_like(xf)
        for e in range(self.n):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                out[rows] = torch.relu(xf[rows] @ self.w1[e].t()) @ self.w2[e].t()
        return out.to(x.dtype)


@pytest.fixture(scope="module", autouse=True)
def toy_registration():
    register_part("mixer", "toy_ema")(ToyEma)
    register_part("mixer", "toy_ema_device")(ToyEmaDevice)
    register_part("block", "toy_parallel")(ToyParallelBlock)
    register_part("position", "toy_gain")(ToyGain)
    register_part("feed_forward", "toy_routed")(ToyRouted)
    register_architecture("ToyLM", ToyConfig, describe_toy)
    yield
    unregister_architecture("ToyLM")
    unregister_part("mixer", "toy_ema")
    unregister_part("mixer", "toy_ema_device")
    unregister_part("block", "toy_parallel")
    unregister_part("position", "toy_gain")
    unregister_part("feed_forward", "toy_routed")


# ------------------------------------------------------------ plain forward of the toy models
def toy_plain(cfg: ToyConfig, w, tokens):
    x = plain_model.embedding(w["model.embed_tokens.weight"], tokens)
    T = len(tokens)
    positions = torch.arange(T)
    sched = cfg.schedule or tuple((i, -1) for i in range(len(cfg.kinds)))
    kv_of = {}
    for e, (l, src) in enumerate(sched):
        p = f"model.layers.{l}."
        h = plain_model.rmsnorm(x, w[p + "input_layernorm.weight"], cfg.eps)
        kind = cfg.kinds[l]
        if kind in ("ema", "ema_gain", "ema_dev"):
            s = torch.zeros(cfg.hidden_size, dtype=torch.float64)
            gain = gain_table(T, cfg.gain_period) if kind == "ema_gain" else torch.ones(T, dtype=torch.float64)
            rows = []
            for t in range(T):
                s = 0.75 * s + 0.25 * h[t] * gain[t]
                rows.append(s)
            a = torch.stack(rows) @ w[p + "mix.proj.weight"].t()
        else:
            H, G, d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
            lin = lambda n: plain_model.linear(h, w[f"{p}self_attn.{n}_proj.weight"], w[f"{p}self_attn.{n}_proj.bias"])
            q = plain_model.rope(lin("q"), positions, H, d, cfg.rope_base)
            if src >= 0:
                k, v = kv_of[src]                       # this run reads what run ``src`` cached
            else:
                k, v = plain_model.rope(lin("k"), positions, G, d, cfg.rope_base), lin("v")
                kv_of[e] = (k, v)
            a = plain_model.attention(q, k, v, H, G, d, cfg.window if kind == "window" else None)
            a = plain_model.linear(a, w[p + "self_attn.o_proj.weight"])
        h = plain_model.rmsnorm(x if cfg.block == "toy_parallel" else x + a,
                                w[p + "post_attention_layernorm.weight"], cfg.eps)
        x = x + a
        if l in cfg.routed_layers:
            choice = (h @ w[p + "moe.router.weight"].t()).argmax(-1)
            y = torch.zeros_like(h)
            for t in range(T):
                e = int(choice[t])
                y[t] = torch.relu(h[t] @ w[f"{p}moe.experts.{e}.w1.weight"].t()) @ w[f"{p}moe.experts.{e}.w2.weight"].t()
            x = x + y
        else:
            x = x + plain_model.swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                           w[p + "mlp.down_proj.weight"])
    return plain_model.linear(plain_model.rmsnorm(x, w["model.norm.weight"], cfg.eps), w["lm_head.weight"])


def run_all_cuttings(cfg, tmp_path, dtype, lengths=(7, 45, 101, 160)):
    from qwen_decoder_b200.engine import ModelRunner
    folder = write_random_model(cfg, str(tmp_path / "model"), seed=11)
    _, w = plain_model.read_folder(folder)
    rng = random.Random(3)
    seqs = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lengths]
    want = [toy_plain(cfg, w, s).numpy() for s in seqs]
    max_tokens = 2 * 192
    for i, make in enumerate([trace_tools.whole, trace_tools.decode_tail, trace_tools.portions,
                              lambda s: trace_tools.mixed(s + s[::-1], max_tokens, seed=5)]):
        runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", num_pages=max_tokens // 16,
                                         page_size=16, max_requests=8)
        tr = make(seqs)
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"out{i}"))
        trace_tools.compare(tr, got, want + want[::-1] if i == 3 else want, TOL[dtype])
        runner.cache.check()
        assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.pools)
    return runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_and_full_layers_in_one_model(tmp_path, dtype):
    cfg = ToyConfig("ToyLM", kinds=("window", "full", "window"))
    runner = run_all_cuttings(cfg, tmp_path, dtype)
    assert len(runner.cache.pools) == 2           # the windowed layers have pages of their own


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_pages_are_given_back_while_a_request_runs(tmp_path, dtype):
    from qwen_decoder_b200.engine import ModelRunner, StepEntry
    cfg = ToyConfig("ToyLM", kinds=("window", "full"))
    folder = write_random_model(cfg, str(tmp_path / "model"), seed=11)
    runner = ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", num_pages=16, max_requests=2)
    rc = runner.open("r")
    runner.step([StepEntry(rc, list(range(100)), [])])
    full, win = (runner.cache.pools[g] for g in range(2))
    by_window = {runner.cache.layout.groups[g].need.window: runner.cache.pools[g] for g in range(2)}
    assert by_window[None].num_used == 7 and by_window[20].num_used == 2      # tokens 81..99 need pages 5, 6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_named_twice_and_a_run_that_reads_another_runs_cache(tmp_path, dtype):
    # runs: layer 0, layer 1, layer 0 again (a cache of its own), layer 1 again reading run 1's cache
    cfg = ToyConfig("ToyLM", kinds=("full", "full"), schedule=((0, -1), (1, -1), (0, -1), (1, 1)))
    runner = run_all_cuttings(cfg, tmp_path, dtype)
    assert runner.cache.kv[0].shape[0] == 3       # three runs own a cache layer, the fourth owns none


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_with_state_of_its_own(tmp_path, dtype):
    cfg = ToyConfig("ToyLM", kinds=("ema", "full", "ema"))
    runner = run_all_cuttings(cfg, tmp_path, dtype)
    # a slot per request and one for the rows that pad a batch
    assert len(runner.cache.states) == 2 and runner.cache.states[0].shape == (8 + 1, 48)
    assert not runner.use_graphs and not runner._graphs        # its forward loops over requests on the host


def test_a_toy_feed_forward_with_routing(tmp_path):
    """A routed feed-forward in some layers, defined and registered in this file: built, bound, stepped and
    cut every way like the rest.  In float32 only: in bfloat16 a near tie of two router logits sends a token
    to another expert than the plain implementation's, which is no fault of the engine."""
    cfg = ToyConfig("ToyLM", kinds=("ema", "full", "window"), routed_layers=(0, 2))
    runner = run_all_cuttings(cfg, tmp_path, "float32")
    model = runner.model
    assert type(model.layers[0].feed_forward).__name__ == "ToyRouted"
    assert type(model.layers[1].feed_forward).__name__ == "SwiGLU"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_position_encoding(tmp_path, dtype):
    """A position encoding that is no rotation (a table of gains the toy mixer uses), registered here and
    named by the layer's configuration like the rotary one."""
    cfg = ToyConfig("ToyLM", kinds=("ema_gain", "full", "ema_gain"))
    runner = run_all_cuttings(cfg, tmp_path, dtype)
    model = runner.model
    assert type(model.positions["gain"]).__name__ == "ToyGain"
    assert model.layers[0].mixer.position is model.positions["gain"] and model.layers[1].mixer.position is model.positions["rope"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_with_state_replays_as_graphs_when_it_works_on_the_device(tmp_path, dtype):
    """The same toy mixer written with device tensors only: batches of single tokens run as replayed CUDA
    graphs (padded batches too: the padding rows use the state slot that belongs to no request), and every
    way of cutting gives the plain implementation's logits."""
    cfg = ToyConfig("ToyLM", kinds=("ema_dev", "full", "ema_dev"))
    runner = run_all_cuttings(cfg, tmp_path, dtype)
    assert runner.use_graphs and runner._graphs
    assert any(g.lay.T > 1 for g in runner._graphs.values())           # the mixed trace decodes several at once
    assert 3 in {len(s["entries"]) for s in trace_tools.mixed([[1] * 40] * 6, 384, seed=5).steps}


def test_another_order_of_the_same_parts_keeps_the_parts_path(tmp_path):
    """A block with the pre-norm block's parts and tensor names in another order (both branches read the same
    x): the native prompt loop, which restates the pre-norm order, must decline it, and the logits are the
    plain implementation's."""
    cfg = ToyConfig("ToyLM", kinds=("full", "full"), block="toy_parallel")
    runner = run_all_cuttings(cfg, tmp_path, "bfloat16")
    assert runner.model.native_prompt is None
    from qwen_decoder_b200.engine import ModelRunner
    usual = ModelRunner.from_folder(str(tmp_path / "model"), dtype="bfloat16", device="cuda:0", num_pages=8)
    assert type(usual.model.layers[0]).__name__ == "ToyParallelBlock"
    plain_cfg = ToyConfig("ToyLM", kinds=("full", "full"))
    folder = write_random_model(plain_cfg, str(tmp_path / "prenorm"), seed=11)
    if os.environ.get("QD_NATIVE_PROMPT", "1") != "0":          # the switch takes the native loop away from every model
        assert ModelRunner.from_folder(folder, dtype="bfloat16", device="cuda:0", num_pages=8).model.native_prompt is not None
