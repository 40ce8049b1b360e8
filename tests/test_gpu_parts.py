"""Each part alone against the plain formulas, and the generality of their arrangement: a toy
architecture, defined here, with a mixer that keeps fixed-size state of its own, a layer that runs
twice, a layer that reads another layer's cache and a windowed attention layer -- registered, built
and stepped without a change to the package."""
import json
from dataclasses import dataclass

import pytest
import torch

import plain_llama as P
from conftest import TINY, assert_close_logits, make_model_dir, plain_inputs
from gpullama3.java_b200.cache import KVCacheNeed, SequenceCache, StateNeed
from gpullama3.java_b200.config import (LayerSpec, LlamaConfig, PartSpec, ScheduleEntry, register_architecture,
                                        unregister_architecture)
from gpullama3.java_b200.parts import (GroupedQueryAttention, Mixer, OutputHead, PreNormBlock, RMSNorm,
                                       RotaryPositionEncoding, SwiGLUFeedForward, TokenEmbedding, register_mixer,
                                       unregister)
from gpullama3.java_b200.weights import ParamSpec

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ctx(cache, dtype, slots, token_lists):
    from gpullama3.java_b200.engine.step import build_context
    start = [cache.length(s) for s in slots]
    cache.reserve([(s, len(t)) for s, t in zip(slots, token_lists)])
    ctx, _ = build_context(dtype, torch.device(DEV), cache, slots, start, token_lists, [])
    return ctx


def _close(got, ref, dtype):
    scale = float(ref.abs().max())
    if dtype == torch.float32:
        torch.testing.assert_close(got.float().cpu(), ref, rtol=0, atol=2e-5 * scale)
    else:
        torch.testing.assert_close(got.float().cpu(), ref, rtol=0, atol=2.0 ** -6 * scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype, w_dtype):
    n = RMSNorm(dim=100, eps=1e-3)
    assert n.parameters()["weight"].shape == (100,)
    w = (1 + 0.2 * torch.randn(100)).to(w_dtype)
    n.load({"weight": w}, dtype, DEV)
    assert n.weight.dtype == (torch.float32 if (dtype == torch.float32 or w_dtype == torch.float32) else torch.bfloat16)
    x = torch.randn(5, 100) * 4
    out = n.forward(x.to(DEV), dtype)
    assert out.dtype == dtype
    _close(out, P.rmsnorm(x, w.float(), 1e-3), dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_rotary_frequencies(name):
    cfg = TINY[name][0]
    r = RotaryPositionEncoding(cfg["head_dim"], cfg["rope_theta"], "half", cfg["rope_scaling"])
    ours = r.inverse_frequencies(DEV).cpu()
    ref = P.rope_inverse_frequencies(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"]).to(torch.float32)
    assert torch.equal(ours, ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, KVH, D, hidden, pairing, window", [(4, 2, 16, 72, "half", None), (3, 1, 32, 40, "interleaved", None),
                                                                (6, 2, 48, 100, "half", 50)])
def test_attention_part_alone(dtype, H, KVH, D, hidden, pairing, window):
    rope = RotaryPositionEncoding(D, 1e4, pairing)
    att = GroupedQueryAttention(hidden, H, KVH, D, rope, window)
    specs = att.parameters()
    assert specs["q"].shape == (H * D, hidden) and specs["k"].shape == (KVH * D, hidden) and specs["o"].shape == (hidden, H * D)
    assert att.cache_need() == KVCacheNeed(KVH, D, window)
    g = torch.Generator().manual_seed(H)
    w = {k: (torch.randn(s.shape, generator=g) * 0.2).to(torch.bfloat16) for k, s in specs.items()}
    att.load(w, dtype, DEV)
    cache = SequenceCache({0: att.cache_need()}, max_tokens=64 * 8, dtype=dtype, device=DEV, window_slack=128)
    lens = [70, 5, 128]
    xs = [torch.randn(n, hidden, generator=g).to(dtype).float() for n in lens]
    slots = [cache.acquire() for _ in lens]
    ctx = _ctx(cache, dtype, slots, [[0] * n for n in lens])
    residual = torch.zeros(sum(lens), hidden, device=DEV)
    att.forward(torch.cat(xs).to(dtype).to(DEV), ctx, cache.view(0), residual)
    rt = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(torch.bfloat16).float())
    refs = []
    for x in xs:
        T = x.shape[0]
        q = rt(P.linear(x, w["q"].float())).view(T, H, D)
        k = rt(P.linear(x, w["k"].float())).view(T, KVH, D)
        v = rt(P.linear(x, w["v"].float())).view(T, KVH, D)
        cos, sin = P.rope_tables(torch.arange(T), P.rope_inverse_frequencies(D, 1e4, None), torch.float32)
        q, k = rt(P.apply_rope(q, cos, sin, pairing)), rt(P.apply_rope(k, cos, sin, pairing))
        a = rt(P.causal_attention(q, k, v, window)).reshape(T, H * D)
        refs.append(P.linear(a, w["o"].float()))
    _close(residual, torch.cat(refs), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part_alone(dtype):
    ff = SwiGLUFeedForward(hidden_size=72, intermediate_size=200)
    g = torch.Generator().manual_seed(2)
    w = {k: (torch.randn(s.shape, generator=g) * 0.2).to(torch.bfloat16) for k, s in ff.parameters().items()}
    ff.load(w, dtype, DEV)
    assert tuple(ff.gate_up.weight.shape) == (400, 72)
    assert torch.equal(ff.gate_up.weight[0::2].float().cpu(), w["gate"].float())     # rows interleaved gate, up
    x = torch.randn(9, 72, generator=g).to(dtype).float()
    residual0 = torch.randn(9, 72, generator=g)
    residual = residual0.clone().to(DEV)
    ff.forward(x.to(dtype).to(DEV), None if False else _Dummy(dtype), residual)
    rt = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(torch.bfloat16).float())
    h = rt(P.swiglu(P.linear(x, w["gate"].float()), P.linear(x, w["up"].float())))
    _close(residual, residual0 + P.linear(h, w["down"].float()), dtype)


class _Dummy:
    """What the feed-forward asks of a step's context: the run's precision and where tensors come from."""

    def __init__(self, dtype):
        self.dtype = dtype

    def empty(self, shape, dtype):
        return torch.empty(tuple(shape), dtype=dtype, device=DEV)


@pytest.mark.parametrize("name", ["A", "B"])
def test_block_with_its_norms_left_to_the_products_around_them(tmp_path, name):
    """In a decode step the pre-norm block hands each norm to the products before and after it (ScaledRows).
    With that switched off in every part the same step runs the norm kernels; both give the same logits up to
    the rounding of a bfloat16 run, the launches differ by the two norms per layer, and a prompt step, which
    does not take that path, is not affected."""
    from gpullama3.java_b200.engine.api import Engine, SequenceInput
    from gpullama3.java_b200.kernels import ops

    cfg_json, norm_std = TINY[name]
    d = make_model_dir(tmp_path, cfg_json, seed=31, norm_std=norm_std)
    cfg, w = plain_inputs(d)
    engines = [Engine.from_folder(d, dtype="bfloat16", max_tokens=64 * 8, max_batch=4) for _ in range(2)]
    for e in engines:
        e.step_fn.use_graphs = False          # launches are counted as they are issued
    for block in engines[1].model.blocks:
        for part in (block, block.mixer, block.feed_forward):
            part.takes_scaled_rows = lambda ctx: False
    prompts = [[5, 9, 3], [7] * 40, [1, 2]]
    outs, launches = [], []
    for e in engines:
        slots = [e.cache.acquire() for _ in prompts]
        first = e.step([SequenceInput(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        before = ops.launch_count()
        second = e.step([SequenceInput(s, [11 + i], [0]) for i, s in enumerate(slots)])
        launches.append(ops.launch_count() - before)
        outs.append((first.float().cpu(), second.float().cpu()))
    assert torch.equal(outs[0][0], outs[1][0])
    n_layers = cfg["num_hidden_layers"]
    assert launches[1] - launches[0] == 2 * n_layers - 1   # every norm but the first layer's first one
    for i, p in enumerate(prompts):
        ref = P.forward(cfg, w, p + [11 + i], round_to=torch.bfloat16)[-1]
        assert_close_logits(outs[0][1][i], ref, torch.bfloat16)
        assert_close_logits(outs[1][1][i], ref, torch.bfloat16)


def test_embedding_and_tied_head_share_memory():
    emb = TokenEmbedding(50, 24)
    table = torch.randn(50, 24).to(torch.bfloat16)
    emb.load({"table": table}, torch.bfloat16, DEV)
    head = OutputHead(50, 24, tied_to=emb)
    assert head.parameters() == {}
    head.load({}, torch.bfloat16, DEV)
    assert head.linear.weight.data_ptr() == emb.table.data_ptr()
    toks = torch.tensor([3, 49, 0], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(toks).cpu(), table.float()[[3, 49, 0]])
    x = torch.randn(2, 24).to(torch.bfloat16)
    logits = head.forward(x.to(DEV))
    assert logits.dtype == torch.float32
    _close(logits, x.float() @ table.float().t(), torch.float32)
    assert OutputHead(50, 24).parameters()["weight"].shape == (50, 24)


# --------------------------------------------------------------------------- a toy architecture
class RunningMeanMixer(Mixer):
    """Toy mixer with fixed-size state: adds proj(mean of the inputs seen so far).  Its state per
    sequence is the running sum and the count; it keeps no keys or values."""

    def __init__(self, hidden_size: int):
        self.h = hidden_size

    def parameters(self):
        return {"proj": ParamSpec((self.h, self.h))}

    def cache_need(self):
        return StateNeed((self.h + 1,), torch.float32)

    def load(self, tensors, dtype, device):
        self.proj = tensors["proj"].to(device=device, dtype=torch.float32)

    def forward(self, x, ctx, cache, residual, writes_cache=True):
        off = 0
        for slot, n in zip(ctx.slots, ctx.q_lens):
            st = cache.data[slot]
            csum = st[: self.h] + torch.cumsum(x[off:off + n].float(), 0)
            cnt = st[self.h] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
            residual[off:off + n] += (csum / cnt[:, None]) @ self.proj.t()
            if writes_cache:
                st[: self.h] = csum[-1]
                st[self.h] = cnt[-1]
            off += n


@dataclass(frozen=True)
class ToyConfig(LlamaConfig):
    """Layers: 0 attention, 1 running mean, 2 attention with a window, 3 attention that keeps
    nothing of its own.  Schedule: 0, 1, 0 again (a second cache entry), 2, 3 reading layer 0's first
    cache."""
    architecture = "ToyStateForCausalLM"
    window: int = 40

    def layer_specs(self):
        base = super().layer_specs()[0]
        toy = base.with_parts(mixer=PartSpec("mixer", "test_running_mean", {"hidden_size": self.hidden_size}))
        windowed = base.with_parts(mixer=base.parts["mixer"].with_args(window=self.window))
        return [base, toy, windowed, base]

    def schedule(self):
        return [ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(2, 3),
                ScheduleEntry(3, 0, writes_cache=False)]

    def tensor_names(self):
        names = {"embedding.table": "tok.weight", "final_norm.weight": "out_norm.weight", "head.weight": "out.weight"}
        for i, kind in enumerate(["att", "mean", "att", "att"]):
            p, c = f"layers.{i}.", f"blk.{i}."
            names[p + "mixer_norm.weight"] = c + "norm1"
            names[p + "feed_forward_norm.weight"] = c + "norm2"
            for w in ("gate", "up", "down"):
                names[p + f"feed_forward.{w}"] = c + f"ffn_{w}"
            if kind == "att":
                for w in ("q", "k", "v", "o"):
                    names[p + f"mixer.{w}"] = c + f"attn_{w}"
            else:
                names[p + "mixer.proj"] = c + "mean_proj"
        return names


TOY = dict(TINY["A"][0], architectures=["ToyStateForCausalLM"], num_hidden_layers=4, tie_word_embeddings=False)


def plain_toy_forward(cfg, w, tokens, window, rt=lambda t: t):
    """The toy architecture written out with the plain functions, whole sequence, no cache.  ``rt`` rounds where
    the engine stores activations in its run precision (after a norm, a projection, the rotation, attention and
    the gated activation)."""
    T = len(tokens)
    H, KVH, D, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    cos, sin = P.rope_tables(torch.arange(T), P.rope_inverse_frequencies(D, cfg["rope_theta"], None), torch.float32)
    x = P.embedding(w["tok.weight"], torch.tensor(tokens))

    def kv(i, xb):
        k = rt(P.apply_rope(rt(P.linear(xb, w[f"blk.{i}.attn_k"])).view(T, KVH, D), cos, sin, "half"))
        return k, rt(P.linear(xb, w[f"blk.{i}.attn_v"])).view(T, KVH, D)

    def attend(i, xb, k, v, win):
        q = rt(P.apply_rope(rt(P.linear(xb, w[f"blk.{i}.attn_q"])).view(T, H, D), cos, sin, "half"))
        return P.linear(rt(P.causal_attention(q, k, v, win)).reshape(T, H * D), w[f"blk.{i}.attn_o"])

    def ffn(i, x):
        xb = rt(P.rmsnorm(x, w[f"blk.{i}.norm2"], eps))
        return x + P.linear(rt(P.swiglu(P.linear(xb, w[f"blk.{i}.ffn_gate"]), P.linear(xb, w[f"blk.{i}.ffn_up"]))),
                            w[f"blk.{i}.ffn_down"])

    xb = rt(P.rmsnorm(x, w["blk.0.norm1"], eps))
    k0, v0 = kv(0, xb)                                   # what cache entry 0 holds
    x = ffn(0, x + attend(0, xb, k0, v0, None))
    xb = rt(P.rmsnorm(x, w["blk.1.norm1"], eps))
    mean = torch.cumsum(xb, 0) / torch.arange(1, T + 1)[:, None]
    x = ffn(1, x + mean @ w["blk.1.mean_proj"].t())
    xb = rt(P.rmsnorm(x, w["blk.0.norm1"], eps))             # layer 0 again, with keys of its own
    x = ffn(0, x + attend(0, xb, *kv(0, xb), None))
    xb = rt(P.rmsnorm(x, w["blk.2.norm1"], eps))
    x = ffn(2, x + attend(2, xb, *kv(2, xb), window))
    xb = rt(P.rmsnorm(x, w["blk.3.norm1"], eps))             # reads what layer 0's first run cached
    x = ffn(3, x + attend(3, xb, k0, v0, None))
    return P.linear(rt(P.rmsnorm(x, w["out_norm.weight"], eps)), w["out.weight"])


@pytest.fixture()
def toy_registered():
    register_mixer("test_running_mean", RunningMeanMixer)
    register_architecture("ToyStateForCausalLM", ToyConfig)
    yield
    unregister("mixer", "test_running_mean")
    unregister_architecture("ToyStateForCausalLM")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_architecture_with_state_is_registered_built_and_stepped(toy_registered, tmp_path, dtype):
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    d = make_model_dir(tmp_path, TOY, seed=6, scale={"attn_q": 8.0, "attn_k": 8.0})
    cfg, w = plain_inputs(d)
    model = load_model(d, dtype)
    needs = model.cache_needs()
    assert needs[1] == StateNeed((65,), torch.float32) and needs[3] == KVCacheNeed(2, 16, 40)
    assert needs[0] == needs[2] == KVCacheNeed(2, 16, None) and set(needs) == {0, 1, 2, 3}
    cache = model.new_cache(64 * 12, max_slots=3, window_slack=256)
    assert len(cache.paged_groups) == 2 and len(cache.slot_groups) == 1
    step = StepFunction(model, cache)
    prompts = [torch.randint(0, 256, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (150, 70, 9)]

    # whole prompts together, then again as a prefix in one step plus the rest token by token
    slots = [cache.acquire() for _ in prompts]
    whole = step([SequenceInput(s, p, list(range(len(p)))) for s, p in zip(slots, prompts)])
    for s in slots:
        cache.release(s)
    slots = [cache.acquire() for _ in prompts]           # the same slots again: state must start from zero
    heads = [max(1, len(p) - 20) for p in prompts]
    first = step([SequenceInput(s, p[:h], [h - 1]) for s, p, h in zip(slots, prompts, heads)])
    tails = {i: [first[i]] for i in range(3)}
    for t in range(20):
        live = [i for i in range(3) if heads[i] + t < len(prompts[i])]
        if not live:
            break
        out = step([SequenceInput(slots[i], [prompts[i][heads[i] + t]], [0]) for i in live])
        for j, i in enumerate(live):
            tails[i].append(out[j])
    cache.check_invariants()
    off = 0
    for i, p in enumerate(prompts):
        rt = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(torch.bfloat16).float())
        ref = plain_toy_forward(cfg, w, p, 40, rt)
        got_whole = whole[off:off + len(p)]
        off += len(p)
        assert_close_logits(got_whole, ref, dtype, f"toy whole {i}")
        assert_close_logits(torch.stack(tails[i]), ref[heads[i] - 1:], dtype, f"toy stepped {i}")


def test_schedule_mistakes_are_refused(toy_registered):
    from gpullama3.java_b200.config import ConfigError, config_from_dict
    from gpullama3.java_b200.engine.model import CausalLM

    class Bad(ToyConfig):
        def schedule(self):
            return [ScheduleEntry(3, 0, writes_cache=False), ScheduleEntry(0, 0)]   # read before any write
    with pytest.raises(ConfigError, match="before any entry writes"):
        CausalLM(Bad.from_dict(TOY), torch.float32, "cpu")

    class Bad2(ToyConfig):
        def schedule(self):
            return [ScheduleEntry(0, 0), ScheduleEntry(2, 0, writes_cache=False)]   # window differs from cache 0's
    with pytest.raises(ConfigError, match="different needs"):
        CausalLM(Bad2.from_dict(TOY), torch.float32, "cpu")


# --------------------------------------------------------------------------- a second toy architecture
class Top1ExpertsFeedForward(__import__("gpullama3.java_b200.parts", fromlist=["FeedForward"]).FeedForward):
    """Toy feed-forward with routing: router logits in float32, each token goes to its best expert (a small
    gated feed-forward), the expert's output is weighted by the router's softmax probability."""

    def __init__(self, hidden_size: int, intermediate_size: int, n_experts: int):
        self.h, self.i, self.e = hidden_size, intermediate_size, n_experts

    def parameters(self):
        p = {"router": ParamSpec((self.e, self.h))}
        for k in range(self.e):
            p[f"gate{k}"] = ParamSpec((self.i, self.h))
            p[f"up{k}"] = ParamSpec((self.i, self.h))
            p[f"down{k}"] = ParamSpec((self.h, self.i))
        return p

    def load(self, tensors, dtype, device):
        from gpullama3.java_b200.parts import Linear
        wd = torch.float32 if dtype == torch.float32 else torch.bfloat16
        self.router = tensors["router"].to(device=device, dtype=torch.float32)
        self.gate_up = [Linear(torch.stack([tensors[f"gate{k}"], tensors[f"up{k}"]], 1).reshape(2 * self.i, self.h)
                               .to(device=device, dtype=wd).contiguous()) for k in range(self.e)]
        self.down = [Linear(tensors[f"down{k}"].to(device=device, dtype=wd).contiguous()) for k in range(self.e)]

    def forward(self, x, ctx, residual):
        probs = torch.softmax(x.float() @ self.router.t(), dim=-1)      # router in 32-bit
        weight, expert = probs.max(dim=-1)
        for k in range(self.e):
            rows = (expert == k).nonzero().flatten()
            if rows.numel() == 0:
                continue
            h = self.gate_up[k].gated_silu(x[rows].contiguous(), ctx.dtype)
            y = self.down[k].store(h, torch.float32)
            residual.index_add_(0, rows, y * weight[rows, None])


class HalfRotaryLinearScaling(__import__("gpullama3.java_b200.parts", fromlist=["PositionEncoding"]).PositionEncoding):
    """Toy position encoding: only the first half of a head is rotated, interleaved pairs, frequencies
    theta^(-i/rotary_dim) divided by a constant factor."""

    def __init__(self, head_dim: int, theta: float, factor: float):
        self.rotary_dim, self.pairing = head_dim // 2, 0
        self.theta, self.factor = theta, factor
        self._cache = {}

    def inverse_frequencies(self, device):
        if str(device) not in self._cache:
            f = [1.0 / (self.theta ** (i / self.rotary_dim)) / self.factor for i in range(0, self.rotary_dim, 2)]
            self._cache[str(device)] = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device)
        return self._cache[str(device)]


@dataclass(frozen=True)
class ToyRoutedConfig(LlamaConfig):
    architecture = "ToyRoutedForCausalLM"
    n_experts: int = 3
    rope_factor: float = 4.0

    def layer_specs(self):
        base = super().layer_specs()[0]
        pos = PartSpec("position", "test_half_rotary", {"head_dim": self.head_dim, "theta": self.rope_theta,
                                                        "factor": self.rope_factor})
        ff = PartSpec("feed_forward", "test_top1_experts", {"hidden_size": self.hidden_size,
                                                            "intermediate_size": self.intermediate_size,
                                                            "n_experts": self.n_experts})
        layer = base.with_parts(mixer=base.parts["mixer"].with_args(position=pos), feed_forward=ff)
        return [layer for _ in range(self.num_hidden_layers)]

    def tensor_names(self):
        names = {"embedding.table": "wte", "final_norm.weight": "ln_f", "head.weight": "head"}
        for i in range(self.num_hidden_layers):
            p, c = f"layers.{i}.", f"h.{i}."
            names[p + "mixer_norm.weight"] = c + "ln1"
            names[p + "feed_forward_norm.weight"] = c + "ln2"
            for w in ("q", "k", "v", "o"):
                names[p + f"mixer.{w}"] = c + w
            names[p + "feed_forward.router"] = c + "router"
            for k in range(self.n_experts):
                for w in ("gate", "up", "down"):
                    names[p + f"feed_forward.{w}{k}"] = c + f"expert{k}.{w}"
        return names


def plain_routed_forward(cfg, w, tokens, n_experts, rope_factor):
    T = len(tokens)
    H, KVH, D, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    R = D // 2
    inv = torch.tensor([1.0 / (cfg["rope_theta"] ** (i / R)) / rope_factor for i in range(0, R, 2)], dtype=torch.float64)
    cos, sin = P.rope_tables(torch.arange(T), inv, torch.float32)

    def rot(x):   # only the first half of each head turns
        return torch.cat([P.apply_rope(x[..., :R], cos, sin, "interleaved"), x[..., R:]], dim=-1)

    x = P.embedding(w["wte"], torch.tensor(tokens))
    for l in range(cfg["num_hidden_layers"]):
        c = f"h.{l}."
        xb = P.rmsnorm(x, w[c + "ln1"], eps)
        q = rot(P.linear(xb, w[c + "q"]).view(T, H, D))
        k = rot(P.linear(xb, w[c + "k"]).view(T, KVH, D))
        v = P.linear(xb, w[c + "v"]).view(T, KVH, D)
        x = x + P.linear(P.causal_attention(q, k, v).reshape(T, H * D), w[c + "o"])
        xb = P.rmsnorm(x, w[c + "ln2"], eps)
        probs = torch.softmax(xb @ w[c + "router"].t(), dim=-1)
        weight, expert = probs.max(dim=-1)
        y = torch.zeros_like(x)
        for t in range(T):
            e = int(expert[t])
            h = P.swiglu(P.linear(xb[t:t + 1], w[c + f"expert{e}.gate"]), P.linear(xb[t:t + 1], w[c + f"expert{e}.up"]))
            y[t] = weight[t] * P.linear(h, w[c + f"expert{e}.down"])[0]
        x = x + y
    return P.linear(P.rmsnorm(x, w["ln_f"], eps), w["head"])


def test_toy_feed_forward_with_routing_and_toy_position_encoding(tmp_path):
    """A feed-forward with a router and a position encoding of its own, both defined here, registered and
    used by a toy architecture: whole prompts and token-by-token decoding against a plain restatement."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model
    from gpullama3.java_b200.parts import register_feed_forward, register_position_encoding

    register_feed_forward("test_top1_experts", Top1ExpertsFeedForward)
    register_position_encoding("test_half_rotary", HalfRotaryLinearScaling)
    register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
    try:
        cfg_json = dict(TINY["B"][0], architectures=["ToyRoutedForCausalLM"], num_hidden_layers=2, rope_scaling=None)
        d = make_model_dir(tmp_path, cfg_json, seed=9, scale={".q": 6.0, ".k": 6.0, "router": 30.0})
        cfg, w = plain_inputs(d)
        model = load_model(d, torch.float32)
        assert not model.graph_safe                       # the routed feed-forward did not promise graph safety
        cache = model.new_cache(64 * 6)
        step = StepFunction(model, cache)
        prompts = [torch.randint(0, 384, (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (90, 33)]
        slots = [cache.acquire() for _ in prompts]
        heads = [len(p) - 10 for p in prompts]
        out = step([SequenceInput(s, p[:h], list(range(h))) for s, p, h in zip(slots, prompts, heads)])
        refs = [plain_routed_forward(cfg, w, p, 3, 4.0) for p in prompts]
        off = 0
        for i, h in enumerate(heads):
            assert_close_logits(out[off:off + h], refs[i][:h], torch.float32, f"routed toy prompt {i}")
            off += h
        for t in range(10):
            o = step([SequenceInput(s, [p[h + t]], [0]) for s, p, h in zip(slots, prompts, heads)])
            for i, h in enumerate(heads):
                assert_close_logits(o[i:i + 1], refs[i][h + t:h + t + 1], torch.float32, f"routed toy decode {t}")
        # bfloat16: the same model steps and gives finite logits close to the float32 ones
        m16 = load_model(d, torch.bfloat16)
        c16 = m16.new_cache(64 * 4)
        s16 = c16.acquire()
        o16 = StepFunction(m16, c16)([SequenceInput(s16, prompts[1], [len(prompts[1]) - 1])])
        assert torch.isfinite(o16).all()
        assert float((o16.cpu() - refs[1][-1:]).abs().max()) < 0.15 * float(refs[1].abs().max())
    finally:
        unregister("feed_forward", "test_top1_experts")
        unregister("position", "test_half_rotary")
        unregister_architecture("ToyRoutedForCausalLM")
