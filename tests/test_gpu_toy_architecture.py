"""A second toy architecture, defined here and registered from here, that needs three things the Llama 3 model
does not: a tied output head that the checkpoint stores again under a name of its own; a layer without a
feed-forward whose mixer output passes a norm before it joins the residual stream (a block with other parts than
the pre-norm block's); and a mixer that caches one short latent row per position, a need with a cache group class
of its own.  It is replayed whole, with the last 32 tokens one by one, and in batches of unequal lengths with the
smallest cache, in both precisions, against a plain restatement.  Nothing under the package knows of it."""
from dataclasses import dataclass

import pytest
import torch

import plain_llama as P
from conftest import TINY, assert_close_logits, make_model_dir, plain_inputs, random_prompts
from gpullama3.java_b200.cache import PagedGroup, register_cache_group, unregister_cache_group
from gpullama3.java_b200.config import LayerSpec, LlamaConfig, PartSpec, register_architecture, unregister_architecture
from gpullama3.java_b200.parts import Block, Mixer, register_block, register_mixer, unregister
from gpullama3.java_b200.weights import ParamSpec
from replay_helpers import (max_live_tokens, read_rows, run_in_process, trace_batches, trace_tail_one_by_one,
                            trace_whole)

pytestmark = pytest.mark.gpu


# --------------------------------------------------------------------------- the parts
@dataclass(frozen=True)
class LatentNeed:
    """One row of ``width`` float32 numbers per position."""
    width: int


@dataclass
class LatentView:
    group: int
    rows: torch.Tensor     # [n_pages, 64, width]


class LatentGroup(PagedGroup):
    def __init__(self, need, entries, sizes):
        super().__init__(need, entries, sizes)
        self.data = torch.full((len(self.entries), self.pool.n_pages, 64, need.width), float("nan"), device=sizes.device)

    def view(self, entry):
        return LatentView(self.index, self.data[self.entry_pos[entry]])

    def bytes_per_token(self):
        return 4 * len(self.entries) * self.need.width


class LatentAttention(Mixer):
    """Each position keeps c = down(x) (``width`` numbers); position t reads softmax_s<=t(query(x_t) . c_s) c_s
    and projects it up.  Written with torch operations over the pages its sequences hold."""

    def __init__(self, hidden_size: int, width: int):
        self.h, self.r = hidden_size, width

    def parameters(self):
        return {"down": ParamSpec((self.r, self.h)), "query": ParamSpec((self.r, self.h)), "up": ParamSpec((self.h, self.r))}

    def cache_need(self):
        return LatentNeed(self.r)

    def load(self, tensors, dtype, device):
        self.w = {k: t.to(device=device, dtype=torch.float32) for k, t in tensors.items()}

    def forward(self, x, ctx, cache, residual, writes_cache=True):
        assert writes_cache
        table = ctx.page_tables[cache.group].cpu()
        off = 0
        for i, (start, n) in enumerate(zip(ctx.start_pos, ctx.q_lens)):
            xs = x[off:off + n].float()
            c_new, q = xs @ self.w["down"].t(), xs @ self.w["query"].t()
            for j in range(n):                               # write the new rows where their positions live
                pos = start + j
                cache.rows[int(table[i, pos // 64]), pos % 64] = c_new[j]
            pages = table[i, : -(-(start + n) // 64)].long().to(x.device)
            c = cache.rows[pages].reshape(-1, self.r)[: start + n]          # every cached row of the sequence, in order
            scores = q @ c.t()
            t = torch.arange(start, start + n, device=x.device)[:, None]
            scores = scores.masked_fill(torch.arange(start + n, device=x.device)[None, :] > t, float("-inf"))
            residual[off:off + n] += (torch.softmax(scores, dim=-1) @ c) @ self.w["up"].t()
            off += n


class MixerThenNormBlock(Block):
    """x += after(mixer(before(x))): no feed-forward, and a norm on the mixer's output."""

    def __init__(self, before, mixer, after):
        super().__init__(before=before, mixer=mixer, after=after)

    def forward(self, residual, ctx, cache, writes_cache=True):
        x = self.before.forward(residual, ctx.dtype)
        y = torch.zeros_like(residual)
        self.mixer.forward(x, ctx, cache, y, writes_cache)
        residual += self.after.forward(y, torch.float32)


@dataclass(frozen=True)
class ToyLatentConfig(LlamaConfig):
    """Layer 0 and 2: the Llama block.  Layer 1: latent attention, then a norm, no feed-forward."""
    architecture = "ToyLatentForCausalLM"
    latent_width: int = 12

    def layer_specs(self):
        base = super().layer_specs()[0]
        norm = self.final_norm()
        latent = LayerSpec("test_mixer_then_norm", {
            "before": norm, "after": norm,
            "mixer": PartSpec("mixer", "test_latent_attention", {"hidden_size": self.hidden_size, "width": self.latent_width})})
        return [base, latent, base]

    def tensor_names(self):
        names = {"embedding.table": "tok", "final_norm.weight": "out_norm"}        # tied: the head is the table
        for i in (0, 2):
            p, c = f"layers.{i}.", f"blk{i}."
            names[p + "mixer_norm.weight"], names[p + "feed_forward_norm.weight"] = c + "n1", c + "n2"
            for w in ("q", "k", "v", "o"):
                names[p + f"mixer.{w}"] = c + w
            for w in ("gate", "up", "down"):
                names[p + f"feed_forward.{w}"] = c + "ff_" + w
        names.update({"layers.1.before.weight": "blk1.before", "layers.1.after.weight": "blk1.after",
                      "layers.1.mixer.down": "blk1.c_down", "layers.1.mixer.query": "blk1.c_query",
                      "layers.1.mixer.up": "blk1.c_up"})
        return names

    def optional_tensor_names(self):
        return {"out.weight"}      # this family's exporter writes the tied head a second time


def plain_latent_forward(cfg, w, tokens, rt):
    """The toy architecture with the plain functions, whole sequence, no cache; ``rt`` rounds where the engine
    stores activations in its run precision."""
    T = len(tokens)
    H, KVH, D, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    cos, sin = P.rope_tables(torch.arange(T), P.rope_inverse_frequencies(D, cfg["rope_theta"], None), torch.float32)
    x = P.embedding(w["tok"], torch.tensor(tokens))

    def llama_block(i, x):
        c = f"blk{i}."
        xb = rt(P.rmsnorm(x, w[c + "n1"], eps))
        q = rt(P.apply_rope(rt(P.linear(xb, w[c + "q"])).view(T, H, D), cos, sin, "half"))
        k = rt(P.apply_rope(rt(P.linear(xb, w[c + "k"])).view(T, KVH, D), cos, sin, "half"))
        v = rt(P.linear(xb, w[c + "v"])).view(T, KVH, D)
        x = x + P.linear(rt(P.causal_attention(q, k, v)).reshape(T, H * D), w[c + "o"])
        xb = rt(P.rmsnorm(x, w[c + "n2"], eps))
        h = rt(P.swiglu(P.linear(xb, w[c + "ff_gate"]), P.linear(xb, w[c + "ff_up"])))
        return x + P.linear(h, w[c + "ff_down"])

    x = llama_block(0, x)
    xb = rt(P.rmsnorm(x, w["blk1.before"], eps))
    c, q = xb @ w["blk1.c_down"].t(), xb @ w["blk1.c_query"].t()
    scores = (q @ c.t()).masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
    y = (torch.softmax(scores, dim=-1) @ c) @ w["blk1.c_up"].t()
    x = x + P.rmsnorm(y, w["blk1.after"], eps)
    x = llama_block(2, x)
    return P.linear(rt(P.rmsnorm(x, w["out_norm"], eps)), w["tok"])


@pytest.fixture(scope="module")
def toy(session_tmp):
    register_mixer("test_latent_attention", LatentAttention)
    register_block("test_mixer_then_norm", MixerThenNormBlock)
    register_cache_group(LatentNeed, LatentGroup)
    register_architecture("ToyLatentForCausalLM", ToyLatentConfig)
    try:
        cfg_json = dict(TINY["A"][0], architectures=["ToyLatentForCausalLM"], num_hidden_layers=3, max_position_embeddings=512)
        d = make_model_dir(session_tmp, cfg_json, seed=21, norm_std=0.1,
                           scale={".q": 8.0, ".k": 8.0, "c_query": 10.0, "c_down": 2.0})   # scores of a few units everywhere
        # the exporter's second copy of the tied head, under the family's own name
        from gpullama3.java_b200.weights import SafetensorsFile, write_safetensors
        stored = SafetensorsFile(d / "model.safetensors")
        tensors = {n: stored.tensor(n).clone() for n in stored.entries}
        if "out.weight" not in tensors:
            tensors["out.weight"] = tensors["tok"].clone()
            write_safetensors(d / "model.safetensors", tensors)
        cfg, w = plain_inputs(d)
        requests = {f"r{i}": p for i, p in enumerate(random_prompts(256, [33, 64, 65, 130, 40, 200, 70], seed=4))}
        yield d, cfg, w, requests, {}
    finally:
        unregister("mixer", "test_latent_attention")
        unregister("block", "test_mixer_then_norm")
        unregister_cache_group(LatentNeed)
        unregister_architecture("ToyLatentForCausalLM")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("cut", ["whole", "tail32", "batches3"])
def test_toy_latent_architecture_in_the_three_cuts(toy, tmp_path, dtype, cut):
    from gpullama3.java_b200.engine.trace import load_model

    d, cfg, w, requests, refs = toy
    rt = (lambda t: t) if dtype == torch.float32 else (lambda t: t.to(torch.bfloat16).float())
    if dtype not in refs:
        refs[dtype] = {r: plain_latent_forward(cfg, w, t, rt) for r, t in requests.items()}
    steps, rows = {"whole": trace_whole, "tail32": lambda r: trace_tail_one_by_one(r, 32),
                   "batches3": lambda r: trace_batches(r, 3)}[cut](requests)
    model = load_model(d, dtype)
    assert model.head.linear is not None and model.head.linear.weight.data_ptr() == model.embedding.table.data_ptr()
    needs = model.cache_needs()
    assert needs[1] == LatentNeed(12) and set(needs) == {0, 1, 2}
    assert "layers.1.after" in model.named_parts() and "layers.1.feed_forward" not in model.named_parts()
    assert not model.graph_safe                                  # the toy parts made no such promise
    run_in_process(model, steps, tmp_path, max_live_tokens(steps))      # checks that no page or slot is left held
    got = read_rows(tmp_path, rows, cfg["vocab_size"])
    by_req: dict = {}
    for (rid, pos), row in got.items():
        by_req.setdefault(rid, []).append((pos, row))
    for rid, items in by_req.items():
        items.sort()
        assert_close_logits(torch.stack([r for _, r in items]), refs[dtype][rid][[p for p, _ in items]], dtype,
                            f"toy latent {cut} request {rid}")


def test_an_unexpected_tensor_is_still_reported(toy, tmp_path):
    """Only the names the configuration declares optional may be stored without being read."""
    from gpullama3.java_b200.engine.trace import load_model
    from gpullama3.java_b200.weights import SafetensorsFile, WeightError, write_safetensors
    import shutil

    d = toy[0]
    other = tmp_path / "m"
    shutil.copytree(d, other)
    stored = SafetensorsFile(other / "model.safetensors")
    tensors = {n: stored.tensor(n).clone() for n in stored.entries}
    tensors["lm_head.weight"] = tensors["tok"].clone()           # the Llama family's name means nothing here
    write_safetensors(other / "model.safetensors", tensors)
    with pytest.raises(WeightError, match=r"unexpected \(1\): lm_head.weight"):
        load_model(other, torch.float32)
