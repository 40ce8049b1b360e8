"""Plain, slow Llama 3 written from the reference's formulas (CPU, whole sequences, no cache).

This file is the oracle of the test-suite.  It shares no code with the product
package: it reads ``config.json`` as a plain dict, takes weights as a dict of
tensors under their checkpoint names, and recomputes every position of a
sequence from scratch each time it is called.

It rests on the formulas of AskMyu/GPULlama3.java only: the reference is a Java
program whose model code imports the TornadoVM API even on its CPU path, and
neither a JDK nor those jars exist on the build machine, so the reference could
not be run to produce golden vectors.  Every function cites the reference file
and lines it restates (paths relative to
``src/main/java/org/beehive/gpullama3/``).

Two deliberate departures from the reference, both stated where they occur:
  * token ``i`` of a prompt sits at position ``i`` (the reference feeds BOS twice,
    ``model/llama/Llama.java:47`` with ``inference/InferenceEngine.java:291-317``);
  * the llama3 rope-scaling constants come from ``config.json`` instead of the
    constants fixed in ``model/loader/ModelLoader.java:235-239``.

``round_to`` emulates a reduced-precision engine: when it is ``torch.bfloat16``
the activations are rounded at the places where a bfloat16 engine stores them
(after a norm, after a projection, after the rotation, after attention, after
the gated activation).  Sums, softmax, norms, angles and the residual stream stay
in the working dtype (float32, or float64 with ``dtype=torch.float64``).
"""
from __future__ import annotations

import math

import numpy as np
import torch


def _round(x: torch.Tensor, round_to) -> torch.Tensor:
    if round_to is None:
        return x
    return x.to(round_to).to(x.dtype)


# --------------------------------------------------------------------------- position encoding
def rope_inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """``inference/operation/RoPE.java:14-28``: freq_i = 1/theta^(i/head_dim) for even i (double
    ``pow``, cast to float), then the Llama 3.1 wavelength rule in ``float`` arithmetic, restated
    with numpy float32 scalars so that each intermediate rounds as the Java ``float`` does."""
    f = np.float32
    out = []
    for i in range(0, head_dim, 2):
        freq = f(1.0 / math.pow(theta, i / float(head_dim)))
        if scaling is not None:
            scale = f(scaling["factor"])
            lo = f(scaling["low_freq_factor"])
            hi = f(scaling["high_freq_factor"])
            old = f(scaling["original_max_position_embeddings"])
            lo_wavelen = old / lo
            hi_wavelen = old / hi
            wavelen = f(2.0 * math.pi / float(freq))
            if wavelen < hi_wavelen:
                pass
            elif wavelen > lo_wavelen:
                freq = freq / scale
            else:
                smooth = (old / wavelen - lo) / (hi - lo)
                freq = (f(1.0) - smooth) * freq / scale + smooth * freq
            assert isinstance(freq, np.float32)
        out.append(float(freq))
    return torch.tensor(out, dtype=torch.float64)


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """``RoPE.java:30-32``: val = pos * freq in float32, then cos and sin.  [T, head_dim/2] each."""
    f = inv_freq.to(torch.float32)
    val = positions.to(torch.float32)[:, None] * f[None, :]
    val = val.to(torch.float64)
    return torch.cos(val).to(dtype), torch.sin(val).to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pairing: str) -> torch.Tensor:
    """``inference/InferenceCore.java:83-95``: rotate pairs of one head by the angle of the pair.
    x: [T, heads, head_dim].  ``interleaved`` pairs (2j, 2j+1) as the reference does; ``half``
    pairs (j, j + head_dim/2), the layout of checkpoints whose q/k rows were not permuted."""
    T, H, D = x.shape
    c = cos[:, None, :]
    s = sin[:, None, :]
    out = torch.empty_like(x)
    if pairing == "interleaved":
        v0 = x[..., 0::2]
        v1 = x[..., 1::2]
        out[..., 0::2] = v0 * c - v1 * s
        out[..., 1::2] = v0 * s + v1 * c
    elif pairing == "half":
        v0 = x[..., : D // 2]
        v1 = x[..., D // 2:]
        out[..., : D // 2] = v0 * c - v1 * s
        out[..., D // 2:] = v0 * s + v1 * c
    else:
        raise ValueError(pairing)
    return out


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """``InferenceCore.java:69``: x = E[token]; no scaling."""
    return table[tokens]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``InferenceCore.java:47-56``: ss = sum(x^2)/n + eps; out = w * (x / sqrt(ss))."""
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    ss = ss + eps
    r = 1.0 / torch.sqrt(ss)
    return weight * (r * x)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``core/model/tensor/FloatTensor.java:98-100``: out_i = sum_j W[i, j] x_j; no bias."""
    return x @ w.t()


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None) -> torch.Tensor:
    """``InferenceCore.java:106-145``: per query head h with kv head h // kv_mul: scores
    q.k / sqrt(head_dim) over t <= pos, softmax (max, exp, sum, divide:
    ``FloatTensor.java:211-219``), weighted sum of values.  q: [T, H, D]; k, v: [T, KVH, D].
    ``window`` (not in the reference's Llama) keeps only the last ``window`` keys."""
    T, H, D = q.shape
    KVH = k.shape[1]
    kv_mul = H // KVH
    out = torch.zeros_like(q)
    scale = math.sqrt(D)
    for h in range(H):
        g = h // kv_mul
        scores = (q[:, h, :] @ k[:, g, :].t()) / scale  # [T, T]
        pos = torch.arange(T, device=q.device)
        mask = pos[None, :] <= pos[:, None]
        if window is not None:
            mask = mask & (pos[None, :] > pos[:, None] - window)
        scores = scores.masked_fill(~mask, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``InferenceCore.java:163-166``: silu(g) * u with silu(g) = g / (1 + exp(-g))."""
    return (gate / (1.0 + torch.exp(-gate))) * up


# --------------------------------------------------------------------------- whole model
def forward(config: dict, weights: dict, tokens, *, dtype=torch.float32, round_to=None,
            pairing: str | None = None, window: int | None = None, device=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence, ``InferenceCore.java:58-180`` run for every
    position at once.  ``weights`` uses checkpoint names (``model.layers.0.self_attn.q_proj.weight``
    ...), the roles of ``model/loader/ModelLoader.java:265-303``.

    ``device``: where torch evaluates these same lines (default: where the weights are, the CPU in
    almost every test).  Tests at the layer sizes of the real models pass ``"cuda"`` so that a float64
    run over a thousand tokens takes seconds instead of minutes; reduced-precision matrix modes must be
    off there, which is checked."""
    if device is not None and torch.device(device).type == "cuda":
        assert not torch.backends.cuda.matmul.allow_tf32 and torch.get_float32_matmul_precision() == "highest"
        weights = {k: t.to(device) for k, t in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    if device is not None:
        tokens = tokens.to(device)
    T = tokens.numel()
    H = config["num_attention_heads"]
    KVH = config.get("num_key_value_heads", H)
    dim = config["hidden_size"]
    D = config.get("head_dim") or dim // H
    eps = config.get("rms_norm_eps", 1e-5)
    theta = config.get("rope_theta", 10000.0)
    scaling = config.get("rope_scaling")
    if scaling is not None and scaling.get("rope_type", scaling.get("type")) != "llama3":
        raise ValueError("plain implementation knows only llama3 rope scaling")
    pairing = pairing or config.get("rope_pairing", "half")
    W = {k: t.to(dtype) for k, t in weights.items()}

    inv_freq = rope_inverse_frequencies(D, theta, scaling)
    cos, sin = rope_tables(torch.arange(T), inv_freq, dtype)
    cos, sin = cos.to(tokens.device), sin.to(tokens.device)

    x = embedding(W["model.embed_tokens.weight"], tokens)
    for l in range(config["num_hidden_layers"]):
        p = f"model.layers.{l}."
        xb = _round(rmsnorm(x, W[p + "input_layernorm.weight"], eps), round_to)
        q = _round(linear(xb, W[p + "self_attn.q_proj.weight"]), round_to).view(T, H, D)
        k = _round(linear(xb, W[p + "self_attn.k_proj.weight"]), round_to).view(T, KVH, D)
        v = _round(linear(xb, W[p + "self_attn.v_proj.weight"]), round_to).view(T, KVH, D)
        q = _round(apply_rope(q, cos, sin, pairing), round_to)
        k = _round(apply_rope(k, cos, sin, pairing), round_to)
        a = _round(causal_attention(q, k, v, window), round_to).reshape(T, H * D)
        x = x + linear(a, W[p + "self_attn.o_proj.weight"])
        xb = _round(rmsnorm(x, W[p + "post_attention_layernorm.weight"], eps), round_to)
        h = _round(swiglu(linear(xb, W[p + "mlp.gate_proj.weight"]), linear(xb, W[p + "mlp.up_proj.weight"])), round_to)
        x = x + linear(h, W[p + "mlp.down_proj.weight"])
    x = _round(rmsnorm(x, W["model.norm.weight"], eps), round_to)
    head = W["lm_head.weight"] if "lm_head.weight" in W else W["model.embed_tokens.weight"]
    return linear(x, head).to(torch.float32).cpu()


# --------------------------------------------------------------------------- sampling
def argmax_first(logits: torch.Tensor) -> int:
    """``FloatTensor.java:138-151``: strict '>' scan, so the first maximum wins."""
    best, best_i = float(logits[0]), 0
    for i in range(1, logits.numel()):
        f = float(logits[i])
        if f > best:
            best, best_i = f, i
    return best_i


def temperature_softmax(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """``inference/sampler/Sampler.java:81-101``: logits / T, then softmax over the vocabulary."""
    z = logits.to(torch.float32) / temperature
    e = torch.exp(z - z.max())
    return e / e.sum()


def sample_categorical(probs: torch.Tensor, u: float) -> int:
    """``inference/sampler/CategoricalSampler.java:31-42``: first i with u < cdf_i, else last."""
    cdf = 0.0
    p = probs.to(torch.float32)
    acc = torch.zeros((), dtype=torch.float32)
    for i in range(p.numel()):
        acc = acc + p[i]
        if u < float(acc):
            return i
    return p.numel() - 1


def sample_top_p(probs: torch.Tensor, top_p: float, u: float) -> int:
    """``inference/sampler/ToppSampler.java:61-80,110-156``: drop p < (1-top_p)/(n-1), take values in
    descending order until their sum exceeds top_p, draw r = u * sum inside the kept set.  Equal
    values are ordered by index here (the reference's heap order among ties is unspecified)."""
    p = probs.to(torch.float32)
    n = p.numel()
    cutoff = (1.0 - top_p) / (n - 1)
    idx = [i for i in range(n) if float(p[i]) >= cutoff]
    idx.sort(key=lambda i: (-float(p[i]), i))
    cum = torch.zeros((), dtype=torch.float32)
    last = len(idx) - 1
    for j, i in enumerate(idx):
        cum = cum + p[i]
        if float(cum) > top_p:
            last = j
            break
    r = torch.tensor(u, dtype=torch.float32) * cum
    cdf = torch.zeros((), dtype=torch.float32)
    for j in range(last + 1):
        cdf = cdf + p[idx[j]]
        if float(r) < float(cdf):
            return idx[j]
    return idx[last]


def generate_greedy(config: dict, weights: dict, prompt: list[int], max_new_tokens: int,
                    stop_ids=(), **kw) -> list[int]:
    """``inference/InferenceEngine.java:309-355`` with temperature 0: append the argmax until a stop
    token (which is kept in the result, ``:346-348``) or the limit."""
    seq = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        logits = forward(config, weights, seq, **kw)[-1]
        t = argmax_first(logits)
        out.append(t)
        seq.append(t)
        if t in stop_ids:
            break
    return out
