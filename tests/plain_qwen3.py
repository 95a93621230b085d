"""A plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part, CPU torch only.

This file is the yardstick the engine's tests compare against. It shares no code with `holon_b200`: it reads
`config.json` and `model.safetensors` itself and spells every formula out. Each function cites the file and lines
of mxinO/holon (paths inside that project) whose arithmetic it restates. `tests/golden/` holds the outputs of
holon's own CPU model on a tiny random model, recorded once by `tests/golden/make_golden.py`;
`tests/test_plain.py` checks this file against them, so the formulas here rest on more than a reading.
"""
from __future__ import annotations

import json
import pathlib

import torch
from safetensors import safe_open


# ---------------------------------------------------------------- model folder

def read_folder(folder, dtype=torch.float32):
    """(config dict, {HF tensor name: tensor as `dtype`}) of a folder holding config.json and *.safetensors
    (std/holon_std/weights/hf/source.py:49-115: config.json is required, every shard is read)."""
    folder = pathlib.Path(folder)
    config = json.loads((folder / "config.json").read_text())
    tensors = {}
    for shard in sorted(folder.glob("*.safetensors")):
        with safe_open(str(shard), framework="pt") as f:
            for name in f.keys():
                tensors[name] = f.get_tensor(name).to(dtype)
    return config, tensors


def rope_theta(config) -> float:
    """plugins/holon_plugins/models/qwen3/recipe.py:32-38: `rope_parameters.rope_theta`, else `rope_theta`."""
    params = config.get("rope_parameters") or {"rope_theta": config["rope_theta"]}
    return float(params["rope_theta"])


# ---------------------------------------------------------------- rounding of a reduced-precision pipeline

_ROUND_TO = None


class rounding:
    """`with rounding(torch.bfloat16): forward(...)` rounds every intermediate result to that type where the
    reference's bfloat16 pipeline does (each product's output, each norm, the rotation, the attention output, silu and
    its product, each residual sum: std/holon_std/ops/reference.py:7-30, std/holon_std/ffn/reference.py:12), while
    the arithmetic inside each function stays 32-bit. The distance of such a run from the exact one is the yardstick
    for what a bfloat16 engine may differ by: the reference's judge measures an engine against a plain bfloat16 run in
    the same way (judge/README.md:64-67)."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global _ROUND_TO
        self.before, _ROUND_TO = _ROUND_TO, self.dtype

    def __exit__(self, *exc):
        global _ROUND_TO
        _ROUND_TO = self.before


def _r(x):
    return x if _ROUND_TO is None else x.to(_ROUND_TO).to(x.dtype)


# ---------------------------------------------------------------- parts

def embedding(ids, table):
    """Row gather, no scaling (std/holon_std/ops/units.py:303-304)."""
    return table[torch.as_tensor(ids, dtype=torch.long)]


def rms_norm(x, weight, eps):
    """x · rsqrt(mean(x²) + eps) · weight, eps inside the root (std/holon_std/ops/reference.py:7-11)."""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return _r(x * torch.rsqrt(variance + eps) * weight)


def rope(x, positions, theta):
    """Half-split ("neox") rotation of x [T, heads, D] over the whole head (std/holon_std/ops/reference.py:21-30):
    inv_freq_i = θ^(−2i/D), angle = position · inv_freq in 32-bit, (a, b) → (a·cos − b·sin, b·cos + a·sin)."""
    d = x.shape[-1]
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angles = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    cos, sin = angles.cos().to(x.dtype)[:, None, :], angles.sin().to(x.dtype)[:, None, :]
    a, b = x[..., : d // 2], x[..., d // 2:]
    return _r(torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1))


def causal_attention(q, k, v, window=0):
    """softmax(q·kᵀ / sqrt(D) + causal mask) · v for one sequence; q [T, Hq, D], k and v [T, Hkv, D]; query head h
    reads KV head h // (Hq/Hkv) (std/holon_std/mixers/gqa/reference.py:7-24). `window` W > 0 hides keys at or
    before position − W (same file, :19-20); Qwen3 in holon has none."""
    t, hq, d = q.shape
    group = hq // k.shape[1]
    k, v = k.repeat_interleave(group, dim=1), v.repeat_interleave(group, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) / d ** 0.5
    pos = torch.arange(t)
    hidden = pos[None, :] > pos[:, None]
    if window:
        hidden = hidden | (pos[:, None] - pos[None, :] >= window)
    probs = scores.masked_fill(hidden, float("-inf")).softmax(dim=-1)
    return _r(torch.einsum("hqk,khd->qhd", probs, v))


def attention_layer(x, w, prefix, config, positions, window=0):
    """Projections without bias, per-head RMSNorm of q and k before the rotation, attention, output projection
    (std/holon_std/mixers/gqa/units.py:234-262, 282-294; recipe.py:47-49 gives q/k-norm the model's eps)."""
    t = x.shape[0]
    hq, hkv, d = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    q = _r(x @ w[prefix + "q_proj.weight"].T).reshape(t, hq, d)
    k = _r(x @ w[prefix + "k_proj.weight"].T).reshape(t, hkv, d)
    v = _r(x @ w[prefix + "v_proj.weight"].T).reshape(t, hkv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], config["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], config["rms_norm_eps"])
    q, k = rope(q, positions, rope_theta(config)), rope(k, positions, rope_theta(config))
    o = causal_attention(q, k, v, window)
    return _r(o.reshape(t, hq * d) @ w[prefix + "o_proj.weight"].T)


def swiglu(x, w, prefix):
    """down(silu(gate(x)) · up(x)), no biases (std/holon_std/ffn/units.py:31-50; ffn/reference.py:7-12)."""
    gate = _r(x @ w[prefix + "gate_proj.weight"].T)
    up = _r(x @ w[prefix + "up_proj.weight"].T)
    return _r(_r(_r(torch.nn.functional.silu(gate)) * up) @ w[prefix + "down_proj.weight"].T)


def block(h, w, i, config, positions):
    """Pre-norm residual block: h += mixer(norm(h)); h += ffn(norm(h)) (std/holon_std/blocks/units.py:23-25)."""
    p = f"model.layers.{i}."
    eps = config["rms_norm_eps"]
    h = _r(h + attention_layer(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", config, positions))
    return _r(h + swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp."))


def forward(config, w, ids):
    """Logits [T, V] for every position of one whole sequence: embed → blocks → norm → head, the head reading the
    embedding table when `tie_word_embeddings` (core/holon/core/build.py:292-307; ops/units.py:313-318, 345-348)."""
    positions = torch.arange(len(ids))
    h = embedding(ids, w["model.embed_tokens.weight"])
    for i in range(config["num_hidden_layers"]):
        h = block(h, w, i, config, positions)
    h = rms_norm(h, w["model.norm.weight"], config["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return _r(h @ head.T)


# ---------------------------------------------------------------- sampling

_M32 = 0xFFFFFFFF


def _mix32(x: int) -> int:
    """lowbias32 (std/holon_std/sampling/sampler.py:24-30)."""
    x ^= x >> 16
    x = (x * 0x7FEB352D) & _M32
    x ^= x >> 15
    x = (x * 0x846CA68B) & _M32
    return x ^ (x >> 16)


def uniform(seed: int, position: int) -> float:
    """The one uniform of (seed, position of the token being drawn) (std/holon_std/sampling/sampler.py:33-40). The
    reference adds the half in 32-bit floating point: from 2^23 on the sum is a tie and rounds to the even neighbour,
    so the value is the reference's bit for bit only if the sum is taken in 32-bit here too."""
    import numpy as np
    h = _mix32(seed & _M32) ^ ((seed >> 32) & _M32) ^ _mix32(position & _M32)
    h = _mix32(h)
    u = (np.float32(h >> 8) + np.float32(0.5)) * np.float32(2.0 ** -24)
    return min(float(u), 1 - 2.0 ** -24)


def distribution(logits, temperature, top_k=0, top_p=1.0, min_p=0.0):
    """The distribution a row is drawn from, float64, in vocabulary order (std/holon_std/sampling/reference.py:13-30):
    logits / temperature → keep the k largest → keep the smallest prefix whose mass reaches p → drop below
    min_p × the largest. Temperature 0 is the arg max."""
    x = logits.double()
    if temperature == 0:
        return torch.nn.functional.one_hot(x.argmax(), x.numel()).double()
    x = x / temperature
    keep = torch.ones_like(x, dtype=torch.bool)
    order = x.argsort(descending=True, stable=True)
    if top_k > 0:
        keep[order[top_k:]] = False
    q = torch.where(keep, x, float("-inf")).softmax(-1)
    if top_p < 1:
        sorted_q = q[order]
        keep[order[sorted_q.cumsum(-1) - sorted_q > top_p]] = False
    if min_p > 0:
        keep &= q >= min_p * q.max()
    return torch.where(keep, x, float("-inf")).softmax(-1)


def draw(probs, u: float) -> int:
    """Inverse CDF in vocabulary order: the first token whose cumulative mass exceeds u × total
    (std/holon_std/sampling/sampler.py:57-61)."""
    c = probs.double().cumsum(-1)
    index = int(torch.searchsorted(c, torch.tensor([u * float(c[-1])], dtype=c.dtype), right=True)[0])
    return min(index, probs.numel() - 1)


def sample(logits, temperature, seed, position, top_k=0, top_p=1.0, min_p=0.0) -> int:
    """The token drawn at `position` (the position the new token will take: input position + 1, sampler.py:135)."""
    if temperature == 0:
        return int(logits.argmax())
    return draw(distribution(logits, temperature, top_k, top_p, min_p), uniform(seed, position))


def logprobs(logits, token: int, k: int):
    """(log-probability of `token`, ids of the k most likely, their log-probabilities) from the raw logits of one
    position: log_softmax, gather, topk (std/holon_std/sampling/sampler.py:118-126)."""
    lp = logits.double().log_softmax(-1)
    order = sorted(range(lp.numel()), key=lambda i: (-float(lp[i]), i))[:k]      # ranked; equal ones by ascending id
    return float(lp[token]), order, [float(lp[i]) for i in order]


def generate(config, w, prompt, max_tokens, temperature=0.0, seed=0, top_k=0, top_p=1.0, min_p=0.0):
    """Tokens generated after `prompt`, each step a whole forward pass (no cache)."""
    ids = list(prompt)
    for _ in range(max_tokens):
        logits = forward(config, w, ids)[-1]
        ids.append(sample(logits, temperature, seed, len(ids), top_k, top_p, min_p))
    return ids[len(prompt):]
