"""Plain, slow implementation of the Llama / DeepSeek-LLM dense decoder.

Whole sequences, no cache, one function per part, torch on the CPU.  It shares
no code with the engine: it exists so that the engine has something simple to
be compared with.  Every function is written from the formulas of
codemk8/fastllm-py and cites the place (path within that project).

`forward()` takes a dict of tensors under their checkpoint names and a dict of
the config.json keys, so it can be run on any model folder the engine reads.

Two knobs exist only for the comparison with the engine:
  * `dtype`: float32 (the reference's validated path) or float64 (to measure
    how much of a difference is rounding);
  * `store`: a function applied wherever the engine writes an activation to
    memory in its activation dtype (identity for the 32-bit path, a round trip
    through bfloat16 for the bfloat16 path).  The residual stream stays in
    32-bit in the engine, so it is not rounded here either.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def identity(x):
    return x


def store_bf16(x):
    """Round to bfloat16 and back: what storing an activation in bf16 does."""
    return x.to(torch.bfloat16).to(x.dtype)


# --------------------------------------------------------------------- parts

def embedding(table, ids):
    """x = embed[ids], no scaling.  fastllm_py/model.py:447"""
    return table[ids]


def rms_norm(x, weight, eps):
    """x * (mean(x^2) + eps)^-1/2 * w, eps inside the root, weight multiplies.
    fastllm_py/kernels/ops.py:24-27"""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * (1.0 / torch.sqrt(var + eps)) * weight


def rope_tables(positions, head_dim, theta, scaling_factor=None):
    """cos/sin tables (T, head_dim/2) in float32.

    inv_freq = 1 / theta^(arange(0, D, 2)/D) in float32
    (fastllm_py/kernels/ops.py:79); linear scaling divides the integer
    positions by the factor in float64 before the float32 cast
    (fastllm_py/model.py:337-338, ops.py:80)."""
    import numpy as np

    # NumPy, as in the reference: its float32 power differs from torch's in the last bit,
    # and that bit times a position of a few hundred is visible in the angles.
    inv_freq = 1.0 / (theta ** (np.arange(0, head_dim, 2, dtype=np.float32) / head_dim))
    pos = np.asarray(positions)
    if scaling_factor is not None:
        pos = pos / float(scaling_factor)
    ang = pos.astype(np.float32)[:, None] * inv_freq[None, :]
    return torch.from_numpy(np.cos(ang)), torch.from_numpy(np.sin(ang))


def apply_rope(x, cos, sin):
    """Rotate-half convention: pairs are (x[i], x[i + D/2]).
    x: (T, heads, D); cos/sin: (T, D/2).  fastllm_py/kernels/ops.py:128-138"""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c = cos[:, None, :].to(x.dtype)
    s = sin[:, None, :].to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def softmax(scores):
    """exp(s - max) / sum, over the last axis.  fastllm_py/kernels/ops.py:166-171"""
    m = scores.max(dim=-1, keepdim=True).values
    e = torch.exp(scores - m)
    return e / e.sum(dim=-1, keepdim=True)


def attention(q, k, v, window=None):
    """Causal attention of a whole sequence with grouped KV heads.

    q: (T, H, D); k, v: (T, KVH, D).  Each KV head serves H/KVH consecutive
    query heads (fastllm_py/model.py:426-428); scores are scaled by D^-1/2 and
    masked scores are replaced by -1e30 (model.py:344-350); softmax and the
    weighted sum are in the compute dtype (model.py:351-353).  `window`
    (not in the reference) keeps only the last `window` keys, for toy layers."""
    T, H, D = q.shape
    rep = H // k.shape[1]
    kx = k.repeat_interleave(rep, dim=1)
    vx = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kx) * (D ** -0.5)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    scores = torch.where(hidden[None], torch.tensor(-1e30, dtype=scores.dtype), scores)
    probs = softmax(scores)
    ctx = torch.einsum("hts,shd->thd", probs, vx)
    return ctx.reshape(T, H * D)


def swiglu(gate, up):
    """g / (1 + exp(-g)) * u.  fastllm_py/kernels/ops.py:157-163"""
    return gate / (1.0 + torch.exp(-gate)) * up


def linear(x, w):
    """x @ W^T for an (out, in) weight.  fastllm_py/model.py:63"""
    return x @ w.t()


# --------------------------------------------------------------------- model

def read_config(cfg: dict) -> dict:
    """The keys and defaults of fastllm_py/config.py:87-104, for this architecture."""
    hidden = cfg["hidden_size"]
    heads = cfg["num_attention_heads"]
    scaling = cfg.get("rope_scaling")
    factor = None
    if scaling:
        kind = scaling.get("type") or scaling.get("rope_type")
        if kind == "linear":
            factor = float(scaling["factor"])
    return dict(
        layers=cfg["num_hidden_layers"], hidden=hidden, heads=heads,
        kv_heads=cfg.get("num_key_value_heads") or heads,
        head_dim=cfg.get("head_dim") or hidden // heads,
        vocab=cfg["vocab_size"],
        theta=float(cfg.get("rope_theta") or 10000.0),
        eps=float(cfg.get("rms_norm_eps") or 1e-6),
        factor=factor, tie=bool(cfg.get("tie_word_embeddings") or False),
    )


def forward(weights: dict, config: dict, ids, dtype=torch.float32, store=identity,
            hooks=None):
    """Logits (T, vocab) of one whole sequence.  fastllm_py/model.py:437-477.

    `hooks`, if given, is a dict that receives intermediate tensors by name
    (for tests of single parts)."""
    c = read_config(config)
    prefix = "model." if "model.embed_tokens.weight" in weights else ""   # model.py:194

    def w(name):
        return weights[name].to(dtype)

    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.shape[0]
    H, KVH, D = c["heads"], c["kv_heads"], c["head_dim"]
    x = embedding(w(f"{prefix}embed_tokens.weight"), ids)           # residual stream
    cos, sin = rope_tables(torch.arange(T), D, c["theta"], c["factor"])
    for i in range(c["layers"]):
        base = f"{prefix}layers.{i}."
        h = store(rms_norm(x, w(base + "input_layernorm.weight"), c["eps"]))
        q = store(linear(h, w(base + "self_attn.q_proj.weight"))).reshape(T, H, D)
        k = store(linear(h, w(base + "self_attn.k_proj.weight"))).reshape(T, KVH, D)
        v = store(linear(h, w(base + "self_attn.v_proj.weight"))).reshape(T, KVH, D)
        q = store(apply_rope(q, cos, sin))
        k = store(apply_rope(k, cos, sin))
        ctx = store(attention(q, k, v))
        x = x + store(linear(ctx, w(base + "self_attn.o_proj.weight")))
        h = store(rms_norm(x, w(base + "post_attention_layernorm.weight"), c["eps"]))
        g = store(linear(h, w(base + "mlp.gate_proj.weight")))
        u = store(linear(h, w(base + "mlp.up_proj.weight")))
        a = store(swiglu(g, u))
        x = x + store(linear(a, w(base + "mlp.down_proj.weight")))
        if hooks is not None:
            hooks[f"layer{i}"] = x
    x = store(rms_norm(x, w(f"{prefix}norm.weight"), c["eps"]))
    head = f"{prefix}embed_tokens.weight" if (c["tie"] or "lm_head.weight" not in weights) \
        else "lm_head.weight"                                         # model.py:228-231
    return linear(x, w(head)).to(torch.float32)


def load_folder(folder):
    """(weights by checkpoint name, config dict) of a model folder."""
    from safetensors.torch import load_file

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    for shard in sorted(folder.glob("*.safetensors")):
        weights.update(load_file(str(shard)))
    return weights, config


# ------------------------------------------------------------------ sampling

def apply_penalties(logits, counts, repetition_penalty=1.0, frequency_penalty=0.0,
                    presence_penalty=0.0):
    """Penalties over the generated-token histogram `counts` (id -> count):
    positive logits are divided by the repetition penalty and negative ones
    multiplied; then frequency*count + presence is subtracted.
    fastllm_py/graph_decode.py:73-93"""
    out = logits.to(torch.float64).clone()
    if not counts:
        return out
    for tok, cnt in counts.items():
        if repetition_penalty != 1.0:
            out[tok] = out[tok] / repetition_penalty if out[tok] > 0 else out[tok] * repetition_penalty
        if frequency_penalty != 0.0 or presence_penalty != 0.0:
            out[tok] -= frequency_penalty * cnt + presence_penalty
    return out


def probabilities(logits, temperature, top_p=1.0, top_k=0, min_p=0.0):
    """Temperature softmax, then top-k, min-p and nucleus truncation, each
    followed by renormalisation.  fastllm_py/graph_decode.py:96-120"""
    lg = logits.to(torch.float64) / temperature
    lg = lg - lg.max()
    p = torch.exp(lg)
    p = p / p.sum()
    if top_k and 0 < top_k < p.numel():
        keep = torch.topk(p, top_k).indices
        mask = torch.zeros_like(p, dtype=torch.bool)
        mask[keep] = True
        p = torch.where(mask, p, torch.zeros_like(p))
        p = p / p.sum()
    if min_p > 0.0:
        p = torch.where(p < min_p * p.max(), torch.zeros_like(p), p)
        p = p / p.sum()
    if top_p < 1.0:
        order = torch.argsort(p, descending=True, stable=True)
        csum = torch.cumsum(p[order], dim=0)
        beyond = order[csum > top_p]
        if beyond.numel() > 1:                 # the first token to cross top_p is kept
            p[beyond[1:]] = 0.0
            p = p / p.sum()
    return p


def sample(logits, temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, uniform=None):
    """Greedy when temperature <= 0 (first index on ties), else a draw by
    inversion of the cumulative distribution with the uniform number given:
    what numpy's Generator.choice(p=...) does with one rng.random().
    fastllm_py/graph_decode.py:123-133"""
    if temperature <= 0.0:
        return int(torch.argmax(logits))
    p = probabilities(logits, temperature, top_p, top_k, min_p)
    cdf = torch.cumsum(p, dim=0)
    cdf = cdf / cdf[-1]
    idx = int(torch.searchsorted(cdf, torch.tensor(uniform, dtype=torch.float64), right=True))
    return min(idx, p.numel() - 1)


def generate(weights, config, prompt, max_new_tokens, temperature=0.0, seed=None,
             stop_ids=(), dtype=torch.float32, store=identity, **sampling):
    """Token-by-token generation by re-running the whole sequence.
    fastllm_py/model.py:531-549: one uniform per sampled token from
    numpy.random.default_rng(seed); the stop token is emitted."""
    import numpy as np

    rng = np.random.default_rng(seed) if temperature > 0.0 else None
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        row = forward(weights, config, ids, dtype=dtype, store=store)[-1]
        u = float(rng.random()) if rng is not None else None
        nxt = sample(row, temperature, uniform=u, **sampling)
        out.append(nxt)
        ids.append(nxt)
        if nxt in stop_ids:
            break
    return out
