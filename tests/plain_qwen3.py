"""Plain, slow Qwen3 dense decoder: the oracle the engine is compared with.

Whole sequences, no cache, no batching, one function per part, written from the
formulas of raun6k/Pylon's model code (each function cites file:line of that project).
It shares no code with ``pylon_b200``: it reads ``config.json`` and ``model.safetensors``
itself and computes in float64 by default, so that rounding faults of the engine's
32-bit path show against it.

``tests/golden/make_golden.py`` compared this file once with Pylon's own ``Qwen3Model``
on the CPU; the stored outputs are checked by ``tests/test_plain_reference.py``.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch


# ---------------------------------------------------------------------------------------
# reading a model folder
# ---------------------------------------------------------------------------------------
def read_model(folder: str | Path, dtype: torch.dtype = torch.float64) -> tuple[dict, dict]:
    """Returns (config dict, weights by checkpoint name) with every tensor cast to ``dtype``."""
    from safetensors import safe_open

    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            weights[name] = handle.get_tensor(name).to(dtype)
    return config, weights


# ---------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x / sqrt(mean(x^2) + eps) * w over the last dim.  src/pylon/model/layers.py:30-40"""
    variance = (x * x).mean(dim=-1, keepdim=True)
    return x / torch.sqrt(variance + eps) * weight


def rope_tables(head_dim: int, theta: float, positions: torch.Tensor, dtype: torch.dtype):
    """cos/sin of p * theta^(-2j/d), angles duplicated over both halves.

    src/pylon/model/layers.py:43-51.  The angle itself is formed in float32 exactly as the
    reference does (float32 inverse frequency times float32 position), then widened, so the
    oracle and a 32-bit engine agree on the angle and differ only in cos/sin rounding.
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    angles = positions.to(torch.float32).unsqueeze(1) * inv_freq.unsqueeze(0)
    angles = torch.cat((angles, angles), dim=1).to(dtype)
    return torch.cos(angles), torch.sin(angles)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin with pairs (j, j+d/2).  src/pylon/model/layers.py:73-78

    x: [heads, T, d]; cos, sin: [T, d].
    """
    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rotated * sin


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None):
    """softmax(q k^T / sqrt(d)) v with key j visible to query i iff j <= i (and i - j < window).

    q: [n_heads, T, d]; k, v: [n_kv_heads, T, d].  Query head h uses KV head h // group.
    Mask and grouping: src/pylon/kv/cache.py:483-491; scale 1/sqrt(d) is the library default
    the reference relies on (src/pylon/kv/cache.py:462-476 passes none).
    """
    n_heads, tokens, dim = q.shape
    group = n_heads // k.shape[0]
    k = k.repeat_interleave(group, dim=0)
    v = v.repeat_interleave(group, dim=0)
    out = torch.empty_like(q)
    rows = tokens if tokens <= 8_192 else 2_048   # long sequences: the same rows, a slice at a time (the scores of all would not fit)
    for begin in range(0, tokens, rows):
        end = min(tokens, begin + rows)
        scores = q[:, begin:end] @ k[:, :end].transpose(1, 2) / math.sqrt(dim)
        i = torch.arange(begin, end, device=q.device).unsqueeze(1)
        j = torch.arange(end, device=q.device).unsqueeze(0)
        visible = j <= i
        if window is not None:
            visible &= (i - j) < window
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, begin:end] = torch.softmax(scores, dim=-1) @ v[:, :end]
    return out


def attention_part(x, w, prefix, cfg, cos, sin, window=None):
    """QKV projection, per-head q/k RMSNorm, RoPE, attention, output projection.

    src/pylon/model/layers.py:81-138 (projection and split 126-131, norms then rotation
    132-134, output 137-138).
    """
    heads, kv_heads, dim = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    tokens = x.shape[0]
    q = (x @ w[prefix + "self_attn.q_proj.weight"].T).view(tokens, heads, dim).transpose(0, 1)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].T).view(tokens, kv_heads, dim).transpose(0, 1)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].T).view(tokens, kv_heads, dim).transpose(0, 1)
    q = apply_rope(rms_norm(q, w[prefix + "self_attn.q_norm.weight"], eps), cos, sin)
    k = apply_rope(rms_norm(k, w[prefix + "self_attn.k_norm.weight"], eps), cos, sin)
    context = causal_attention(q, k, v, window).transpose(0, 1).reshape(tokens, heads * dim)
    return context @ w[prefix + "self_attn.o_proj.weight"].T


def swiglu_part(x, w, prefix):
    """down(silu(gate(x)) * up(x)).  src/pylon/model/layers.py:13-27"""
    gate = x @ w[prefix + "mlp.gate_proj.weight"].T
    up = x @ w[prefix + "mlp.up_proj.weight"].T
    return (gate * torch.sigmoid(gate) * up) @ w[prefix + "mlp.down_proj.weight"].T


def block(x, w, prefix, cfg, cos, sin):
    """Pre-norm residual block.  src/pylon/model/layers.py:168-200"""
    eps = cfg["rms_norm_eps"]
    x = x + attention_part(rms_norm(x, w[prefix + "input_layernorm.weight"], eps), w, prefix, cfg, cos, sin)
    return x + swiglu_part(rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps), w, prefix)


def forward(cfg: dict, w: dict, token_ids) -> torch.Tensor:
    """Logits at every position of one whole sequence, [T, vocab].

    src/pylon/model/model.py:124-144: embedding, blocks, final norm, LM head (the embedding
    table when ``tie_word_embeddings``, else ``lm_head.weight``).
    """
    device = w["model.embed_tokens.weight"].device   # the weights may have been moved to a GPU for large shapes
    ids = torch.as_tensor(list(token_ids), dtype=torch.long, device=device)
    dtype = w["model.embed_tokens.weight"].dtype
    x = w["model.embed_tokens.weight"][ids]
    cos, sin = rope_tables(cfg["head_dim"], float(cfg["rope_theta"]), torch.arange(len(ids)), dtype)
    cos, sin = cos.to(device), sin.to(device)
    for layer in range(cfg["num_hidden_layers"]):
        x = block(x, w, f"model.layers.{layer}.", cfg, cos, sin)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------
def greedy(logits: torch.Tensor) -> int:
    """argmax, lowest index on ties.  src/pylon/decode/runner.py:511-512"""
    return int(torch.argmax(logits.double()))


def sampling_distribution(logits: torch.Tensor, temperature: float, top_p: float) -> torch.Tensor:
    """softmax(logits / T), then nucleus: in descending order drop a token when the mass
    before it exceeds top_p (the first is always kept), renormalise.

    src/pylon/decode/runner.py:513-525.  Returned in vocabulary order, float64.
    """
    probs = torch.softmax(logits.double() / temperature, dim=-1)
    if top_p >= 1:
        return probs
    ordered, index = torch.sort(probs, descending=True, stable=True)
    before = torch.cumsum(ordered, dim=-1) - ordered
    keep = before <= top_p
    keep[0] = True
    ordered = torch.where(keep, ordered, torch.zeros_like(ordered))
    out = torch.zeros_like(probs)
    out[index] = ordered / ordered.sum()
    return out


def generate_greedy(cfg: dict, w: dict, prompt, new_tokens: int, stop_ids=()) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token."""
    tokens = list(prompt)
    out: list[int] = []
    for _ in range(new_tokens):
        token = greedy(forward(cfg, w, tokens)[-1])
        if token in stop_ids:
            break
        out.append(token)
        tokens.append(token)
    return out


def as_numpy(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float64).cpu().numpy()
