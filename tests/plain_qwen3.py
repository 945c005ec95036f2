"""Plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

This is the oracle the engine is compared with.  It shares no code with
`socrates_b200`: it reads config.json as a dict and the tensors by checkpoint name,
and computes in whatever dtype `compute_dtype` names (float32 or float64) on the
CPU.  Each function cites the lines of the reference whose formula it restates.
The one extension over the reference is the key window (`sliding_window`), which
the reference's configs carry but its code never reads; its rule is stated in
`attention_mask`.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * w, eps inside the root, gain is w itself.

    model/qwen/qwen_kv_cont.py:45-53
    """
    rms = torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x / rms * weight


def rope_tables(positions, head_dim, theta):
    """cos, sin [T, head_dim] for absolute positions; angles in float32.

    inv_freq_j = theta^(-2j/D); angle = pos * inv_freq; the half table is repeated
    to full width.  model/qwen/qwen_kv_cont.py:56-64
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    angles = positions.float()[..., None] * inv_freq
    angles = torch.cat([angles, angles], dim=-1)
    return angles.cos(), angles.sin()


def rotate_half(x):
    """cat(-x[D/2:], x[:D/2]): dim j pairs with j + D/2.  model/qwen/qwen_kv_cont.py:67-69"""
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rope(x, cos, sin):
    """x [T, heads, D]; x*cos + rotate_half(x)*sin.  model/qwen/qwen_kv_cont.py:72-77"""
    cos = cos[:, None, :].to(x.dtype)
    sin = sin[:, None, :].to(x.dtype)
    return x * cos + rotate_half(x) * sin


def attention_mask(q_positions, k_positions, window):
    """True where a query may see a key.

    Causal: key position <= query position (model/qwen/qwen_kv_cont.py:228-230,
    explicit masked form model/qwen/qwen.py:119-126).  With a window of w keys a
    query at position p sees positions p-w+1 .. p, itself included.
    """
    keep = k_positions[None, :] <= q_positions[:, None]
    if window is not None:
        keep &= k_positions[None, :] > q_positions[:, None] - window
    return keep


def attention_core(q, k, v, scale, keep):
    """softmax(scale * q k^T, masked) v per head, GQA: head h uses kv head h // G.

    q [T, Hq, D], k/v [S, Hkv, D], keep [T, S] -> [T, Hq, D].
    model/qwen/qwen_kv_paged.py:139,171-173; model/qwen/qwen.py:119-126
    """
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = torch.empty_like(q)
    for h in range(Hq):
        kv = h // G
        s = (q[:, h, :] @ k[:, kv, :].T) * scale
        s = s.masked_fill(~keep, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kv, :]
    return out


def attention(x, w, prefix, cfg, positions, window):
    """Projections, per-head QK-norm, rotation, causal GQA attention, output projection.

    model/qwen/qwen_kv_paged.py:130-175 (projections 150-152, QK-norm then RoPE
    153-154, o_proj 175)
    """
    T = x.shape[0]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = (x @ w[prefix + "q_proj.weight"].T).view(T, Hq, D)
    k = (x @ w[prefix + "k_proj.weight"].T).view(T, Hkv, D)
    v = (x @ w[prefix + "v_proj.weight"].T).view(T, Hkv, D)
    cos, sin = rope_tables(positions, D, cfg["rope_theta"])
    q = apply_rope(rms_norm(q, w[prefix + "q_norm.weight"], eps), cos, sin)
    k = apply_rope(rms_norm(k, w[prefix + "k_norm.weight"], eps), cos, sin)
    keep = attention_mask(positions, positions, window)
    o = attention_core(q, k, v, D ** -0.5, keep)
    return o.reshape(T, Hq * D) @ w[prefix + "o_proj.weight"].T


def swiglu(x, w, prefix):
    """down(up(x) * silu(gate(x))).  model/qwen/qwen_kv_cont.py:250-266"""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (u * (g * torch.sigmoid(g))) @ w[prefix + "down_proj.weight"].T


def block(x, w, i, cfg, positions, window):
    """x + attn(norm(x)); then x + mlp(norm(x)).  model/qwen/qwen_kv_paged.py:186-189"""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    x = x + attention(rms_norm(x, w[p + "input_layernorm.weight"], eps), w,
                      p + "self_attn.", cfg, positions, window)
    return x + swiglu(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")


def layer_windows(cfg):
    """Window per layer from config.json: `layer_types` if present, else
    `use_sliding_window` with `max_window_layers` (layers at or above it)."""
    n = cfg["num_hidden_layers"]
    win = cfg.get("sliding_window")
    if cfg.get("layer_types") is not None:
        return [win if t == "sliding_attention" else None for t in cfg["layer_types"]]
    if cfg.get("use_sliding_window", False):
        first = cfg.get("max_window_layers", n)
        return [win if i >= first else None for i in range(n)]
    return [None] * n


def hidden_states(w, cfg, token_ids, compute_dtype=torch.float64):
    """Final-normed hidden state [T, d] of one whole sequence starting at position 0."""
    cfg = dict(cfg)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    w = {k: v.to(compute_dtype) for k, v in w.items()}
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    x = w["model.embed_tokens.weight"][ids]                  # model/qwen/qwen_kv_paged.py:219
    wins = layer_windows(cfg)
    for i in range(cfg["num_hidden_layers"]):
        x = block(x, w, i, cfg, positions, wins[i])
    return rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])   # :223


def logits(w, cfg, token_ids, compute_dtype=torch.float64):
    """Logits [T, V] at every position of one whole sequence.

    Tied head: x @ embed^T (model/qwen/qwen_kv_paged.py:224); untied: x @ lm_head^T.
    """
    h = hidden_states(w, cfg, token_ids, compute_dtype)
    name = "model.embed_tokens.weight" if cfg.get("tie_word_embeddings", False) else "lm_head.weight"
    return h @ w[name].to(compute_dtype).T


def load_folder(model_dir):
    """(config dict, {checkpoint name: tensor}) of a model folder."""
    from safetensors import safe_open
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    w = {}
    with safe_open(str(model_dir / "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k)
    return cfg, w


# --------------------------------------------------------------------------- sampling

def greedy(logits_row):
    """argmax, ties to the lowest index.  model/inference_paged.py:166,193"""
    return int(torch.argmax(logits_row))


def _mix32(x):
    """The 32-bit finalizer of the counter-based generator the sampler documents
    (socrates_b200/sampling): three xorshift-multiply rounds on unsigned 32-bit."""
    m = 0xFFFFFFFF
    x = x & m
    x ^= x >> 16
    x = (x * 0x7FEB352D) & m
    x ^= x >> 15
    x = (x * 0x846CA68B) & m
    x ^= x >> 16
    return x


def uniform_for(seed, counter, index):
    """The uniform in (0,1) that belongs to (seed, counter, vocabulary index)."""
    h = _mix32(int(seed) ^ 0x9E3779B9)
    h = _mix32(h ^ _mix32(int(counter) + 0x85EBCA6B))
    idx = torch.as_tensor(index, dtype=torch.int64)
    m = 0xFFFFFFFF
    x = (idx + 0x165667B1) & m
    x = x ^ h
    x ^= x >> 16
    x = (x * 0x7FEB352D) & m
    x ^= x >> 15
    x = (x * 0x846CA68B) & m
    x ^= x >> 16
    return ((x >> 9).to(torch.float64) + 0.5) / 8388608.0


def temperature_scores(logits_row, temperature, seed, counter):
    """logits/T + Gumbel noise; the sampled token is the argmax of these.

    Sampling from softmax(logits/T) (docs/day_1_docs.md:45-52 describes the
    distribution) by the Gumbel-max rule: argmax_i (l_i/T - log(-log u_i)).
    """
    V = logits_row.numel()
    u = uniform_for(seed, counter, torch.arange(V))
    g = -torch.log(-torch.log(u))
    return logits_row.to(torch.float64) / temperature + g


def sample_temperature(logits_row, temperature, seed, counter):
    return int(torch.argmax(temperature_scores(logits_row, temperature, seed, counter)))
