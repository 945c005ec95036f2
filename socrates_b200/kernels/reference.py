"""A plain PyTorch statement of what each CUDA kernel computes, in float32.

These functions are the oracles of the per-kernel tests (as the reference keeps
model/kernels/reference.py beside its kernel).  They are never called on the product
path.  Each takes the same arguments as its kernel's entry point in `ops` and returns
what the kernel writes.
"""

from __future__ import annotations

from typing import Optional

import torch


def embed_ref(table, ids):
    return table[ids.long()].float()


def add_rmsnorm_ref(residual, delta, gain, eps, row_index=None):
    """Returns (new residual, normed rows in float32)."""
    v = residual.clone()
    if delta is not None:
        for s in range(delta.shape[0]):            # the kernel's order of additions
            v = v + delta[s]
    rows = v if row_index is None else v[row_index.long()]
    normed = rows / torch.sqrt(rows.pow(2).mean(-1, keepdim=True) + eps) * gain
    return v, normed


def qk_norm_rope_ref(qkv, q_gain, k_gain, inv_freq, rotary_dim, positions, eps, Hq, Hkv, D):
    """Returns float32 (q [N,Hq,D], k [N,Hkv,D], v [N,Hkv,D]) after norm and rotation."""
    N = qkv.shape[0]
    x = qkv.float().view(N, Hq + 2 * Hkv, D)
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]

    def norm(t, g):
        if g is None:
            return t
        return t / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + eps) * g

    def rotate(t):
        if rotary_dim == 0:
            return t
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq[:half].float()[None, :]     # [N, half]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = t[..., :half], t[..., half:rotary_dim]
        return torch.cat([a * c - b * s, b * c + a * s, t[..., rotary_dim:]], dim=-1)

    return rotate(norm(q, q_gain)), rotate(norm(k, k_gain)), v.clone()


def kv_slots(block_table, token_rows, positions, page_size):
    """(page, offset) of each token's slot."""
    page = block_table[token_rows.long(), (positions // page_size).long()].long()
    return page, (positions % page_size).long()


def silu_mul_ref(gate_up):
    F = gate_up.shape[1] // 2
    g, u = gate_up[:, :F].float(), gate_up[:, F:].float()
    return u * (g * torch.sigmoid(g))


def gemm_ref(a, w):
    return a.double() @ w.double().T


def paged_attention_ref(q, k_pool, v_pool, block_table, token_rows, positions, Hq, scale, window=0):
    """One query per token against its row's pages; float64 softmax. Returns [N, Hq*D]."""
    N = q.shape[0]
    _, Hkv, BS, D = k_pool.shape
    G = Hq // Hkv
    out = torch.zeros(N, Hq, D, dtype=torch.float64, device=q.device)
    qf = q.double().view(N, Hq, D)
    for n in range(N):
        row, pos = int(token_rows[n]), int(positions[n])
        lo = max(0, pos + 1 - window) if window else 0
        keys = torch.arange(lo, pos + 1, device=q.device)
        pages = block_table[row, (keys // BS).long()].long()
        offs = (keys % BS).long()
        k = k_pool[pages, :, offs].double()            # [S, Hkv, D]
        v = v_pool[pages, :, offs].double()
        for h in range(Hq):
            s = (k[:, h // G] @ qf[n, h]) * scale
            p = torch.softmax(s, dim=0)
            out[n, h] = p @ v[:, h // G]
    return out.view(N, Hq * D)


def _mix32(x):
    m = 0xFFFFFFFF
    x = x & m
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & m
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & m
    x = x ^ (x >> 16)
    return x


def sample_scores_ref(logits, temperature, seeds, counters):
    """The scores whose argmax the kernel returns: logits where temperature is 0, else
    logits / T + Gumbel noise from the counter-based generator.  float64 [M, V]."""
    M, V = logits.shape
    out = logits.double().clone()
    idx = torch.arange(V, dtype=torch.int64, device=logits.device)
    for m in range(M):
        T = float(temperature[m]) if temperature is not None else 0.0
        if T <= 0:
            continue
        seed = int(seeds[m]) & 0xFFFFFFFF
        ctr = int(counters[m]) & 0xFFFFFFFF
        key = _mix32(torch.tensor(seed ^ 0x9E3779B9, dtype=torch.int64))
        key = _mix32(key ^ _mix32(torch.tensor((ctr + 0x85EBCA6B) & 0xFFFFFFFF, dtype=torch.int64)))
        x = _mix32(((idx + 0x165667B1) & 0xFFFFFFFF) ^ int(key))
        u = ((x >> 9).double() + 0.5) / 8388608.0
        out[m] = logits[m].double() / T - torch.log(-torch.log(u))
    return out
