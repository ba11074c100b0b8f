"""A plain PyTorch restatement of the decoder the plans execute (RMSNorm, RoPE, causal GQA
attention, SwiGLU or a softmax top-k mixture of SwiGLU experts, tied LM head, mean next-token
cross-entropy).

It is the fp32 reference that GPU tests compare the engine against: it reads the engine's own
parameters, so both sides start from identical weights. It is never on a hot path.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def rope(x, seq, theta):
    """x: [B, S, heads, hd]; rotate-half convention with position = index inside the sequence."""
    hd = x.shape[-1]
    half = hd // 2
    pos = torch.arange(seq, device=x.device, dtype=x.dtype)
    inv = theta ** (-torch.arange(half, device=x.device, dtype=x.dtype) / half)
    ang = pos[:, None] * inv[None, :]
    c, s = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def moe_ffn(h, wr, wgu, wd, top_k):
    """Mixture of experts without capacity drops. h [..., H]; wr [E, H]; wgu [E*2F, H] (per expert:
    gate rows then up rows); wd [E*H, F]. Weights are the softmax probabilities of the chosen
    experts renormalised over the chosen k."""
    E, H = wr.shape
    F_ = wd.shape[1]
    flat = h.reshape(-1, H)
    prob = torch.softmax(flat @ wr.t(), -1)
    top_p, top_e = prob.topk(top_k, -1)
    top_w = top_p / top_p.sum(-1, keepdim=True)
    out = torch.zeros_like(flat)
    wgu, wd = wgu.view(E, 2 * F_, H), wd.view(E, H, F_)
    for e in range(E):
        tok, slot = (top_e == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        g, u = (flat[tok] @ wgu[e].t()).chunk(2, -1)
        y = (F.silu(g) * u) @ wd[e].t()
        out = out.index_add(0, tok, y * top_w[tok, slot, None])
    return out.view_as(h)


def forward_loss(params: dict, tokens, targets, *, layers, heads, kv_heads, head_dim, seq, eps, theta,
                 dtype=torch.float32, top_k=0):
    """params: name -> tensor (``embed``, ``L{i}.g1/wqkv/wo/g2/wgu/wd``, ``gf``, optional ``lm_head``).
    tokens / targets: int64 [B, S]. Returns the mean cross-entropy."""
    B, S = tokens.shape
    p = {k: v.to(dtype) for k, v in params.items()}
    x = p["embed"][tokens]                                     # B S H

    def norm(h, g):
        return h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps) * g.view(-1)

    rep = heads // kv_heads
    for l in range(layers):
        pre = f"L{l}."
        h = norm(x, p[pre + "g1"])
        qkv = h @ p[pre + "wqkv"].t()
        q, k, v = qkv.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], -1)
        q = rope(q.view(B, S, heads, head_dim), seq, theta)
        k = rope(k.view(B, S, kv_heads, head_dim), seq, theta)
        v = v.view(B, S, kv_heads, head_dim)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        k = k.repeat_interleave(rep, 1)
        v = v.repeat_interleave(rep, 1)
        s = (q @ k.transpose(-1, -2)) * head_dim ** -0.5
        mask = torch.ones(S, S, device=x.device, dtype=torch.bool).tril()
        s = s.masked_fill(~mask, float("-inf"))
        a = torch.softmax(s, -1) @ v
        a = a.transpose(1, 2).reshape(B, S, heads * head_dim)
        x = x + a @ p[pre + "wo"].t()
        h = norm(x, p[pre + "g2"])
        if pre + "wr" in p:
            x = x + moe_ffn(h, p[pre + "wr"], p[pre + "experts.wgu"], p[pre + "experts.wd"], top_k)
            continue
        gu = h @ p[pre + "wgu"].t()
        g, u = gu.chunk(2, -1)
        x = x + (F.silu(g) * u) @ p[pre + "wd"].t()
    h = norm(x, p["gf"])
    head = p.get("lm_head", p["embed"])
    logits = h @ head.t()
    return F.cross_entropy(logits.view(B * S, -1), targets.reshape(-1))
