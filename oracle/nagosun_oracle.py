"""Plain, slow restatement of the Nagosun design in fp32 PyTorch on the CPU: one function per mechanism.

Test infrastructure only; it shares no code with the product path (``pegainfer_b200/nagosun.py`` and the CUDA kernels
behind it).  Weights are a dict ``name -> tensor`` with the checkpoint's tensor names, configuration is the parsed
``config.json`` dict.  Everything is fp32 (float64 where ``dtype`` says so), the attention is the dense
[queries x keys] form with an explicit visibility matrix, and the latent attention expands keys and values per head
(the product path never does).

Nagosun: a decoder on an fp32 residual stream whose every sublayer is wrapped in two grouped RMS norms,

    h = gn(x, w_pre);   x <- x + m * gn(f(h) * logistic(R h + r), w_post),

with f a mixer (grouped-query attention with soft-capped scores, a linear distance bias, a sliding window, a zero-score
sink, unit-RMS values and an element-wise output gate; or latent attention with interleaved rotary pairs and the same
window) or a dense SwiGLU.
"""
from __future__ import annotations

import torch

F32 = torch.float32
SLOPE_LOG2 = 8.0  # head h of H subtracts 2^(-8 (h + 1) / H) * distance from its scores


def f32(t):
    return t.to(F32)


def group_norm(x, weight, groups: int, eps: float):
    """Each of `groups` equal consecutive parts of the last axis is divided by sqrt(mean(part^2) + eps); then times `weight`."""
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)
    return parts.reshape(x.shape) * weight.to(x.dtype)


def unit_rms(x, eps: float):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def visible(pos_q, pos_k, window: int):
    """[queries, keys] bool: a key is seen when it lies d positions behind the query with 0 <= d < window (window 0: any d >= 0)."""
    d = pos_q[:, None] - pos_k[None, :]
    ok = d >= 0
    if window:
        ok &= d < window
    return ok


def distance_slopes(heads: int, dtype=F32):
    return torch.tensor([2.0 ** (-SLOPE_LOG2 * (h + 1) / heads) for h in range(heads)], dtype=dtype)


def soft_cap(s, cap: float):
    return cap * torch.tanh(s / cap) if cap else s


def softmax_plus_one(s, ok):
    """weights e^{s_k} / (1 + sum of e^{s_k'} over the visible keys k'): the softmax over the keys plus one slot of score zero that
    carries no value (computed with the usual shift by the largest score, the extra slot included)."""
    m = torch.where(ok, s, torch.full_like(s, -float("inf"))).max(-1, keepdim=True).values.clamp(min=0.0)
    e = torch.where(ok, torch.exp(s - m), torch.zeros_like(s))
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def attention_mixer(h, w, pre, mx, pos, eps, pos_k=None, h_k=None):
    """h [T, width] -> [T, width].  `h_k` / `pos_k`: the rows that supply keys and values (default: the same rows)."""
    hk = h if h_k is None else h_k
    pk = pos if pos_k is None else pos_k
    H, G, D, Dv = mx["heads"], mx.get("kv_heads") or mx["heads"], mx["dim"], mx["vdim"]
    W = lambda n: w[pre + n].to(h.dtype)  # noqa: E731
    q = (h @ W("q").T + W("q.b")).reshape(-1, H, D)
    k = (hk @ W("k").T + W("k.b")).reshape(-1, G, D)
    v = unit_rms((hk @ W("v").T + W("v.b")).reshape(-1, G, Dv), eps)
    ok = visible(pos, pk, int((mx.get("mask") or {}).get("size", 0)))
    dist = (pos[:, None] - pk[None, :]).to(h.dtype)
    slopes = distance_slopes(H, h.dtype)
    heads = []
    for i in range(H):
        g = i // (H // G)
        s = soft_cap((q[:, i] @ k[:, g].T) * mx["scale"], float(mx.get("softcap") or 0.0)) - slopes[i] * dist
        heads.append(softmax_plus_one(s, ok) @ v[:, g])
    o = torch.cat(heads, -1) * torch.sigmoid(h @ W("g").T)
    return o @ W("o").T + W("o.b")


def rotate_pairs(x, pos, rot):
    """x [T, ..., d]: entries (2i, 2i + 1), i < dims / 2, turn by pos * base^(-2i / dims); entries from `dims` on pass."""
    dims, base = int(rot["dims"]), float(rot["base"])
    if dims == 0:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    a = pos.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    cos, sin = torch.cos(a).to(x.dtype), torch.sin(a).to(x.dtype)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def latent_attention_mixer(h, w, pre, mx, pos, eps):
    """Per token one normed latent c [kv_rank] and one rotated key part [rot_dim] shared by the heads; head keys W_uk c, values W_uv c."""
    H, D, R, Dv, K = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    rot = mx.get("rot") or {"dims": 0, "base": 1.0}
    W = lambda n: w[pre + n].to(h.dtype)  # noqa: E731
    q = (h @ W("q").T).reshape(-1, H, D + R)
    down = h @ W("dkv").T
    c = unit_rms(down[:, :K], eps) * W("dkv.norm")
    k_rot = rotate_pairs(down[:, K:], pos, rot)
    q_rot = rotate_pairs(q[..., D:], pos, rot)
    keys = (c @ W("uk").T).reshape(-1, H, D)
    vals = (c @ W("uv").T).reshape(-1, H, Dv)
    ok = visible(pos, pos, int((mx.get("mask") or {}).get("size", 0)))
    heads = []
    for i in range(H):
        s = (q[:, i, :D] @ keys[:, i].T + q_rot[:, i] @ k_rot.T) * mx["scale"]
        s = torch.where(ok, s, torch.full_like(s, -float("inf")))
        heads.append(torch.softmax(s, -1) @ vals[:, i])
    return torch.cat(heads, -1) @ W("o").T


def swiglu(h, w, pre):
    g = h @ w[pre + "gate"].to(h.dtype).T
    return (g * torch.sigmoid(g) * (h @ w[pre + "up"].to(h.dtype).T)) @ w[pre + "down"].to(h.dtype).T


def result_gate(y, h, w, name):
    """The sublayer's result times logistic(R h + r), element by element."""
    return y * torch.sigmoid(h @ w[name].to(h.dtype).T + w[name + ".b"].to(h.dtype))


def forward(cfg, w, tokens, trail=None, dtype=F32):
    """Logits [T, vocab] of one sequence from position 0; `trail` (a list) receives the residual stream after every layer."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps, groups, m = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1)), float(cfg.get("residual_mult", 1.0))
    gn = lambda x, name: group_norm(x, w[name], groups, eps)  # noqa: E731
    toks = torch.as_tensor(tokens)
    pos = torch.arange(len(toks))
    x = gn(w["embed"][toks], "embed.norm")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = gn(x, p + "norm1")
        mixer = attention_mixer if layer["type"] == "attention" else latent_attention_mixer
        x = x + m * gn(result_gate(mixer(h, w, p + "mix.", layer["mixer"], pos, eps), h, w, p + "rg1"), p + "norm1b")
        if layer.get("mlp"):
            h = gn(x, p + "norm2")
            x = x + m * gn(result_gate(swiglu(h, w, p + "mlp."), h, w, p + "rg2"), p + "norm2b")
        if trail is not None:
            trail.append(x.clone())
    return (gn(x, "final.norm") @ w["head"].T) * float(cfg.get("logit_scale", 1.0))
