"""Plain, slow restatement of the Goguzen design in PyTorch on the CPU: one function per mechanism.

Test infrastructure only; it shares no code with the product path (``pegainfer_b200/goguzen.py`` and the CUDA kernels
behind it).  Weights are a dict ``name -> tensor`` with the checkpoint's tensor names, configuration is the parsed
``config.json`` dict.  Everything runs in one floating type (fp32, or fp64 where ``dtype`` says so); attention is the dense
[queries x keys] form with an explicit visibility matrix, the state-space recurrence runs token by token, and every
token visits its experts one after the other.

Goguzen: a pre-norm decoder on a residual stream, ``x <- x + mixer(rms(x) w1)``, ``x <- x + ff(rms(x) w2)``.  Mixers:

* ``attention`` -- grouped-query softmax attention; q and k are RMS-normed over their WHOLE projection (all heads at once),
  then the first ``rot.dims`` entries of every head turn in half-split pairs with frequencies rescaled by wavelength; a
  query sees the last ``mask.size`` positions and, besides, the first ``mask.keep_first`` positions of the sequence; a
  learned per-head sink sits in the softmax denominator.
* ``parallel`` -- two branches read the same input.  Left: attention without a value projection (a head's values are its
  keys as projected, the keys it scores with are RMS-normed per head afterwards), no rotation, queries stretched by a factor
  that grows with the logarithm of the position, plain causal mask, sink.  Right: a selective state-space layer (scalar decay per
  head, short causal convolution, gated and group-normed read-out).  Each branch's result is RMS-normed over the width and
  the mixer returns the mean of the two.

Feed-forward: routed experts (the ``top`` largest router logits, weights = softmax over those logits alone) plus an always-on
shared expert; an expert is a gated unit with clamped pre-activations.  Layers may borrow another layer's weights.  The
logits are scaled and soft-capped.
"""
from __future__ import annotations

import math

import torch

F32 = torch.float32
GATE_SLOPE = 1.702        # expert activation: g * logistic(GATE_SLOPE * g)


def rms(x, eps: float):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


# ---------------------------------------------------------------- positions
def rescaled_frequencies(rot: dict):
    """Angular frequency of every rotated pair [dims / 2] in float64.  Pair i turns at base^(-2i / dims); with ``scaling`` a pair
    whose wavelength exceeds original / low is slowed by ``factor``, one below original / high is kept, and in between the two are
    blended linearly in original / wavelength."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
    wavelength = 2.0 * math.pi / f
    blend = ((orig / wavelength - low) / (high - low))
    mid = (1.0 - blend) * f / factor + blend * f
    return torch.where(wavelength < orig / high, f, torch.where(wavelength > orig / low, f / factor, mid))


def rotate_halves(x, pos, rot):
    """x [T, heads, d]: entry i pairs with entry i + dims / 2 (i < dims / 2); entries from ``dims`` on pass unchanged."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    half = dims // 2
    a = pos.to(torch.float64)[:, None] * rescaled_frequencies(rot)[None, :]
    cos, sin = torch.cos(a).to(x.dtype)[:, None, :], torch.sin(a).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def query_stretch(pos, q_temp: dict, dtype):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    steps = torch.div(pos + 1, int(q_temp["every"]), rounding_mode="floor")
    return 1.0 + float(q_temp["coef"]) * torch.log(steps.to(dtype) + 1.0)


def visible(pos_q, pos_k, size: int = 0, keep_first: int = 0):
    """[queries, keys] bool.  Causal; with ``size`` only keys fewer than ``size`` positions behind, or among the first ``keep_first``."""
    d = pos_q[:, None] - pos_k[None, :]
    ok = d >= 0
    if size:
        ok = ok & ((d < size) | (pos_k[None, :] < keep_first))
    return ok


def softmax_with_sink(s, ok, sink):
    """Softmax over the visible keys of every row with one more term exp(sink) in the denominator (no value goes with it)."""
    s = torch.where(ok, s, torch.full_like(s, -float("inf")))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def grouped_heads_attention(q, k, v, ok, scale, sinks):
    """q [T, H, D], k [S, G, D], v [S, G, Dv] -> [T, H * Dv]; query head h reads key/value head h // (H / G)."""
    H, G = q.shape[1], k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        p = softmax_with_sink((q[:, h] @ k[:, g].T) * scale, ok, sinks[h])
        out.append(p @ v[:, g])
    return torch.cat(out, -1)


# ---------------------------------------------------------------- mixers
def windowed_attention(h, w, pre, mx, pos, eps):
    """The ``attention`` mixer for one sequence: h [T, width] at positions ``pos`` (all keys of the sequence are among the rows)."""
    H, G, D, Dv = int(mx["heads"]), int(mx.get("kv_heads") or mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    W = lambda n: w[pre + n].to(h.dtype)  # noqa: E731
    q = rms(h @ W("q").T, eps) * W("q.norm")          # one RMS over the H * D entries
    k = rms(h @ W("k").T, eps) * W("k.norm")
    v = (h @ W("v").T).reshape(-1, G, Dv)
    q, k = q.reshape(-1, H, D), k.reshape(-1, G, D)
    if mx.get("rot"):
        q, k = rotate_halves(q, pos, mx["rot"]), rotate_halves(k, pos, mx["rot"])
    mask = mx.get("mask") or {}
    ok = visible(pos, pos, int(mask.get("size", 0)), int(mask.get("keep_first", 0)))
    return grouped_heads_attention(q, k, v, ok, float(mx["scale"]), W("sink")) @ W("o").T


def keys_as_values_attention(h, w, pre, mx, pos, eps):
    """Left branch of ``parallel``: v = k as projected; q and k are then RMS-normed head by head with one weight for all heads."""
    H, G, D = int(mx["heads"]), int(mx.get("kv_heads") or mx["heads"]), int(mx["dim"])
    W = lambda n: w[pre + n].to(h.dtype)  # noqa: E731
    q = (h @ W("q").T).reshape(-1, H, D)
    k = (h @ W("k").T).reshape(-1, G, D)
    v = k
    q = rms(q, eps) * W("q.norm")
    k = rms(k, eps) * W("k.norm")
    if mx.get("q_temp"):
        q = q * query_stretch(pos, mx["q_temp"], h.dtype)[:, None, None]
    ok = visible(pos, pos)
    return grouped_heads_attention(q, k, v, ok, float(mx["scale"]), W("sink")) @ W("o").T


def causal_conv(x, weight, bias, tail=None):
    """x [T, C]; weight [C, taps] whose LAST column multiplies the current token; zeros (or ``tail`` [taps - 1, C]) before the start."""
    taps = weight.shape[1]
    pad = torch.zeros(taps - 1, x.shape[1], dtype=x.dtype) if tail is None else tail
    xp = torch.cat([pad, x], 0)
    out = bias.expand(x.shape[0], -1).clone()
    for j in range(taps):
        out = out + xp[j:j + x.shape[0]] * weight[:, j]
    return out


def state_space_branch(h, w, pre, mx, eps, state=None):
    """Right branch of ``parallel`` for one sequence, token by token.  ``state`` = (S [heads, N, P], conv tail [taps - 1, C]) or None
    for a fresh sequence; returns (output [T, width], new state)."""
    Hs, P, N, Gs, taps, ng = int(mx["heads"]), int(mx["vdim"]), int(mx["state"]), int(mx["groups"]), int(mx["conv"]), int(mx["norm_groups"])
    inner, C = Hs * P, Hs * P + 2 * Gs * N
    W = lambda n: w[pre + n].to(h.dtype)  # noqa: E731
    T = h.shape[0]
    proj = h @ W("in").T
    z, xbc, dt = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
    S, tail = (torch.zeros(Hs, N, P, dtype=h.dtype), torch.zeros(taps - 1, C, dtype=h.dtype)) if state is None else state
    conv = causal_conv(xbc, W("conv"), W("conv.b"), tail)
    new_tail = torch.cat([tail, xbc], 0)[T:T + taps - 1] if taps > 1 else tail
    conv = conv * torch.sigmoid(conv)
    xs, B, Cm = conv[:, :inner].reshape(T, Hs, P), conv[:, inner:inner + Gs * N].reshape(T, Gs, N), conv[:, inner + Gs * N:].reshape(T, Gs, N)
    dt = torch.nn.functional.softplus(dt + W("dt_bias"), threshold=1e9)
    decay = torch.exp(-torch.exp(W("A_log")) * dt)                 # [T, heads]
    y = torch.empty(T, Hs, P, dtype=h.dtype)
    S = S.clone()
    for t in range(T):
        for hd in range(Hs):
            g = hd // (Hs // Gs)
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], xs[t, hd])
            y[t, hd] = S[hd].T @ Cm[t, g] + W("D")[hd] * xs[t, hd]
    y = y.reshape(T, inner) * (z * torch.sigmoid(z))
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W("norm")
    return y @ W("o").T, (S, new_tail)


def parallel_mixer(h, w, pre, mx, pos, eps):
    left = keys_as_values_attention(h, w, pre + "left.", mx["left"], pos, eps)
    right, _ = state_space_branch(h, w, pre + "right.", mx["right"], eps)
    return 0.5 * (rms(left, eps) * w[pre + "left.out"].to(h.dtype) + rms(right, eps) * w[pre + "right.out"].to(h.dtype))


# ---------------------------------------------------------------- feed-forward
def clamped_expert(h, w, pre, limit: float):
    g = (h @ w[pre + "gate"].to(h.dtype).T).clamp(max=limit)
    u = (h @ w[pre + "up"].to(h.dtype).T).clamp(-limit, limit)
    return (g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0)) @ w[pre + "down"].to(h.dtype).T


def route(h, w, pre, top: int):
    """(expert ids [T, top], weights [T, top]): the largest logits, softmax over those alone."""
    z = h @ w[pre + "router"].to(h.dtype).T + w[pre + "router.b"].to(h.dtype)
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, -1)


def expert_mixture(h, w, pre, mlp):
    top = int(mlp["router"]["top"])
    idx, wt = route(h, w, pre, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += wt[t, j] * clamped_expert(h[t:t + 1], w, f"{pre}e{int(idx[t, j])}.", float(mlp["expert"]["limit"]))[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, pre + "shared.", float(mlp["shared"]["limit"]))
    return out


# ---------------------------------------------------------------- the model
def forward(cfg, w, tokens, trail=None, dtype=F32):
    """Logits [T, vocab] of one sequence from position 0; ``trail`` (a list) receives the residual stream after every layer."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    toks = torch.as_tensor(tokens)
    pos = torch.arange(len(toks))
    x = w["embed"][toks] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{int(layer.get('weights_of', i))}."
        h = rms(x, eps) * w[p + "norm1"]
        if layer["type"] == "attention":
            x = x + windowed_attention(h, w, p + "mix.", layer["mixer"], pos, eps)
        else:
            x = x + parallel_mixer(h, w, p + "mix.", layer["mixer"], pos, eps)
        if layer.get("mlp"):
            x = x + expert_mixture(rms(x, eps) * w[p + "norm2"], w, p + "mlp.", layer["mlp"])
        if trail is not None:
            trail.append(x.clone())
    z = (rms(x, eps) * w["final.norm"]) @ w["head"].T * float(cfg.get("logit_scale", 1.0))
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap else z
