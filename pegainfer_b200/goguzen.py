"""The Goguzen design on the layer-list host (``pegainfer_b200/layered.py``, csrc/host/layered_host.cpp).

Goguzen is a pre-norm decoder whose ``config.json`` lists its layers one by one, on an fp32 residual stream:

    x += mixer(rms(x) * w1);   x += ff(rms(x) * w2)        rms(v) = v / sqrt(mean(v^2) + eps)

A layer may carry ``weights_of: j`` instead of tensors of its own: it then runs with layer ``j``'s weights over a cache and a
state of its own.  The embedding is multiplied by ``embedding.scale``; the logits are multiplied by ``logit_scale`` and then
soft-capped, ``cap * tanh(z / cap)``.  Two mixers:

* ``attention`` -- grouped-query attention.  q and k are RMS-normed over their whole projection (all heads at once, weights of
  that size), then the first ``rot.dims`` entries of every head rotate in half-split pairs (entry i with entry i + dims / 2)
  with frequencies that ``rot.scaling`` rescales by wavelength.  A query sees the last ``mask.size`` positions and the first
  ``mask.keep_first`` positions of its sequence.  A learned per-head sink joins the softmax denominator.  Paged K/V cache.
* ``parallel`` -- two branches read the same normed input; each result is RMS-normed over the model width with its own weight
  and the mixer returns half their sum.  ``left`` is attention without a value projection: a head's values are its keys as
  projected; q and k are then RMS-normed head by head (one weight of ``dim`` entries for all heads), nothing rotates, the query
  is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)`` at position p, the mask is plain causal, with a sink.  ``right``
  is a state-space layer: one projection yields ``[z | x | B | C | dt]``; x, B and C pass a short causal convolution with bias
  and SiLU; per head ``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x`` with ``dt = softplus(dt + dt_bias)``; y
  times ``silu(z)`` is RMS-normed in ``norm_groups`` equal parts and projected.  The fp32 state ``S`` and the convolution's last
  inputs live in a per-request state slot.

The feed-forward routes every token to the ``top`` experts with the largest router logits (a bias is added) and weighs them
by the softmax over those logits alone; an always-on shared expert is added.  An expert computes
``g = min(W_gate h, limit)``, ``u = clamp(W_up h, -limit, limit)``, ``W_down (g * logistic(1.702 g) * (u + 1))``.

All sizes and constants come from the configuration; nothing here depends on one particular checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace

import torch

from .layered import LayerCfg, LayeredModel, ModelCfg

MIXER_KINDS = {"attention": 1, "parallel": 4}
GATE_SLOPE = 1.702  # the experts' activation g * logistic(GATE_SLOPE * g), fixed by the design


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0          # mask.size; 0: plain causal
    keep_first: int = 0      # mask.keep_first
    rot_dims: int = 0        # 0: nothing rotates
    rot_base: float = 1.0
    rot_scaling: tuple | None = None  # (factor, low, high, original)
    temp_coef: float = 0.0   # q_temp.coef
    temp_every: int = 0      # q_temp.every; 0: no query factor

    @staticmethod
    def parse(d: dict) -> "AttentionConfig":
        mask, rot, qt = d.get("mask") or {}, d.get("rot") or {}, d.get("q_temp") or {}
        sc = rot.get("scaling")
        return AttentionConfig(int(d["heads"]), int(d.get("kv_heads") or d["heads"]), int(d["dim"]), int(d["vdim"]), float(d["scale"]),
                               int(mask.get("size", 0)), int(mask.get("keep_first", 0)), int(rot.get("dims", 0)), float(rot.get("base", 1.0)),
                               tuple(float(sc[k]) for k in ("factor", "low", "high", "original")) if sc else None,
                               float(qt.get("coef", 0.0)), int(qt.get("every", 0)))

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot_dims:
            d["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
            if self.rot_scaling:
                d["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), self.rot_scaling))
        if self.temp_every:
            d["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return d


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @staticmethod
    def parse(d: dict) -> "StateSpaceConfig":
        return StateSpaceConfig(*(int(d[k]) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))

    def to_dict(self) -> dict:
        return {k: getattr(self, k) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float
    shared_ff: int = 0       # 0: no shared expert
    shared_limit: float = 0.0

    @staticmethod
    def parse(d: dict | None) -> "ExpertsConfig | None":
        if not d:
            return None
        if d.get("kind") != "moe":
            raise ValueError(f"unknown feed-forward kind {d.get('kind')!r}")
        sh = d.get("shared") or {}
        return ExpertsConfig(int(d["router"]["experts"]), int(d["router"]["top"]), int(d["expert"]["ff"]), float(d["expert"]["limit"]),
                             int(sh.get("ff", 0)), float(sh.get("limit", 0.0)))

    def to_dict(self) -> dict:
        d = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class GoguzenLayerConfig:
    kind: str                              # "attention" | "parallel"
    attention: AttentionConfig             # the mixer itself, or the left branch of "parallel"
    state_space: StateSpaceConfig | None   # right branch of "parallel"
    mlp: ExpertsConfig | None
    weights_of: int | None = None

    @staticmethod
    def parse(l: dict) -> "GoguzenLayerConfig":
        kind = l["type"]
        if kind not in MIXER_KINDS:
            raise ValueError(f"unknown mixer type {kind!r}")
        wo = l.get("weights_of")
        if kind == "attention":
            return GoguzenLayerConfig(kind, AttentionConfig.parse(l["mixer"]), None, ExpertsConfig.parse(l.get("mlp")), None if wo is None else int(wo))
        return GoguzenLayerConfig(kind, AttentionConfig.parse(l["mixer"]["left"]), StateSpaceConfig.parse(l["mixer"]["right"]),
                                  ExpertsConfig.parse(l.get("mlp")), None if wo is None else int(wo))

    def to_dict(self) -> dict:
        mixer = self.attention.to_dict() if self.kind == "attention" else {"left": self.attention.to_dict(), "right": self.state_space.to_dict()}
        d = {"type": self.kind, "mixer": mixer, "mlp": self.mlp.to_dict() if self.mlp else None}
        if self.weights_of is not None:
            d["weights_of"] = self.weights_of
        return d


@dataclass(frozen=True)
class GoguzenConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    logit_scale: float
    logit_softcap: float
    layers: tuple = field(default_factory=tuple)
    name: str = "custom"

    @staticmethod
    def from_dict(raw: dict, name: str = "custom") -> "GoguzenConfig":
        layers = [GoguzenLayerConfig.parse(l) for l in raw["layers"]]
        for i, l in enumerate(layers):
            if l.weights_of is None:
                continue
            j, hops = l.weights_of, 0
            while 0 <= j < len(layers) and layers[j].weights_of is not None and hops <= len(layers):
                j, hops = layers[j].weights_of, hops + 1  # a borrower of a borrower runs with the weights at the end of the chain
            if not 0 <= j < len(layers) or layers[j].weights_of is not None:
                raise ValueError(f"layer {i}: weights_of must lead to a layer with weights of its own")
            if j != l.weights_of:
                layers[i] = l = replace(l, weights_of=j)
            o = layers[l.weights_of]
            if (l.kind, l.attention, l.state_space, l.mlp) != (o.kind, o.attention, o.state_space, o.mlp):
                raise ValueError(f"layer {i}: its entry differs from layer {l.weights_of}, whose weights it uses")
        return GoguzenConfig(int(raw["vocab"]), int(raw["width"]), float(raw["norm"]["eps"]), float((raw.get("embedding") or {}).get("scale", 1.0)),
                             float(raw.get("logit_scale", 1.0)), float(raw.get("logit_softcap") or 0.0), tuple(layers), name)

    def to_dict(self) -> dict:
        """The ``config.json`` form (round-trips through ``from_dict``)."""
        d = {"architecture": "Goguzen", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embed_scale}, "logit_scale": self.logit_scale, "layers": [l.to_dict() for l in self.layers]}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d


def weight_shapes(c: GoguzenConfig) -> dict:
    """Checkpoint tensor name -> shape (linear weights are [out, in]).  A layer with ``weights_of`` has no tensors."""
    W = c.width
    s = {"embed": (c.vocab, W)}
    for i, l in enumerate(c.layers):
        if l.weights_of is not None:
            continue
        p, a = f"l{i}.", l.attention
        s[p + "norm1"] = (W,)
        if l.mlp:
            s[p + "norm2"] = (W,)
        m = p + ("mix." if l.kind == "attention" else "mix.left.")
        s[m + "q"], s[m + "k"] = (a.heads * a.dim, W), (a.kv_heads * a.dim, W)
        if l.kind == "attention":
            s[m + "v"] = (a.kv_heads * a.vdim, W)
            s[m + "q.norm"], s[m + "k.norm"] = (a.heads * a.dim,), (a.kv_heads * a.dim,)
        else:
            s[m + "q.norm"], s[m + "k.norm"] = (a.dim,), (a.dim,)
        s[m + "sink"], s[m + "o"] = (a.heads,), (W, a.heads * a.vdim)
        if l.kind == "parallel":
            r, ss = p + "mix.right.", l.state_space
            s[r + "in"] = (2 * ss.inner + 2 * ss.groups * ss.state + ss.heads, W)
            s[r + "conv"], s[r + "conv.b"] = (ss.conv_channels, ss.conv), (ss.conv_channels,)
            s[r + "dt_bias"], s[r + "A_log"], s[r + "D"] = (ss.heads,), (ss.heads,), (ss.heads,)
            s[r + "norm"], s[r + "o"] = (ss.inner,), (W, ss.inner)
            s[p + "mix.left.out"], s[p + "mix.right.out"] = (W,), (W,)
        f = l.mlp
        if f:
            for e in range(f.experts):
                s[f"{p}mlp.e{e}.gate"], s[f"{p}mlp.e{e}.up"], s[f"{p}mlp.e{e}.down"] = (f.ff, W), (f.ff, W), (W, f.ff)
            s[p + "mlp.router"], s[p + "mlp.router.b"] = (f.experts, W), (f.experts,)
            if f.shared_ff:
                s[p + "mlp.shared.gate"], s[p + "mlp.shared.up"], s[p + "mlp.shared.down"] = (f.shared_ff, W), (f.shared_ff, W), (W, f.shared_ff)
    s["final.norm"] = (W,)
    s["head"] = (c.vocab, W)
    return s


def iter_random_weights(c: GoguzenConfig, seed: int = 0, device: str = "cpu"):
    """Random-init checkpoint (bf16): projections N(0, 1/fan_in) so activations stay O(1); norm weights near one; sinks, biases and the
    state-space parameters of order one."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def rn(shape, std=1.0):
        return std * torch.randn(shape, generator=g, device=device)

    for name, shape in weight_shapes(c).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm", "norm1", "norm2", "out"):
            t = 1.0 + 0.1 * rn(shape)
        elif leaf == "conv":
            t = rn(shape, 0.5)
        elif leaf == "A_log":
            t = rn(shape, 0.5) - 1.0
        elif leaf == "D":
            t = 1.0 + 0.2 * rn(shape)
        elif len(shape) == 1:
            t = rn(shape, 0.5 if leaf in ("sink", "dt_bias") else 0.2)
        elif name == "embed":
            t = rn(shape)
        else:
            t = rn(shape) / shape[1] ** 0.5
        yield name, t.to(torch.bfloat16)


# ---------------------------------------------------------------- the model class
def _layer_struct(l: GoguzenLayerConfig) -> LayerCfg:
    a, ss, f = l.attention, l.state_space, l.mlp
    par = l.kind == "parallel"
    sc = a.rot_scaling
    return LayerCfg(heads=a.heads, dim=a.dim, rot_dim=0, vdim=a.vdim, kv_rank=0, kv_from=-1, rot_dims=a.rot_dims, rot_base=a.rot_base, scale=a.scale,
                    has_scaling=int(sc is not None), s_factor=sc[0] if sc else 1.0, s_original=sc[3] if sc else 1.0, s_fast=sc[2] if sc else 1.0,
                    s_slow=sc[1] if sc else 1.0, mlp_kind=2 if f else 0, ff=0, experts=f.experts if f else 0, top=f.top if f else 0, groups=1, keep=1,
                    route_scale=1.0, expert_ff=f.ff if f else 0, shared_ff=f.shared_ff if f else 0, mixer_kind=MIXER_KINDS[l.kind], kv_heads=a.kv_heads,
                    chunk=0, conv=ss.conv if par else 0, rot_interleaved=0, gate_cap=0.0, router_kind=2, expert_act=2, window=a.window, softcap=0.0,
                    slope_log2=0.0, value_norm=0, sink_kind=0, out_gate=0, proj_bias=0, keep_first=a.keep_first, qk_norm=1 if par else 2,
                    q_temp_coef=a.temp_coef, q_temp_every=a.temp_every, values_are_keys=int(par), scaling_kind=1,
                    ssm_heads=ss.heads if par else 0, ssm_vdim=ss.vdim if par else 0, ssm_state=ss.state if par else 0,
                    ssm_groups=ss.groups if par else 0, ssm_norm_groups=ss.norm_groups if par else 0, act_limit=f.limit if f else 0.0,
                    act_slope=GATE_SLOPE, shared_limit=f.shared_limit if f else 0.0, weights_of=-1 if l.weights_of is None else l.weights_of)


def _model_struct(cfg: GoguzenConfig, mc: ModelCfg) -> ModelCfg:
    mc.block_kind, mc.embed_scale, mc.logit_scale, mc.logit_softcap = 3, cfg.embed_scale, cfg.logit_scale, cfg.logit_softcap
    return mc


class GoguzenModel(LayeredModel):
    architecture = "Goguzen"
    config_class = GoguzenConfig
    weight_shapes = staticmethod(weight_shapes)
    layer_struct = staticmethod(_layer_struct)
    model_struct = staticmethod(_model_struct)
