"""The Nagosun design on the layer-list host (``pegainfer_b200/layered.py``, csrc/host/layered_host.cpp).

Nagosun is a decoder whose ``config.json`` lists its layers one by one.  Every sublayer sits in a *sandwich* of grouped RMS
norms on an fp32 residual stream, its result is gated by a logistic projection of its (normed) input, and the sum is scaled:

    h = gn(x, w_pre);   x += m * gn(f(h) * logistic(W_rg h + b_rg), w_post)

where ``gn`` splits a row into ``norm.groups`` equal consecutive parts and divides each by its own root mean square.  The
embedding and the last hidden state pass the same norm; the logits carry a multiplier.  Two mixers:

* ``attention`` -- grouped-query attention with projection biases and no rotary embedding: the only position signal is a linear
  distance bias (head ``h`` of ``H`` subtracts ``2^(-8 (h + 1) / H)`` times the distance from the score).  The scaled score is
  soft-capped (``cap * tanh(s / cap)``) before the bias; a sliding window limits the visible keys; the softmax denominator
  carries a sink of score zero (one is added to it); cached values are unit-RMS per head; the concatenated heads are multiplied
  by ``logistic(W_g h)`` before the output projection.  Paged K/V cache.
* ``latent_attention`` -- attention over a compressed cache (one normed latent vector plus one rotated key part per token,
  shared by all heads; keys and values of a head are linear maps of the latent), interleaved rotary pairs on the rotated
  parts, the same sliding window, ordinary softmax.

The feed-forward is a dense SwiGLU or absent.  All sizes and constants come from the configuration; nothing here depends on
one particular checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .layered import LayerCfg, LayeredModel, ModelCfg
from .vamadra import RotaryConfig

MIXER_KINDS = {"latent_attention": 0, "attention": 1}
BIAS_SLOPE_LOG2 = 8.0  # head h of H: slope 2^(-8 (h + 1) / H), fixed by the design


@dataclass(frozen=True)
class MixerConfig:
    kind: str            # "attention" | "latent_attention"
    heads: int
    dim: int             # query/key entries per head (latent attention: the unrotated ones)
    vdim: int
    scale: float
    window: int = 0      # mask.size; 0: plain causal
    kv_heads: int = 0    # attention
    softcap: float = 0.0  # attention; 0: no cap
    rot_dim: int = 0     # latent attention: rotated entries per head (the key part of this width is shared by all heads)
    kv_rank: int = 0     # latent attention
    rot: RotaryConfig | None = None

    @staticmethod
    def parse(kind: str, d: dict) -> "MixerConfig":
        if kind not in MIXER_KINDS:
            raise ValueError(f"unknown mixer type {kind!r}")
        heads, dim, vdim, scale = int(d["heads"]), int(d["dim"]), int(d["vdim"]), float(d["scale"])
        window = int((d.get("mask") or {}).get("size", 0))
        if kind == "attention":
            return MixerConfig(kind, heads, dim, vdim, scale, window, kv_heads=int(d.get("kv_heads") or heads), softcap=float(d.get("softcap") or 0.0))
        rot_dim = int(d["rot_dim"])
        rot = RotaryConfig.parse(d["rot"]) if d.get("rot") else RotaryConfig(0, 1.0, None)
        return MixerConfig(kind, heads, dim, vdim, scale, window, rot_dim=rot_dim, kv_rank=int(d["kv_rank"]), rot=rot)

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.kind == "attention":
            d["kv_heads"] = self.kv_heads
            if self.softcap:
                d["softcap"] = self.softcap
        else:
            d.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank)
            if self.rot and self.rot.dims:
                d["rot"] = {"dims": self.rot.dims, "base": self.rot.base}
        return d


@dataclass(frozen=True)
class NagosunLayerConfig:
    mixer: MixerConfig
    ff: int = 0          # hidden size of the dense feed-forward; 0: none


@dataclass(frozen=True)
class NagosunConfig:
    vocab: int
    width: int
    eps: float
    groups: int
    residual_mult: float
    logit_scale: float
    layers: tuple = field(default_factory=tuple)
    name: str = "custom"

    @staticmethod
    def from_dict(raw: dict, name: str = "custom") -> "NagosunConfig":
        layers = []
        for i, l in enumerate(raw["layers"]):
            mlp = l.get("mlp")
            if mlp and mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            layers.append(NagosunLayerConfig(MixerConfig.parse(l["type"], l["mixer"]), int(mlp["ff"]) if mlp else 0))
        width, groups = int(raw["width"]), int(raw["norm"].get("groups", 1))
        if groups <= 0 or width % groups:
            raise ValueError(f"norm.groups {groups} does not divide the width {width}")
        return NagosunConfig(int(raw["vocab"]), width, float(raw["norm"]["eps"]), groups, float(raw.get("residual_mult", 1.0)),
                             float(raw.get("logit_scale", 1.0)), tuple(layers), name)

    def to_dict(self) -> dict:
        """The ``config.json`` form (round-trips through ``from_dict``)."""
        return {"architecture": "Nagosun", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps, "groups": self.groups},
                "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
                "layers": [{"type": l.mixer.kind, "mixer": l.mixer.to_dict(), "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None}
                           for l in self.layers]}


def weight_shapes(c: NagosunConfig) -> dict:
    """Checkpoint tensor name -> shape (linear weights are [out, in], a bias is the weight's name + '.b')."""
    W = c.width
    s = {"embed": (c.vocab, W), "embed.norm": (W,)}
    for i, l in enumerate(c.layers):
        m, p = l.mixer, f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if l.ff else ()):
            s[p + n] = (W,)
        H, D, Dv = m.heads, m.dim, m.vdim
        if m.kind == "attention":
            for n, rows in (("q", H * D), ("k", m.kv_heads * D), ("v", m.kv_heads * Dv)):
                s[p + "mix." + n], s[p + "mix." + n + ".b"] = (rows, W), (rows,)
            s[p + "mix.g"] = (H * Dv, W)
            s[p + "mix.o"], s[p + "mix.o.b"] = (W, H * Dv), (W,)
        else:
            s[p + "mix.q"] = (H * (D + m.rot_dim), W)
            s[p + "mix.dkv"], s[p + "mix.dkv.norm"] = (m.kv_rank + m.rot_dim, W), (m.kv_rank,)
            s[p + "mix.uk"], s[p + "mix.uv"] = (H * D, m.kv_rank), (H * Dv, m.kv_rank)
            s[p + "mix.o"] = (W, H * Dv)
        if l.ff:
            s[p + "mlp.gate"], s[p + "mlp.up"], s[p + "mlp.down"] = (l.ff, W), (l.ff, W), (W, l.ff)
        for n in ("rg1",) + (("rg2",) if l.ff else ()):
            s[p + n], s[p + n + ".b"] = (W, W), (W,)
    s["final.norm"] = (W,)
    s["head"] = (c.vocab, W)
    return s


def iter_random_weights(c: NagosunConfig, seed: int = 0, device: str = "cpu"):
    """Random-init checkpoint (bf16): projections N(0, 1/fan_in) so activations stay O(1), norm weights near one, biases small."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    for name, shape in weight_shapes(c).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf.startswith("norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=device)
        elif len(shape) == 1:
            t = 0.2 * torch.randn(shape, generator=g, device=device)
        elif name == "embed":
            t = torch.randn(shape, generator=g, device=device)
        else:
            t = torch.randn(shape, generator=g, device=device) / shape[1] ** 0.5
        yield name, t.to(torch.bfloat16)


# ---------------------------------------------------------------- the model class
def _layer_struct(l: NagosunLayerConfig) -> LayerCfg:
    m = l.mixer
    att = m.kind == "attention"
    rot = m.rot if m.rot else RotaryConfig(0, 1.0, None)
    return LayerCfg(heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, kv_from=-1, rot_dims=0 if att else rot.dims,
                    rot_base=rot.base, scale=m.scale, has_scaling=0, s_factor=1.0, s_original=1.0, s_fast=1.0, s_slow=1.0,
                    mlp_kind=1 if l.ff else 0, ff=l.ff, experts=0, top=0, groups=1, keep=1, route_scale=1.0, expert_ff=0, shared_ff=0,
                    mixer_kind=MIXER_KINDS[m.kind], kv_heads=m.kv_heads if att else 1, chunk=0, conv=0, rot_interleaved=1, gate_cap=0.0,
                    router_kind=0, expert_act=0, window=m.window, softcap=m.softcap if att else 0.0, slope_log2=BIAS_SLOPE_LOG2 if att else 0.0,
                    value_norm=int(att), sink_kind=2 if att else 1, out_gate=int(att), proj_bias=int(att))


def _model_struct(cfg: NagosunConfig, mc: ModelCfg) -> ModelCfg:
    mc.block_kind, mc.logit_scale, mc.norm_groups, mc.residual_mult, mc.gated_residual = 2, cfg.logit_scale, cfg.groups, cfg.residual_mult, 1
    return mc


class NagosunModel(LayeredModel):
    architecture = "Nagosun"
    config_class = NagosunConfig
    weight_shapes = staticmethod(weight_shapes)
    layer_struct = staticmethod(_layer_struct)
    model_struct = staticmethod(_model_struct)
