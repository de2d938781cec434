"""Fovunex adapter: a text-only decoder-only LM on ``HybridEngine`` (hybrid_engine.py) built from pre-norm layers with
gated residuals, x += sigmoid(W_r h + b) * sublayer(h) with h = norm(x), around an fp32 stream; every norm of the stack
is an RMS norm with ONE number as its weight; the embedding is multiplied by a constant.  A span of layers may run
several times in a row with the same weights (``loop``): each pass has its own cache or state, and the embedding output
is added to the stream again before every pass but the first.

  * mixers, in any order the configuration gives:
      latent attention -- queries straight from the input, heads of ``dim`` unrotated + ``rot_dim`` rotated dims; keys'
        unrotated parts and values are per-head expansions of one normed latent per token, the rotated key part is one
        vector per token shared by all heads; interleaved rotary pairs with YaRN frequency scaling; only [latent |
        rotated key part] is cached;
      attention with two score maps per head over the same values (o = a1 - lambda a2, unit RMS per head, times
        1 - diff), grouped key/value heads, query/key RMS norm per head and map, rotary positions on (i, i + dims/2)
        pairs, visibility restricted to the position's own chunk, sigmoid output gate;
      minGRU -- an element-wise gated recurrence over an fp32 state per request.
  * feed-forward: none, or down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate h, limit), u = clamp(up h, +-limit).
  * output: scalar-weight RMS norm, head.

Everything a model of this design can vary is read from its ``config.json``; serving (worker, scheduler, pages, slots,
sampler, command lines) is what ``BobavikModel`` set up for hybrid-engine designs.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .._lib import VoxB200Error
from ..hybrid_engine import (DiffAttentionConfig, GluMLPConfig, HybridConfig, HybridLayerConfig, LatentAttentionConfig,
                             MinGRUConfig, RotaryConfig)
from .bobavik import BobavikModel

GLU_SLOPE = 1.702        # the feed-forward's gate is g * sigmoid(1.702 g)


def _rotary(r: Optional[Dict[str, Any]], layout: str) -> Optional[RotaryConfig]:
    if not r:
        return None
    sc = r.get("scaling") or None
    if sc:
        return RotaryConfig(int(r["dims"]), float(r["base"]), float(sc["factor"]), original=float(sc["original"]),
                            layout=layout, scaling="yarn", fast=float(sc["fast"]), slow=float(sc["slow"]))
    return RotaryConfig(int(r["dims"]), float(r["base"]), layout=layout)


def fovunex_config(c: Dict[str, Any]) -> HybridConfig:
    """config.json -> HybridConfig.  Keys: ``width``, ``vocab``, ``norm.eps``, ``embedding.scale``, ``loop`` {start, stop,
    times} (optional) and ``layers``: per layer ``type`` (latent_attention | attention | mingru), ``mixer`` (latent_attention:
    heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims, scaling {factor, original, fast, slow}?}?; attention: heads,
    kv_heads, dim, vdim, scale, diff, mask {size}?, rot {base, dims}?; mingru: width) and ``mlp``: null or {kind: dense, ff,
    limit}."""
    layers = []
    for i, L in enumerate(c["layers"]):
        kind, m = L["type"], L["mixer"]
        if kind == "latent_attention":
            rot_dim = int(m.get("rot_dim", 0) or 0)
            rot = _rotary(m.get("rot"), "interleaved") if rot_dim else None
            mixer = LatentAttentionConfig(int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), int(m["kv_rank"]), 0,
                                          float(m["scale"]), None, rot_dim=rot_dim, rotary=rot, head_gate=False)
            if rot is not None and (rot.dims > rot_dim or rot.dims % 2):
                raise VoxB200Error(f"layer {i}: rotary dims {rot.dims} do not fit the rotated part of {rot_dim} dims")
            layer = HybridLayerConfig("latent", mixer)
        elif kind == "attention":
            H, G = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
            if G <= 0 or H % G:
                raise VoxB200Error(f"layer {i}: {H} heads do not divide into {G} key/value heads")
            mask = m.get("mask") or {}
            mixer = DiffAttentionConfig(H, G, int(m["dim"]), int(m.get("vdim", m["dim"])), float(m["scale"]), float(m["diff"]),
                                        chunk=int(mask.get("size", 0) or 0), rotary=_rotary(m.get("rot"), "half"))
            layer = HybridLayerConfig("diff_attention", mixer)
        elif kind == "mingru":
            layer = HybridLayerConfig("mingru", MinGRUConfig(int(m["width"])))
        else:
            raise VoxB200Error(f"layer {i}: unknown mixer type '{kind}'")
        f = L.get("mlp")
        if f:
            if f.get("kind", "dense") != "dense":
                raise VoxB200Error(f"layer {i}: unknown feed-forward kind '{f.get('kind')}'")
            layer.mlp = GluMLPConfig(int(f["ff"]), float(f["limit"]), GLU_SLOPE)
            if layer.mlp.limit <= 0:
                raise VoxB200Error(f"layer {i}: the feed-forward's limit must be positive")
        layers.append(layer)
    loop = c.get("loop") or {}
    a, b, times = int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))
    if not (0 <= a <= len(layers) and b <= len(layers) and times >= 0):
        raise VoxB200Error(f"loop {loop} does not fit {len(layers)} layers")
    return HybridConfig(int(c["width"]), int(c["vocab"]), float(c["norm"]["eps"]), 1.0, layers, block="gated",
                        norm="rmsnorm_scalar", embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)),
                        loop_start=a, loop_stop=b, loop_times=times)


def synthetic_state_dict(cfg: HybridConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """Seeded random weights with the checkpoint's names (bf16), generated on ``device``."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = cfg.width

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(tuple(shape), generator=g, device=device) * std + mean).to(torch.bfloat16)

    sd = {"embed": rnd(cfg.vocab, W), "head": rnd(cfg.vocab, W, std=W ** -0.5), "final.norm": rnd(std=0.1, mean=1.0)}
    s = W ** -0.5
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        sd[p + "norm1"], sd[p + "rg1"], sd[p + "rg1.b"] = rnd(std=0.1, mean=1.0), rnd(W, W, std=s), rnd(W, std=0.5)
        if L.kind == "latent":
            sd[p + "mix.q"] = rnd(m.heads * (m.dim + m.rot_dim), W, std=s)
            sd[p + "mix.dkv"], sd[p + "mix.dkv.norm"] = rnd(m.kv_rank + m.rot_dim, W, std=s), rnd(m.kv_rank, std=0.1, mean=1.0)
            sd[p + "mix.uk"] = rnd(m.heads * m.dim, m.kv_rank, std=m.kv_rank ** -0.5)
            sd[p + "mix.uv"] = rnd(m.heads * m.vdim, m.kv_rank, std=m.kv_rank ** -0.5)
            sd[p + "mix.o"] = rnd(W, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
        elif L.kind == "diff_attention":
            sd[p + "mix.q"], sd[p + "mix.k"] = rnd(m.heads * 2 * m.dim, W, std=s), rnd(m.kv_heads * 2 * m.dim, W, std=s)
            sd[p + "mix.v"], sd[p + "mix.g"] = rnd(m.kv_heads * m.vdim, W, std=s), rnd(m.heads * m.vdim, W, std=s)
            sd[p + "mix.q.norm"], sd[p + "mix.k.norm"] = rnd(m.dim, std=0.1, mean=1.0), rnd(m.dim, std=0.1, mean=1.0)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                sd[p + "mix." + n] = rnd(m.dim, std=0.1)
            sd[p + "mix.o"] = rnd(W, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
        else:
            for n in ("z", "x", "g"):
                sd[p + "mix." + n] = rnd(m.width, W, std=s)
            sd[p + "mix.z.b"], sd[p + "mix.x.b"] = rnd(m.width, std=0.5), rnd(m.width, std=0.5)
            sd[p + "mix.o"] = rnd(W, m.width, std=m.width ** -0.5)
        f = L.mlp
        if f is not None:
            sd[p + "norm2"], sd[p + "rg2"], sd[p + "rg2.b"] = rnd(std=0.1, mean=1.0), rnd(W, W, std=s), rnd(W, std=0.5)
            sd[p + "mlp.gate"], sd[p + "mlp.up"] = rnd(f.ff, W, std=s), rnd(f.ff, W, std=s)
            sd[p + "mlp.down"] = rnd(W, f.ff, std=f.ff ** -0.5)
    return sd


class FovunexModel(BobavikModel):
    design = "Fovunex"
    synthetic_name = "fovunex-synthetic"
    has_recurrent_state = True
    build_profile = "text_gated"

    @staticmethod
    def read_config(config: Dict[str, Any]) -> HybridConfig:
        return fovunex_config(config)

    @staticmethod
    def synthetic_weights(cfg: HybridConfig, seed: int, device) -> Dict[str, torch.Tensor]:
        return synthetic_state_dict(cfg, seed, device)
