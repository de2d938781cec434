"""Nadevik adapter: a text-only decoder-only LM on ``HybridEngine`` (hybrid_engine.py) whose layers norm only what a sublayer
puts out, x += norm1(mixer(c(x))) and x += norm2(ff(x)) around an fp32 stream: the sublayers read the stream itself, the
mixer through an input convolution c(h) = h + conv(h) over time on every channel.  Every norm is an RMS norm whose stored
weight is an offset from one.  The embedding is multiplied by a constant and a second, hashed embedding of the (previous
token, token) pair is added; the output head is the embedding table itself.

  * mixers, in any order the configuration gives:
      latent attention -- queries straight from the input, heads of ``dim`` unrotated + ``rot_dim`` rotated dims; keys'
        unrotated parts and values are per-head expansions of one normed latent per token, the rotated key part is one
        vector per token shared by all heads (interleaved rotary pairs); sliding window; softmax; the concatenated heads
        times sigmoid(W_g h); a layer may read the rows an earlier layer cached (``kv_from``) instead of projecting its own;
      a pair of mixers side by side on the same input, left_scale * left + right_scale * right:
        left -- grouped-head attention without rotation: short causal convolutions on q, k, v right after their projection,
          RMS norm of q and of k over the whole projection, soft-capped scores, a sliding window plus one pooled (mean) key /
          value per block of positions entirely older than the window, weights sigmoid(score + bias of the head) that are not
          normalised over the keys;
        right -- a selective scan (Mamba form) over an fp32 state per request.
  * feed-forward: none, or a mixture of clamped gated experts, down(g * sigmoid(1.702 g) * (u + 1)) with g = min(gate h,
    limit), u = clamp(up h, +-limit), behind a router that scores all experts with one softmax, keeps the groups of
    neighbours with the largest best score, takes the ``top`` largest scores among them and weighs the chosen experts by
    those scores as they are.
  * output: the stack's norm, then the embedding table (without the embedding's constant) as the head.

Per request the design keeps, beside the pages of its attention layers: the pooled blocks, the scan's state, the last inputs
of every short convolution and of every layer's input convolution, and the last token (for the pair embedding) -- all in the
request's slot of ``HybridCache``.  Everything a model of this design can vary is read from its ``config.json``; serving
(worker, scheduler, pages, slots, sampler, command lines) is what ``BobavikModel`` set up for hybrid-engine designs.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from .._lib import VoxB200Error
from ..hybrid_engine import (HybridConfig, HybridLayerConfig, LatentAttentionConfig, MixerPairConfig, MoEConfig, PairEmbedConfig,
                             PooledSigmoidAttentionConfig, RotaryConfig, SelectiveScanConfig)
from .bobavik import BobavikModel

GLU_SLOPE = 1.702        # the experts' gate is g * sigmoid(1.702 g)


def _mask(m: Dict[str, Any], key: str) -> int:
    return int((m.get("mask") or {}).get(key, 0) or 0)


def nadevik_config(c: Dict[str, Any]) -> HybridConfig:
    """config.json -> HybridConfig.  Keys: ``width``, ``vocab``, ``norm.eps``, ``embedding`` {scale, bigram {buckets, mul_prev,
    mul_cur}?}, ``canon.taps`` and ``layers``: per layer ``type`` (latent_attention | parallel), ``mixer`` (latent_attention:
    heads, dim, rot_dim, vdim, kv_rank, scale, mask {size}?, rot {base, dims}?, kv_from?; parallel: left {heads, kv_heads, dim,
    vdim, scale, softcap, conv, mask {size, pool}}, right {inner, state, dt_rank, conv}, left_scale, right_scale) and ``mlp``:
    null or {kind: moe, expert {ff, limit}, router {experts, top, groups {count, keep}?}}."""
    layers = []
    for i, L in enumerate(c["layers"]):
        kind, m = L["type"], L["mixer"]
        if kind == "latent_attention":
            rot_dim = int(m.get("rot_dim", 0) or 0)
            r = m.get("rot") if rot_dim else None
            rot = RotaryConfig(int(r["dims"]), float(r["base"]), layout="interleaved") if r else None
            if rot is not None and (rot.dims > rot_dim or rot.dims % 2):
                raise VoxB200Error(f"layer {i}: rotary dims {rot.dims} do not fit the rotated part of {rot_dim} dims")
            src = m.get("kv_from")
            mixer = LatentAttentionConfig(int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])), int(m["kv_rank"]), 0,
                                          float(m["scale"]), None if src is None else int(src), rot_dim=rot_dim, rotary=rot,
                                          head_gate=False, window=_mask(m, "size"), value_gate=True)
            layer = HybridLayerConfig("latent", mixer)
        elif kind == "parallel":
            a, r = m["left"], m["right"]
            H, G = int(a["heads"]), int(a.get("kv_heads", a["heads"]))
            if G <= 0 or H % G:
                raise VoxB200Error(f"layer {i}: {H} heads do not divide into {G} key/value heads")
            left = PooledSigmoidAttentionConfig(H, G, int(a["dim"]), int(a.get("vdim", a["dim"])), float(a["scale"]),
                                                window=_mask(a, "size"), pool=_mask(a, "pool"),
                                                softcap=float(a.get("softcap", 0.0) or 0.0), conv=int(a.get("conv", 0) or 0))
            right = SelectiveScanConfig(int(r["inner"]), int(r["state"]), int(r["dt_rank"]), int(r["conv"]))
            layer = HybridLayerConfig("mixer_pair", MixerPairConfig(left, right, float(m.get("left_scale", 1.0)),
                                                                    float(m.get("right_scale", 1.0))))
        else:
            raise VoxB200Error(f"layer {i}: unknown mixer type '{kind}'")
        f = L.get("mlp")
        if f:
            if f.get("kind", "moe") != "moe":
                raise VoxB200Error(f"layer {i}: unknown feed-forward kind '{f.get('kind')}'")
            rt, gr = f["router"], (f["router"].get("groups") or {})
            E, top = int(rt["experts"]), int(rt["top"])
            count, keep = int(gr.get("count", 0) or 0), int(gr.get("keep", 0) or 0)
            if count > 1 and (E % count or not 1 <= keep <= count or keep * (E // count) < top):
                raise VoxB200Error(f"layer {i}: {count} groups (keep {keep}) do not fit {E} experts, top {top}")
            layer.mlp = MoEConfig(E, top, int(f["expert"]["ff"]), act="clamped_glu", router="softmax_all", groups=count,
                                  groups_keep=keep, limit=float(f["expert"]["limit"]), slope=GLU_SLOPE)
            if layer.mlp.limit <= 0 or not 1 <= top <= E:
                raise VoxB200Error(f"layer {i}: the experts' limit must be positive and 1 <= top <= experts")
        layers.append(layer)
    e = c.get("embedding") or {}
    b = e.get("bigram")
    pair = PairEmbedConfig(int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])) if b else None
    return HybridConfig(int(c["width"]), int(c["vocab"]), float(c["norm"]["eps"]), 1.0, layers, block="post",
                        norm="rmsnorm_offset", embed_scale=float(e.get("scale", 1.0)), tied_head=True, pair_embed=pair,
                        input_conv=int((c.get("canon") or {}).get("taps", 0) or 0))


def synthetic_state_dict(cfg: HybridConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """Seeded random weights with the checkpoint's names (bf16), generated on ``device``."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = cfg.width

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(tuple(shape), generator=g, device=device) * std + mean).to(torch.bfloat16)

    sd = {"embed": rnd(cfg.vocab, W, std=W ** -0.5), "final.norm": rnd(W, std=0.1)}
    if cfg.pair_embed is not None:
        sd["bigram"] = rnd(cfg.pair_embed.buckets + 1, W, std=0.5)
    s = W ** -0.5
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        sd[p + "norm1"] = rnd(W, std=0.1)
        if cfg.input_conv:
            sd[p + "canon1"] = rnd(W, cfg.input_conv, std=0.3)
        if L.kind == "latent":
            sd[p + "mix.q"] = rnd(m.heads * (m.dim + m.rot_dim), W, std=s)
            if m.kv_from is None:
                sd[p + "mix.dkv"], sd[p + "mix.dkv.norm"] = rnd(m.kv_rank + m.rot_dim, W, std=s), rnd(m.kv_rank, std=0.1, mean=1.0)
            sd[p + "mix.uk"] = rnd(m.heads * m.dim, m.kv_rank, std=m.kv_rank ** -0.5)
            sd[p + "mix.uv"] = rnd(m.heads * m.vdim, m.kv_rank, std=m.kv_rank ** -0.5)
            sd[p + "mix.g"] = rnd(m.heads * m.vdim, W, std=s)
            sd[p + "mix.o"] = rnd(W, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
        else:
            a, r = m.left, m.right
            lp, rp = p + "mix.left.", p + "mix.right."
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            sd[lp + "q"], sd[lp + "k"], sd[lp + "v"] = rnd(nq, W, std=s), rnd(nk, W, std=s), rnd(nv, W, std=s)
            sd[lp + "q.norm"], sd[lp + "k.norm"] = rnd(nq, std=0.1, mean=1.0), rnd(nk, std=0.1, mean=1.0)
            if a.conv >= 1:
                for n, c in (("q", nq), ("k", nk), ("v", nv)):
                    sd[lp + n + ".conv"] = rnd(c, a.conv, std=0.5)
            sd[lp + "pb"] = rnd(a.heads, std=0.5, mean=-2.0)
            sd[lp + "o"] = rnd(W, a.heads * a.vdim, std=(a.heads * a.vdim) ** -0.5)
            sd[rp + "in"] = rnd(2 * r.inner, W, std=s)
            sd[rp + "conv"], sd[rp + "conv.b"] = rnd(r.inner, r.conv, std=0.5), rnd(r.inner, std=0.1)
            sd[rp + "x"] = rnd(r.dt_rank + 2 * r.state, r.inner, std=r.inner ** -0.5)
            sd[rp + "dt"], sd[rp + "dt.b"] = rnd(r.inner, r.dt_rank, std=r.dt_rank ** -0.5), rnd(r.inner, std=0.5, mean=-2.0)
            sd[rp + "A_log"] = torch.log(torch.rand(r.inner, r.state, generator=g, device=device) * 4.0 + 0.5).to(torch.bfloat16)
            sd[rp + "D"] = rnd(r.inner, std=0.5)
            sd[rp + "o"] = rnd(W, r.inner, std=r.inner ** -0.5)
        f = L.mlp
        if f is not None:
            sd[p + "norm2"] = rnd(W, std=0.1)
            sd[p + "mlp.router"] = rnd(f.experts, W, std=s)
            for e in range(f.experts):
                sd[p + f"mlp.e{e}.gate"], sd[p + f"mlp.e{e}.up"] = rnd(f.ff, W, std=s), rnd(f.ff, W, std=s)
                sd[p + f"mlp.e{e}.down"] = rnd(W, f.ff, std=f.ff ** -0.5)
    return sd


class NadevikModel(BobavikModel):
    design = "Nadevik"
    synthetic_name = "nadevik-synthetic"
    has_recurrent_state = True
    build_profile = "text_conv"

    @staticmethod
    def read_config(config: Dict[str, Any]) -> HybridConfig:
        return nadevik_config(config)

    @staticmethod
    def synthetic_weights(cfg: HybridConfig, seed: int, device) -> Dict[str, torch.Tensor]:
        return synthetic_state_dict(cfg, seed, device)
