"""A slow float64 restatement of the Nadevik design, one function per mechanism, written from its equations.  It takes a
configuration dictionary and a name -> tensor mapping and shares no code with the package: whole sequences, keys and
values formed explicitly per head, every recurrence token by token, pooled keys formed by averaging on the spot.

Notation: h is a sublayer's input [T, W]; linear weights are [out, in] and act as W h; positions count from 0.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def _w(sd: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return sd[name].to(F64)


# ---- element-wise pieces ---------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j) with zeros before the start (the last column weighs
    the current token)."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    if bias is not None:
        y = y + bias
    return y


# ---- embedding -------------------------------------------------------------------------------------------------------
def bigram_rows(tokens: List[int], b: Dict[str, Any]) -> List[int]:
    """Row of the pair table for every token: a hash of (previous, current); the first token takes the extra last row."""
    n = int(b["buckets"])
    out = []
    for t, tok in enumerate(tokens):
        out.append(n if t == 0 else (tokens[t - 1] * int(b["mul_prev"]) + tok * int(b["mul_cur"])) % n)
    return out


def embed(cfg: Dict[str, Any], sd, tokens: List[int]) -> torch.Tensor:
    e = cfg.get("embedding") or {}
    x = _w(sd, "embed")[tokens] * float(e.get("scale", 1.0))
    if e.get("bigram"):
        x = x + _w(sd, "bigram")[bigram_rows(tokens, e["bigram"])]
    return x


# ---- rotary ----------------------------------------------------------------------------------------------------------
def rotate_pairs(x: torch.Tensor, positions: List[int], rot: Dict[str, Any]) -> torch.Tensor:
    """x [T, ..., D]: coordinates (2i, 2i + 1), i < dims / 2, turn by position * base^(-2i / dims); the rest pass."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = x.clone()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, ..., 2 * i], x[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = u * c - v * s
            out[t, ..., 2 * i + 1] = v * c + u * s
    return out


# ---- visibility ------------------------------------------------------------------------------------------------------
def window_keys(i: int, size: int) -> List[int]:
    """Positions j that position i sees directly: 0 <= i - j < size (size 0: all earlier ones)."""
    lo = 0 if size <= 0 else max(0, i - size + 1)
    return list(range(lo, i + 1))


def pooled_blocks(i: int, size: int, pool: int) -> List[int]:
    """Blocks b (positions b pool .. b pool + pool - 1) that are entirely older than position i's window."""
    if pool <= 0 or size <= 0:
        return []
    out, b = [], 0
    while b * pool + pool - 1 <= i - size:
        out.append(b)
        b += 1
    return out


# ---- mixers ----------------------------------------------------------------------------------------------------------
def sigmoid_attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: torch.Tensor, scale: float, cap: float,
                   size: int, pool: int) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V] of ONE sequence from position 0 -> [T, H, V]: position i weighs the tokens of its
    window and the means of the blocks entirely older than it by sigmoid(capped score + bias[head]); nothing is normalised."""
    T, H, _ = q.shape
    G, V = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        js, bs = window_keys(i, size), pooled_blocks(i, size, pool)
        for hh in range(H):
            g = hh // (H // G)
            keys = [k[b * pool:(b + 1) * pool, g].mean(0) for b in bs] + [k[j, g] for j in js]
            vals = [v[b * pool:(b + 1) * pool, g].mean(0) for b in bs] + [v[j, g] for j in js]
            s = torch.stack(keys) @ q[i, hh] * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            out[i, hh] = sigmoid(s + bias[hh]) @ torch.stack(vals)
    return out


def pooled_sigmoid_attention(m: Dict[str, Any], sd, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Grouped-head attention without rotation and without softmax: short causal convolutions on q, k, v; RMS norm of q and
    of k over their whole projection; soft-capped scores; keys = the window's tokens plus the means of the blocks wholly
    before it; weight sigmoid(score + bias of the head), not normalised."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"]))
    q, k, v = h @ _w(sd, p + "q").T, h @ _w(sd, p + "k").T, h @ _w(sd, p + "v").T
    if int(m.get("conv", 0) or 0) >= 1:
        q, k, v = (causal_conv(t, _w(sd, p + n + ".conv")) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q = unit_rms(q, eps) * _w(sd, p + "q.norm")
    k = unit_rms(k, eps) * _w(sd, p + "k.norm")
    mask = m.get("mask") or {}
    out = sigmoid_attend(q.view(T, H, D), k.view(T, G, D), v.view(T, G, V), _w(sd, p + "pb"), float(m["scale"]),
                         float(m.get("softcap", 0.0) or 0.0), int(mask.get("size", 0) or 0), int(mask.get("pool", 0) or 0))
    return out.reshape(T, H * V) @ _w(sd, p + "o").T


def scan(x: torch.Tensor, dt: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor, A: torch.Tensor, Dv: torch.Tensor,
         S: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """x, dt [T, inner]; Bm, Cm [T, N]; A [inner, N]; S the state before the first row (None: zero) -> (y [T, inner], S after)."""
    T, inner = x.shape
    S = torch.zeros(inner, A.shape[1], dtype=F64) if S is None else S.clone()
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t, :, None] * A) * S + (dt[t] * x[t])[:, None] * Bm[t][None, :]
        y[t] = S @ Cm[t] + Dv * x[t]
    return y, S


def selective_scan(m: Dict[str, Any], sd, p: str, h: torch.Tensor) -> torch.Tensor:
    """S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;  out = W_o (y silu(z))."""
    T = h.shape[0]
    inner, N, R = int(m["inner"]), int(m["state"]), int(m["dt_rank"])
    xz = h @ _w(sd, p + "in").T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, _w(sd, p + "conv"), _w(sd, p + "conv.b")))
    low = x @ _w(sd, p + "x").T
    dt = softplus(low[:, :R] @ _w(sd, p + "dt").T + _w(sd, p + "dt.b"))
    y, _ = scan(x, dt, low[:, R:R + N], low[:, R + N:R + 2 * N], -torch.exp(_w(sd, p + "A_log")), _w(sd, p + "D"))
    return (y * silu(z)) @ _w(sd, p + "o").T


def parallel_mixer(m: Dict[str, Any], sd, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    return (float(m.get("left_scale", 1.0)) * pooled_sigmoid_attention(m["left"], sd, p + "left.", h, eps) +
            float(m.get("right_scale", 1.0)) * selective_scan(m["right"], sd, p + "right.", h))


def latent_kv(m: Dict[str, Any], sd, p: str, h: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(normed latent [T, kv_rank], rotated shared key part [T, rot_dim]) of a layer that projects its own."""
    R, Rd = int(m["kv_rank"]), int(m.get("rot_dim", 0) or 0)
    d = h @ _w(sd, p + "dkv").T
    c = unit_rms(d[:, :R], eps) * _w(sd, p + "dkv.norm")
    kr = d[:, R:R + Rd]
    if Rd and m.get("rot"):
        kr = rotate_pairs(kr, list(range(h.shape[0])), m["rot"])
    return c, kr


def latent_attention(m: Dict[str, Any], sd, p: str, h: torch.Tensor, eps: float,
                     kv: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """Softmax attention in a window whose per-head keys [W_uk c | shared rotated part] and values W_uv c are formed here
    explicitly from the latents ``kv`` (this layer's or another's); output gated element by element by sigmoid(W_g h)."""
    T = h.shape[0]
    H, D, Rd, V = int(m["heads"]), int(m["dim"]), int(m.get("rot_dim", 0) or 0), int(m.get("vdim", m["dim"]))
    c, kr = kv
    q = (h @ _w(sd, p + "q").T).view(T, H, D + Rd)
    qu, qr = q[:, :, :D], q[:, :, D:]
    if Rd and m.get("rot"):
        qr = rotate_pairs(qr, list(range(T)), m["rot"])
    ku = (c @ _w(sd, p + "uk").T).view(T, H, D)
    vv = (c @ _w(sd, p + "uv").T).view(T, H, V)
    size = int((m.get("mask") or {}).get("size", 0) or 0)
    out = torch.zeros(T, H, V, dtype=F64)
    for i in range(T):
        js = window_keys(i, size)
        for hh in range(H):
            s = (ku[js, hh] @ qu[i, hh] + (kr[js] @ qr[i, hh] if Rd else 0.0)) * float(m["scale"])
            out[i, hh] = torch.softmax(s, 0) @ vv[js, hh]
    o = out.reshape(T, H * V)
    if (p + "g") in sd:
        o = o * sigmoid(h @ _w(sd, p + "g").T)
    return o @ _w(sd, p + "o").T


# ---- feed-forward ----------------------------------------------------------------------------------------------------
def route(scores: torch.Tensor, top: int, groups: int, keep: int) -> List[int]:
    """The ``top`` largest scores among the experts of the ``keep`` groups (of neighbours) whose largest score is largest."""
    E = scores.numel()
    ok = [True] * E
    if groups > 1 and 0 < keep < groups:
        per = E // groups
        best = sorted(range(groups), key=lambda g: (-float(scores[g * per:(g + 1) * per].max()), g))[:keep]
        ok = [(e // per) in best for e in range(E)]
    order = sorted([e for e in range(E) if ok[e]], key=lambda e: (-float(scores[e]), e))
    return order[:top]


def clamped_expert(sd, p: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ _w(sd, p + "gate").T, max=limit)
    u = torch.clamp(h @ _w(sd, p + "up").T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ _w(sd, p + "down").T


def mixture(f: Dict[str, Any], sd, p: str, h: torch.Tensor) -> torch.Tensor:
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    gr = r.get("groups") or {}
    s = torch.softmax(h @ _w(sd, p + "router").T, -1)
    outs = [clamped_expert(sd, p + f"e{e}.", h, float(f["expert"]["limit"])) for e in range(E)]
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in route(s[t], top, int(gr.get("count", 0) or 0), int(gr.get("keep", 0) or 0)):
            y[t] += s[t, e] * outs[e][t]
    return y


# ---- the model -------------------------------------------------------------------------------------------------------
def forward(cfg: Dict[str, Any], sd: Dict[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None) -> torch.Tensor:
    """-> logits float64 [T, vocab]; ``taps`` (a list) receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(cfg, sd, tokens)
    canon = int((cfg.get("canon") or {}).get("taps", 0) or 0)
    latents: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = x
        if canon:
            h = h + causal_conv(h, _w(sd, p + "canon1"))
        if L["type"] == "parallel":
            y = parallel_mixer(m, sd, p + "mix.", h, eps)
        elif L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_kv(m, sd, p + "mix.", h, eps)
                src = i
            y = latent_attention(m, sd, p + "mix.", h, eps, latents[int(src)])
        else:
            raise ValueError(L["type"])
        x = x + one_plus_norm(y, _w(sd, p + "norm1"), eps)
        if L.get("mlp"):
            x = x + one_plus_norm(mixture(L["mlp"], sd, p + "mlp.", x), _w(sd, p + "norm2"), eps)
        if taps is not None:
            taps.append(x.clone())
    return one_plus_norm(x, _w(sd, "final.norm"), eps) @ _w(sd, "embed").T


# ---- small configurations and random weights for the tests -----------------------------------------------------------
def make_config(layers=("latent", "pair", "pair-", "shared:0", "pair"), width=48, vocab=97, eps=1e-5, embed_scale=3.0,
                bigram=(53, 5, 3), canon=3, l_heads=3, l_dim=8, l_rot=6, l_rot_dims=None, l_vdim=10, l_rank=12, l_window=11,
                l_base=300.0, a_heads=4, a_kv_heads=2, a_dim=12, a_vdim=6, a_window=9, a_pool=4, a_cap=5.0, a_conv=3,
                s_inner=40, s_state=5, s_rank=6, s_conv=4, left_scale=0.7, right_scale=1.3, experts=6, top=2, ff=24, limit=1.2,
                groups=(3, 2)) -> Dict[str, Any]:
    """layers: "latent" (own cached rows), "shared:<j>" (reads layer j's), "pair"; a trailing "-" leaves the feed-forward out."""
    out = []
    for spec in layers:
        has_ff = not spec.endswith("-")
        kind = spec.rstrip("-")
        if kind == "pair":
            left = {"heads": a_heads, "kv_heads": a_kv_heads, "dim": a_dim, "vdim": a_vdim, "scale": 0.31, "softcap": a_cap,
                    "conv": a_conv, "mask": {"size": a_window, "pool": a_pool}}
            right = {"inner": s_inner, "state": s_state, "dt_rank": s_rank, "conv": s_conv}
            layer = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}
        else:
            m = {"heads": l_heads, "dim": l_dim, "rot_dim": l_rot, "vdim": l_vdim, "kv_rank": l_rank, "scale": 0.27,
                 "mask": {"size": l_window}}
            if l_rot:
                m["rot"] = {"base": l_base, "dims": l_rot if l_rot_dims is None else l_rot_dims}
            if kind.startswith("shared:"):
                m["kv_from"] = int(kind.split(":")[1])
            layer = {"type": "latent_attention", "mixer": m}
        layer["mlp"] = None
        if has_ff:
            r = {"experts": experts, "top": top}
            if groups:
                r["groups"] = {"count": groups[0], "keep": groups[1]}
            layer["mlp"] = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}
        out.append(layer)
    cfg = {"architecture": "Nadevik", "width": width, "vocab": vocab, "norm": {"eps": eps},
           "embedding": {"scale": embed_scale}, "layers": out}
    if canon:
        cfg["canon"] = {"taps": canon}
    if bigram:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return cfg


def make_weights(cfg: Dict[str, Any], seed: int = 0, calm: bool = False) -> Dict[str, torch.Tensor]:
    """Random bf16 weights with the checkpoint's names, scaled so that every mechanism matters in the logits.  calm: smaller
    inputs and routers that are less sharp, for comparisons in bfloat16 (where a sharp router turns a rounding into another
    expert)."""
    g = torch.Generator().manual_seed(seed)
    W = int(cfg["width"])
    hot = 0.5 if calm else 1.0

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(tuple(shape), generator=g) * std + mean).to(torch.bfloat16)

    sd = {"embed": rnd(int(cfg["vocab"]), W, std=0.5 * hot), "final.norm": rnd(W, std=0.2)}
    b = (cfg.get("embedding") or {}).get("bigram")
    if b:
        sd["bigram"] = rnd(int(b["buckets"]) + 1, W, std=hot)
    taps = int((cfg.get("canon") or {}).get("taps", 0) or 0)
    s = W ** -0.5
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        sd[p + "norm1"] = rnd(W, std=0.2)
        if taps:
            sd[p + "canon1"] = rnd(W, taps, std=0.4)
        if L["type"] == "latent_attention":
            H, D, Rd, V, R = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
            sd[p + "mix.q"] = rnd(H * (D + Rd), W, std=2 * s)
            if m.get("kv_from") is None:
                sd[p + "mix.dkv"], sd[p + "mix.dkv.norm"] = rnd(R + Rd, W, std=2 * s), rnd(R, std=0.2, mean=1.0)
            sd[p + "mix.uk"], sd[p + "mix.uv"] = rnd(H * D, R, std=R ** -0.5), rnd(H * V, R, std=R ** -0.5)
            sd[p + "mix.g"] = rnd(H * V, W, std=2 * s)
            sd[p + "mix.o"] = rnd(W, H * V, std=(H * V) ** -0.5)
        else:
            a, r = m["left"], m["right"]
            H, G, D, V = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a["vdim"])
            lp, rp = p + "mix.left.", p + "mix.right."
            sd[lp + "q"], sd[lp + "k"], sd[lp + "v"] = rnd(H * D, W, std=s), rnd(G * D, W, std=s), rnd(G * V, W, std=s)
            sd[lp + "q.norm"], sd[lp + "k.norm"] = rnd(H * D, std=0.3, mean=1.5), rnd(G * D, std=0.3, mean=1.5)
            if int(a.get("conv", 0) or 0) >= 1:
                for n, c in (("q", H * D), ("k", G * D), ("v", G * V)):
                    sd[lp + n + ".conv"] = rnd(c, int(a["conv"]), std=0.6)
            sd[lp + "pb"] = rnd(H, std=0.7, mean=-1.0)
            sd[lp + "o"] = rnd(W, H * V, std=(H * V) ** -0.5)
            inner, N, R = int(r["inner"]), int(r["state"]), int(r["dt_rank"])
            sd[rp + "in"] = rnd(2 * inner, W, std=s)
            sd[rp + "conv"], sd[rp + "conv.b"] = rnd(inner, int(r["conv"]), std=0.6), rnd(inner, std=0.2)
            sd[rp + "x"] = rnd(R + 2 * N, inner, std=2 * inner ** -0.5)
            sd[rp + "dt"], sd[rp + "dt.b"] = rnd(inner, R, std=R ** -0.5), rnd(inner, std=0.7, mean=-1.5)
            sd[rp + "A_log"] = torch.log(torch.rand(inner, N, generator=g) * 3.0 + 0.05).to(torch.bfloat16)
            sd[rp + "D"] = rnd(inner, std=0.5)
            sd[rp + "o"] = rnd(W, inner, std=inner ** -0.5)
        f = L.get("mlp")
        if f:
            E, ff = int(f["router"]["experts"]), int(f["expert"]["ff"])
            sd[p + "norm2"] = rnd(W, std=0.2)
            sd[p + "mlp.router"] = rnd(E, W, std=(0.7 if calm else 3.0) * s)
            for e in range(E):
                sd[p + f"mlp.e{e}.gate"], sd[p + f"mlp.e{e}.up"] = rnd(ff, W, std=2 * s), rnd(ff, W, std=2 * s)
                sd[p + f"mlp.e{e}.down"] = rnd(W, ff, std=ff ** -0.5)
    return sd
