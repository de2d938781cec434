"""A slow float64 restatement of the Fovunex design, one function per mechanism, written from its equations.  It takes a
configuration dictionary and a name -> tensor mapping and shares no code with the package: whole sequences, keys and
values formed explicitly per head, every recurrence token by token, every looped layer run written out.

Notation: h is a sublayer's input [T, W]; linear weights are [out, in] and act as W h; positions count from 0.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def _w(sd: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return sd[name].to(F64)


# ---- norms and activations -------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is ONE number for all coordinates."""
    return unit_rms(x, eps) * g.reshape(())


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


# ---- rotary positions ------------------------------------------------------------------------------------------------
def rotary_frequencies(rot: Dict[str, Any]) -> Tuple[List[float], float]:
    """(f_i for i < dims / 2, multiplier of cos and sin).  Plain: f_i = base^(-2i / dims), multiplier 1.  With
    ``scaling`` {factor, original, fast, slow}: the index at which a pair turns t times within ``original`` positions is
    d(t) = dims ln(original / (2 pi t)) / (2 ln base); pairs below lo = max(floor d(fast), 0) keep their frequency, pairs
    above hi = min(ceil d(slow), dims - 1) are slowed by ``factor``, linear in between; multiplier 0.1 ln factor + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def d(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(d(float(sc["fast"]))), 0)
    hi = min(math.ceil(d(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[Dict[str, Any]], layout: str) -> torch.Tensor:
    """x [T, ..., D]: the first rot.dims coordinates of the last axis are rotated by position * f_i, the rest pass.
    layout "interleaved": coordinate 2i goes with 2i + 1; "half": coordinate i goes with i + dims / 2."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, mult = rotary_frequencies(rot)
    out = x.clone()
    for t in range(x.shape[0]):
        p = float(positions[t])
        for i in range(dims // 2):
            a, b = (2 * i, 2 * i + 1) if layout == "interleaved" else (i, i + dims // 2)
            c, s = math.cos(p * f[i]) * mult, math.sin(p * f[i]) * mult
            u, v = x[t, ..., a], x[t, ..., b]
            out[t, ..., a] = u * c - v * s
            out[t, ..., b] = v * c + u * s
    return out


# ---- mixers ----------------------------------------------------------------------------------------------------------
def visible(i: int, j: int, chunk: int) -> bool:
    """May position i look at position j?  Causal; with chunk > 0 only inside i's own block of `chunk` positions."""
    return j <= i and (chunk <= 0 or i // chunk == j // chunk)


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, chunk: int = 0) -> torch.Tensor:
    """q [T, dq], k [T, dq], v [T, dv] of ONE head -> [T, dv]."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for i in range(T):
        js = [j for j in range(T) if visible(i, j, chunk)]
        s = (k[js] @ q[i]) * scale
        w = torch.softmax(s, 0)
        out[i] = (w[:, None] * v[js]).sum(0)
    return out


def latent_attention(h: torch.Tensor, sd, p: str, m: Dict[str, Any], eps: float) -> torch.Tensor:
    """Keys and values are per-head expansions of one normed latent per token; every head's query and key have an
    unrotated part and a rotated part, and the rotated key part is one vector shared by all heads."""
    T = h.shape[0]
    H, D, Rd, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ _w(sd, p + "q").T).view(T, H, D + Rd)
    dkv = h @ _w(sd, p + "dkv").T
    c = unit_rms(dkv[:, :R], eps) * _w(sd, p + "dkv.norm")
    k_rot = rotate(dkv[:, R:], pos, m.get("rot"), "interleaved")                    # [T, Rd], all heads
    q_rot = rotate(q[:, :, D:], pos, m.get("rot"), "interleaved")
    k_un = (c @ _w(sd, p + "uk").T).view(T, H, D)
    v = (c @ _w(sd, p + "uv").T).view(T, H, V)
    heads = []
    for a in range(H):
        qa = torch.cat([q[:, a, :D], q_rot[:, a]], 1)
        ka = torch.cat([k_un[:, a], k_rot], 1)
        heads.append(softmax_attention(qa, ka, v[:, a], m["scale"]))
    return torch.cat(heads, 1) @ _w(sd, p + "o").T


def differential_attention(h: torch.Tensor, sd, p: str, m: Dict[str, Any], eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values, the second subtracted times lambda; unit RMS per head; gate."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    diff, chunk = float(m["diff"]), int((m.get("mask") or {}).get("size", 0) or 0)
    pos = torch.arange(T)
    q = (h @ _w(sd, p + "q").T).view(T, H, 2, D)
    k = (h @ _w(sd, p + "k").T).view(T, G, 2, D)
    v = (h @ _w(sd, p + "v").T).view(T, G, V)
    q = rotate(unit_rms(q, eps) * _w(sd, p + "q.norm"), pos, m.get("rot"), "half")
    k = rotate(unit_rms(k, eps) * _w(sd, p + "k.norm"), pos, m.get("rot"), "half")
    lam = (torch.exp((_w(sd, p + "lq1") * _w(sd, p + "lk1")).sum())
           - torch.exp((_w(sd, p + "lq2") * _w(sd, p + "lk2")).sum()) + diff)
    heads = []
    for a in range(H):
        g = a // (H // G)
        a1 = softmax_attention(q[:, a, 0], k[:, g, 0], v[:, g], m["scale"], chunk)
        a2 = softmax_attention(q[:, a, 1], k[:, g, 1], v[:, g], m["scale"], chunk)
        heads.append(unit_rms(a1 - lam * a2, eps) * (1.0 - diff))
    o = torch.cat(heads, 1) * sigmoid(h @ _w(sd, p + "g").T)
    return o @ _w(sd, p + "o").T


def mingru(h: torch.Tensor, sd, p: str, state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """S_t = (1 - z_t) S_(t-1) + z_t c_t with z = sigmoid(W_z h + b_z), c = u + 1/2 where u >= 0 and sigmoid(u) where
    u < 0, u = W_x h + b_x; output W_o (S_t * silu(W_g h)).  Returns (output, last state)."""
    z = sigmoid(h @ _w(sd, p + "z").T + _w(sd, p + "z.b"))
    u = h @ _w(sd, p + "x").T + _w(sd, p + "x.b")
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    gate = h @ _w(sd, p + "g").T
    gate = gate * sigmoid(gate)
    S = torch.zeros(z.shape[1], dtype=F64) if state is None else state.clone()
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * gate[t])
    return torch.stack(rows) @ _w(sd, p + "o").T, S


# ---- feed-forward ----------------------------------------------------------------------------------------------------
def clamped_glu(h: torch.Tensor, sd, p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ _w(sd, p + "gate").T, max=limit)
    u = torch.clamp(h @ _w(sd, p + "up").T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ _w(sd, p + "down").T


# ---- the model -------------------------------------------------------------------------------------------------------
def layer_runs(cfg: Dict[str, Any]) -> List[Tuple[int, bool]]:
    """(layer index, does a repeated pass start here) for every layer run in order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for r in range(times if b > a else 0):
        runs += [(i, r > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(max(a, b), n)]


def mixer(kind: str, h: torch.Tensor, sd, p: str, m: Dict[str, Any], eps: float) -> torch.Tensor:
    if kind == "latent_attention":
        return latent_attention(h, sd, p, m, eps)
    if kind == "attention":
        return differential_attention(h, sd, p, m, eps)
    if kind == "mingru":
        return mingru(h, sd, p)[0]
    raise ValueError(kind)


def forward(cfg: Dict[str, Any], sd: Dict[str, torch.Tensor], tokens) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """tokens [T] -> (logits [T, vocab], the residual stream after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    e0 = _w(sd, "embed")[tokens] * float(cfg["embedding"]["scale"])
    x = e0.clone()
    taps = []
    for i, restart in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if restart:
            x = x + e0
        h = scalar_norm(x, _w(sd, p + "norm1"), eps)
        y = mixer(L["type"], h, sd, p + "mix.", L["mixer"], eps)
        x = x + sigmoid(h @ _w(sd, p + "rg1").T + _w(sd, p + "rg1.b")) * y
        if L.get("mlp"):
            h = scalar_norm(x, _w(sd, p + "norm2"), eps)
            y = clamped_glu(h, sd, p + "mlp.", float(L["mlp"]["limit"]))
            x = x + sigmoid(h @ _w(sd, p + "rg2").T + _w(sd, p + "rg2.b")) * y
        taps.append(x.clone())
    logits = scalar_norm(x, _w(sd, "final.norm"), eps) @ _w(sd, "head").T
    return logits, taps


def greedy(cfg, sd, prompt, n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, sd, toks)[0][-1].argmax()))
    return toks[len(prompt):]


# ---- small configurations and random weights for the tests ----------------------------------------------------------------
def make_config(width=40, vocab=53, layers=("latent", "gru", "attention", "latent"), loop=(1, 3, 2), eps=1e-5, embed_scale=2.0,
                heads=3, dim=8, rot_dim=6, vdim=10, kv_rank=12, lat_scale=0.27, yarn=(4.0, 64, 8.0, 1.0), lat_base=500.0,
                a_heads=4, a_kv_heads=2, a_dim=12, a_vdim=6, a_scale=0.29, diff=0.4, chunk=9, a_rot=(8, 3000.0),
                gru_width=28, ff=24, limit=1.2) -> Dict[str, Any]:
    """layers: "latent" / "attention" / "gru" (each with a feed-forward), the same with "-" appended (no feed-forward), or a
    dictionary {"kind": ..., "ff": n or None, **overrides of the mixer's sizes}.  yarn = (factor, original, fast, slow) or
    None; a_rot = (dims, base) or None; loop = (start, stop, times) or None."""
    out = []
    for spec in layers:
        spec = {"kind": spec} if isinstance(spec, str) else dict(spec)
        kind = spec.pop("kind")
        has_ff = not kind.endswith("-")
        kind = kind.rstrip("-")
        f = spec.pop("ff", ff if has_ff else None)
        lim = spec.pop("limit", limit)
        if kind == "latent":
            m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": lat_scale}
            m.update(spec)
            if m["rot_dim"] and "rot" not in m:
                m["rot"] = {"base": lat_base, "dims": m["rot_dim"]}
                if yarn:
                    m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
            t = "latent_attention"
        elif kind == "attention":
            m = {"heads": a_heads, "kv_heads": a_kv_heads, "dim": a_dim, "vdim": a_vdim, "scale": a_scale, "diff": diff}
            if chunk:
                m["mask"] = {"size": chunk}
            if a_rot:
                m["rot"] = {"dims": a_rot[0], "base": a_rot[1]}
            m.update(spec)
            t = "attention"
        else:
            m = {"width": gru_width}
            m.update(spec)
            t = "mingru"
        out.append({"type": t, "mixer": m, "mlp": {"kind": "dense", "ff": f, "limit": lim} if f else None})
    cfg = {"architecture": "Fovunex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "layers": out}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg: Dict[str, Any], seed: int = 0, head_gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors under the checkpoint's names."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(tuple(shape), generator=g) * std + mean).to(torch.bfloat16)

    sd = {"embed": rnd(cfg["vocab"], W), "head": rnd(cfg["vocab"], W, std=head_gain * W ** -0.5), "final.norm": rnd(std=0.1, mean=1.2)}
    s = W ** -0.5
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        sd[p + "norm1"], sd[p + "rg1"], sd[p + "rg1.b"] = rnd(std=0.2, mean=1.0), rnd(W, W, std=2 * s), rnd(W, std=0.7)
        if L["type"] == "latent_attention":
            H, D, Rd, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            sd[p + "mix.q"], sd[p + "mix.dkv"] = rnd(H * (D + Rd), W, std=3 * s), rnd(R + Rd, W, std=3 * s)
            sd[p + "mix.dkv.norm"] = rnd(R, std=0.2, mean=1.0)
            sd[p + "mix.uk"], sd[p + "mix.uv"] = rnd(H * D, R, std=2 * R ** -0.5), rnd(H * V, R, std=R ** -0.5)
            sd[p + "mix.o"] = rnd(W, H * V, std=2 * (H * V) ** -0.5)
        elif L["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            sd[p + "mix.q"], sd[p + "mix.k"] = rnd(H * 2 * D, W, std=s), rnd(G * 2 * D, W, std=s)
            sd[p + "mix.v"], sd[p + "mix.g"] = rnd(G * V, W, std=s), rnd(H * V, W, std=2 * s)
            sd[p + "mix.q.norm"], sd[p + "mix.k.norm"] = rnd(D, std=0.4, mean=1.5), rnd(D, std=0.4, mean=1.5)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                sd[p + "mix." + n] = rnd(D, std=0.25)
            sd[p + "mix.o"] = rnd(W, H * V, std=2 * (H * V) ** -0.5)
        else:
            Wm = m["width"]
            for n in ("z", "x", "g"):
                sd[p + "mix." + n] = rnd(Wm, W, std=2 * s)
            sd[p + "mix.z.b"], sd[p + "mix.x.b"] = rnd(Wm, std=0.7), rnd(Wm, std=0.7)
            sd[p + "mix.o"] = rnd(W, Wm, std=2 * Wm ** -0.5)
        f = L["mlp"]
        if f:
            sd[p + "norm2"], sd[p + "rg2"], sd[p + "rg2.b"] = rnd(std=0.2, mean=1.0), rnd(W, W, std=2 * s), rnd(W, std=0.7)
            sd[p + "mlp.gate"], sd[p + "mlp.up"] = rnd(f["ff"], W, std=2 * s), rnd(f["ff"], W, std=2 * s)
            sd[p + "mlp.down"] = rnd(W, f["ff"], std=2 * f["ff"] ** -0.5)
    return sd
