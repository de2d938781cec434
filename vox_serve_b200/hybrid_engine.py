"""Decoder stacks that mix softmax attention (sliding window, grouped heads, partial interleaved rotary, cross-layer
value mixing, sigmoid output gate), linear attention with a per-head decay and a recurrent fp32 state, latent attention
(queries and keys/values through low-rank latents, only the key/value latent cached, optionally shared between layers)
and dense or mixture-of-experts feed-forwards, around an fp32 residual stream.  Two block forms: ``sequential``
(LayerNorm before and after every sublayer, mixer then feed-forward) and ``parallel`` (mixer and feed-forward read two
RMS norms of the same stream and their sum is added, scaled; optionally followed by a per-token side input).  ``LlamaEngine`` (engine.py) is the engine of the Llama-shaped speech LMs; this one is configured layer
by layer from a ``HybridConfig`` and runs the same way: a fixed sequence of C-ABI launches over preallocated buffers, no
host synchronisation, CUDA-graph capturable.

One step serves a batch of requests that each bring one or more new tokens (a decoded token, a whole prompt or a portion
of one).  Per layer:
    [fused q|k|v|gate projection]  ->  rotary + value mixing + page append  ->  window attention (* gate)  ->  o projection
    [fused q|k|v|gate projection]  ->  decay attention over the slot's state  ->  gated RMS norm         ->  o projection
    [fused q-latent|kv-latent|gate projection] -> RMS norms + page append of the kv latent -> q up-projection -> queries
        carried into latent space per head -> attention over the cached latents (one shared key = value head) -> per-head
        value expansion * gate -> o projection
    router -> group by expert -> grouped gate/up (silu * up) -> grouped down -> shared expert -> weighted sum
each followed (sequential form) by ``x += LayerNorm(y)`` fused with the LayerNorm that feeds the next sublayer, or
(parallel form) by ``x += m * (mixer + feed-forward)`` fused with the side input and the next block's two RMS norms.
A third block form, ``gated`` (pre-norm, ``x += sigmoid(W_r h + b) * sublayer(h)``, scalar RMS norms, optionally a span of
layers run several times with a cache or state per pass), carries three more mixers -- latent attention with direct queries
and a shared rotated key part, attention with two score maps per head restricted to chunks, minGRU -- and a clamped gated
feed-forward (``_forward_gated``).  A fourth, ``post`` (what a sublayer returns is normed, what it reads is not: the sublayers take the stream
itself -- the mixer through a short causal input convolution with state), carries latent attention in a window with a gate per
output value and rows that layers may share, and a pair of mixers side by side -- attention whose weights are sigmoids over a
window plus pooled blocks, and a selective scan -- with a group-limited softmax router over clamped gated experts, a hashed
token-pair embedding and a tied head (``_forward_post`` at the end of this file).

Precision: ``dtype`` bfloat16 keeps projections' operands, q / k / v, the page cache and the attention output in bf16 with
fp32 accumulation; norms, softmax, router, residual, recurrent state, decays and the lightning path after its projection
are fp32.  ``dtype`` float32 runs everything in fp32 (sequential FMA chains, no reduced-precision matrix mode).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import ops
from ._lib import VoxB200Error

BF16, F32, I32 = torch.bfloat16, torch.float32, torch.int32


# ------------------------------------------------------------------------------------------------------------------
# configuration
# ------------------------------------------------------------------------------------------------------------------
@dataclass
class RotaryConfig:
    dims: int
    base: float
    factor: Optional[float] = None       # frequency scaling when set (``scaling`` says which kind)
    low: float = 1.0
    high: float = 4.0
    original: float = 8192.0
    layout: str = "interleaved"          # "interleaved": dim 2i goes with 2i + 1; "half": dim i goes with i + dims / 2
    scaling: str = "wavelength"          # "wavelength" (Llama-3.1 style, low / high) | "yarn" (fast / slow turns, ramp over the
    #                                      pair index, cos and sin times 0.1 ln(factor) + 1)
    fast: float = 32.0
    slow: float = 1.0

    def key(self) -> Tuple:
        return (self.dims, self.base, self.factor, self.low, self.high, self.original, self.scaling, self.fast, self.slow)

    def multiplier(self) -> float:
        """What cos and sin are multiplied by."""
        return 0.1 * math.log(self.factor) + 1.0 if (self.factor is not None and self.scaling == "yarn") else 1.0

    def frequencies(self) -> torch.Tensor:
        """float64 [dims / 2]: base^(-2i/dims).  "wavelength" scaling: wavelengths above original/low are slowed by
        ``factor``, those below original/high kept, the band in between interpolated linearly in original/wavelength.
        "yarn" scaling: with d(t) = dims ln(original / (2 pi t)) / (2 ln base) the pair index that turns t times within
        ``original`` positions, pairs up to lo = max(floor d(fast), 0) keep their frequency, pairs from
        hi = min(ceil d(slow), dims - 1) on are slowed by ``factor``, linearly mixed in between."""
        if self.factor is not None and self.scaling == "yarn":
            def d(t):
                return self.dims * math.log(self.original / (2.0 * math.pi * t)) / (2.0 * math.log(self.base))
            lo, hi = max(math.floor(d(self.fast)), 0), min(math.ceil(d(self.slow)), self.dims - 1)
            out = []
            for i in range(self.dims // 2):
                f = self.base ** (-2.0 * i / self.dims)
                ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                out.append(f / self.factor * ramp + f * (1.0 - ramp))
            return torch.tensor(out, dtype=torch.float64)
        out = []
        for i in range(self.dims // 2):
            f = self.base ** (-2.0 * i / self.dims)
            if self.factor is not None:
                wl = 2.0 * math.pi / f
                if wl < self.original / self.high:
                    pass
                elif wl > self.original / self.low:
                    f = f / self.factor
                else:
                    s = (self.original / wl - self.low) / (self.high - self.low)
                    f = (1.0 - s) * f / self.factor + s * f
            out.append(f)
        return torch.tensor(out, dtype=torch.float64)


@dataclass
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                       # 0: every earlier position is visible
    rotary: Optional[RotaryConfig] = None
    v_mix: bool = False
    gate: bool = True


@dataclass
class DecayAttentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: List[float] = field(default_factory=list)


@dataclass
class LatentAttentionConfig:
    """Causal softmax attention whose keys and values are per-head expansions of ONE normed latent of kv_rank dims per token
    -- with the shared rotated key part, if there is one, the only thing cached.  Queries go through a normed latent of
    q_rank dims, or come straight from the input (q_rank = 0).  kv_from: the layer whose cached latents this layer reads
    instead of projecting its own.  head_gate: one sigmoid gate per head."""
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    q_rank: int                           # 0: queries are projected from the sublayer's input directly (no query latent)
    scale: float
    kv_from: Optional[int] = None
    # heads with a rotated part: every query head has rot_dim more dims behind its `dim` unrotated ones, and every token has
    # ONE rotated key part of rot_dim dims shared by all heads, cached behind the latent ([kv_rank | rot_dim] per token)
    rot_dim: int = 0
    rotary: Optional[RotaryConfig] = None
    head_gate: bool = True
    window: int = 0                       # > 0: position i sees the keys j with 0 <= i - j < window
    value_gate: bool = False              # the concatenated heads times sigmoid(W_g h), one gate per output value


@dataclass
class PooledSigmoidAttentionConfig:
    """Grouped-head attention without rotation whose weights are sigmoid(score + bias of the head), not normalised over the
    keys.  q, k, v pass a short causal convolution (conv taps; 0 / 1: none) right after their projection; q and k are then
    RMS-normed over their WHOLE projection (all heads at once, one weight per coordinate).  Scores are soft-capped
    (softcap * tanh(score / softcap); 0: no cap).  A position sees the tokens of its window and, with pool = P > 0, one mean
    key / value per block of P positions whose last position is older than the window's oldest."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0
    pool: int = 0
    softcap: float = 0.0
    conv: int = 0
    qk_norm: bool = True


@dataclass
class SelectiveScanConfig:
    """Mamba-form recurrence: [x | z] = W_in h; x through a causal convolution (conv taps, with bias) and silu; [dt | B | C] =
    W_x x with dt of dt_rank dims, dt <- softplus(W_dt dt + b); S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n over an fp32
    state [inner, state] per request; y_c = sum_n S[c, n] C_n + D_c x_c; output W_o (y * silu(z))."""
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass
class MixerPairConfig:
    """Two mixers side by side on the same input; the result is left_scale * left + right_scale * right."""
    left: PooledSigmoidAttentionConfig
    right: SelectiveScanConfig
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass
class PairEmbedConfig:
    """A second embedding of (previous token, token) pairs: row (prev * mul_prev + token * mul_cur) mod buckets of a table of
    buckets + 1 rows, whose last row serves a sequence's first token."""
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass
class DiffAttentionConfig:
    """Softmax attention with two score maps per head over the same values (queries and keys hold [map 1 | map 2] per head):
    o = a1 - lambda * a2, divided by its root mean square over the head's vdim values, times (1 - diff); lambda is one number
    per layer.  Queries and keys are RMS-normed per head and map (qk_norm) before the rotation; chunk > 0 restricts a position
    to the keys of its own block of `chunk` positions; a sigmoid gate per output value."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    chunk: int = 0
    window: int = 0
    rotary: Optional[RotaryConfig] = None
    qk_norm: bool = True
    gate: bool = True


@dataclass
class MinGRUConfig:
    """Element-wise gated recurrence: S_t = (1 - z) S_(t-1) + z c with z = sigmoid(W_z h + b), c = u + 1/2 (u >= 0) or
    sigmoid(u), u = W_x h + b; output W_o (S_t * silu(W_g h)); fp32 state of `width` values per request."""
    width: int


@dataclass
class DenseMLPConfig:
    ff: int
    act: str = "relu2"                    # "relu2" | "gelu" | "gelu_tanh": down(act(up h))


@dataclass
class GluMLPConfig:
    """down(g * sigmoid(slope * g) * (u + 1)) with g = min(gate h, limit), u = clamp(up h, -limit, limit)."""
    ff: int
    limit: float
    slope: float = 1.702


@dataclass
class MoEConfig:
    experts: int
    top: int
    ff: int
    shared_ff: int = 0                    # 0: no shared expert
    act: str = "silu_glu"                 # "silu_glu": down(silu(gate h) * up h); "clamped_glu": down(g sigmoid(slope g) (u + 1))
    #                                       with g = min(gate h, limit), u = clamp(up h, +-limit); else down(act(up h)) as
    #                                       DenseMLPConfig.act
    router: str = "softmax"               # "softmax": top logits, softmax over the chosen.  "sigmoid": sigmoid scores, chosen
    #                                       by score + correction within the kept groups, weights = chosen scores / their sum.
    #                                       "softmax_all": scores = softmax over ALL experts, the largest within the kept
    #                                       groups chosen, weights = the chosen scores as they are
    groups: int = 0                       # group routers: experts form this many groups of neighbours (0 / 1: one pool)
    groups_keep: int = 0                  # ... of which the best this many stay eligible
    shared_gate: bool = False             # the shared expert's output times sigmoid(w_sg . h)
    limit: float = 0.0                    # "clamped_glu"
    slope: float = 1.702


@dataclass
class HybridLayerConfig:
    kind: str                             # "attention" | "lightning" | "latent" | "diff_attention" | "mingru" | "mixer_pair"
    mixer: Any
    mlp: Any = None                       # MoEConfig | DenseMLPConfig | GluMLPConfig | None


@dataclass
class HybridConfig:
    width: int
    vocab: int
    eps: float
    logit_scale: float
    layers: List[HybridLayerConfig]
    block: str = "sequential"             # "sequential": x += LN(mixer(LN x)); x += LN(ff(LN x)).  "parallel": x += m * (mixer(n1 x) + ff(n2 x))
    #                                       "gated": pre-norm, x += sigmoid(W_r h + b) * sublayer(h) with h = norm(x), mixer then ff
    #                                       "post": x += norm(sublayer(x)): only what a sublayer returns is normed; the sublayers
    #                                       read the stream itself (the mixer through the input convolution, if any)
    norm: str = "layernorm"               # "layernorm" (weight and bias) | "rmsnorm" (weight) | "rmsnorm_scalar" (one number) |
    #                                       "rmsnorm_offset" (the stored weight is an offset from one: x / rms * (1 + w))
    residual_mult: float = 1.0            # m of the parallel form
    positions: int = 0                    # rows of the learned position table added to the embedding (0: none)
    side_dim: int = 0                     # per-token side input of every block (parallel form): dims per layer (0: none)
    logit_softcap: float = 0.0            # logits <- cap * tanh(logits / cap) (0: none)
    embed_scale: float = 1.0              # the embedding rows are multiplied by this
    # layers loop_start .. loop_stop - 1 run loop_times times in a row with the same weights; every pass has its own cache and
    # state, and before each pass but the first the embedding output is added to the stream
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    tied_head: bool = False               # the output head is the embedding table itself (unscaled); no "head" tensor
    pair_embed: Optional[PairEmbedConfig] = None   # a hashed (previous token, token) embedding added to the token's
    input_conv: int = 0                   # "post" blocks: the mixer reads h + conv(h), a causal convolution of this many taps
    #                                       over time on every channel of the stream (0: it reads h)

    def runs(self) -> List[Tuple[int, bool]]:
        """(layer index, does a repeated pass start here) for every layer run in order.  Caches and states are kept per run."""
        n, a, b = len(self.layers), self.loop_start, self.loop_stop
        if b <= a:
            return [(i, False) for i in range(n)]
        out = [(i, False) for i in range(a)]
        for r in range(self.loop_times):
            out += [(i, r > 0 and i == a) for i in range(a, b)]
        return out + [(i, False) for i in range(b, n)]

    @classmethod
    def from_json(cls, c: Dict[str, Any]) -> "HybridConfig":
        layers = []
        for L in c["layers"]:
            m = L["mixer"]
            kind = L["type"]
            if kind == "attention":
                rot = None
                if m.get("rot"):
                    r = m["rot"]
                    sc = r.get("scaling") or {}
                    rot = RotaryConfig(int(r["dims"]), float(r["base"]), float(sc["factor"]) if sc else None,
                                       float(sc.get("low", 1.0)), float(sc.get("high", 4.0)),
                                       float(sc.get("original", 8192)))
                mask = m.get("mask") or {}
                mixer = WindowAttentionConfig(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]),
                                              int(m.get("vdim", m["dim"])), float(m.get("scale", m["dim"] ** -0.5)),
                                              int(mask.get("size", 0) or 0), rot, bool(m.get("v_mix", False)))
            elif kind == "lightning":
                mixer = DecayAttentionConfig(int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])),
                                             [float(d) for d in m["decay"]])
                if len(mixer.decay) != mixer.heads:
                    raise VoxB200Error(f"{len(mixer.decay)} decays for {mixer.heads} heads")
            else:
                raise VoxB200Error(f"unknown mixer type '{kind}'")
            mlp = None
            if L.get("mlp"):
                f = L["mlp"]
                if f.get("kind", "moe") != "moe":
                    raise VoxB200Error(f"unknown feed-forward kind '{f.get('kind')}'")
                sh = f.get("shared") or {}
                mlp = MoEConfig(int(f["router"]["experts"]), int(f["router"]["top"]), int(f["expert"]["ff"]),
                                int(sh.get("ff", 0) or 0))
            layers.append(HybridLayerConfig(kind, mixer, mlp))
        return cls(int(c["width"]), int(c["vocab"]), float(c["norm"]["eps"]), float(c.get("logit_scale", 1.0)), layers)


# ------------------------------------------------------------------------------------------------------------------
# weights
# ------------------------------------------------------------------------------------------------------------------
class HybridWeights:
    """Device-resident weights from a name -> tensor mapping with the checkpoint names ``embed``, ``l<i>.norm1[.b]``,
    ``l<i>.norm1b[.b]``, ``l<i>.norm2[.b]``, ``l<i>.norm2b[.b]``, ``l<i>.mix.{q,k,v,g,o,vmix,norm}``,
    ``l<i>.mlp.{router,router.b,e<j>.{gate,up,down},shared.{gate,up,down}}``, ``final.norm[.b]``, ``head``.
    q | k | v | g are concatenated into one projection, gate | up of every expert into one matrix, the experts into
    [E, ...] stacks.  Matrices take the compute dtype; norm weights, router, decays and mixing coefficients stay fp32.
    Parallel blocks with RMS norms have ``l<i>.norm1``, ``l<i>.norm2`` (weights only), optionally ``pos`` (learned
    positions), ``side.embed`` + ``l<i>.side.{gate,proj,norm}`` (per-token side input); latent-attention mixers and
    experts without a gate matrix are described at ``_load_latent`` / ``_load_plain_moe``."""

    def __init__(self, sd: Dict[str, torch.Tensor], cfg: HybridConfig, dtype: torch.dtype, device,
                 tensor_core: bool = True):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        dev = self.device
        # bf16 dense projections (q|k|v|gate, o, shared expert, output head) are re-tiled for the tcgen05 kernel of gemm.cu
        # when their reduction size allows its 16-byte rows; the row-major copy is then dropped
        self.tensor_core = bool(tensor_core) and dtype == BF16 and self.device.type == "cuda"

        def mat(*names):
            ts = [sd[n] for n in names]
            t = ts[0] if len(ts) == 1 else torch.cat([x.reshape(-1, x.shape[-1]) for x in ts], 0)
            return t.to(device=dev, dtype=dtype).contiguous()

        def vec(name):
            return sd[name].to(device=dev, dtype=F32).contiguous()

        def norm(name):
            return vec(name), vec(name + ".b")

        def dense(t):
            if self.tensor_core and t.shape[1] % 8 == 0:
                return ops.pack_weight(t, 128)
            return t

        def gate_up(gate_name, up_name):
            """shared expert: [gate rows | up rows] for vb_linear, or gate / up interleaved per tile for the tcgen05 kernel's
            silu(gate) * up epilogue"""
            if self.tensor_core and sd[gate_name].shape[1] % 8 == 0:
                half = ops.gate_up_tile_half(sd[gate_name].shape[0])
                return ops.pack_weight(ops.interleave_gate_up(mat(gate_name), mat(up_name), half), 2 * half)
            return mat(gate_name, up_name)

        self._mat, self._vec, self._dense = mat, vec, dense      # (for the per-mechanism loaders below; dropped at the end)
        if cfg.norm == "rmsnorm":
            def norm(name):                                        # noqa: F811  (weight only)
                return vec(name), None
        elif cfg.norm == "rmsnorm_scalar":
            def norm(name):                                        # noqa: F811  (one number, kept as a constant vector)
                return vec(name).reshape(1).expand(cfg.width).contiguous(), None
        elif cfg.norm == "rmsnorm_offset":
            def norm(name):                                        # noqa: F811  (the checkpoint holds w, the weight is 1 + w, formed in fp32)
                return (vec(name) + 1.0).contiguous(), None
        self._gate_up = gate_up
        self.embed = mat("embed")
        head_name = "embed" if cfg.tied_head else "head"          # (tied: the table itself, whatever scale the embedding takes)
        self.head = dense(mat(head_name))
        self.final_norm = norm("final.norm")
        # the tcgen05 kernel has no output scale: logit_scale is folded into the final norm's weight and bias there
        self.final_norm_scaled = tuple(t * cfg.logit_scale if t is not None else None for t in self.final_norm)
        if tuple(self.embed.shape) != (cfg.vocab, cfg.width) or tuple(sd[head_name].shape) != (cfg.vocab, cfg.width):
            raise VoxB200Error("embed / head shapes do not match the configuration")
        self.pos = self.side_embed = self.pair_table = None
        if cfg.pair_embed is not None:
            self.pair_table = mat("bigram")
            if tuple(self.pair_table.shape) != (cfg.pair_embed.buckets + 1, cfg.width):
                raise VoxB200Error("pair embedding shape does not match the configuration")
        if cfg.positions:
            self.pos = mat("pos")
            if tuple(self.pos.shape) != (cfg.positions, cfg.width):
                raise VoxB200Error("position table shape does not match the configuration")
        if cfg.side_dim:
            self.side_embed = mat("side.embed")
            if tuple(self.side_embed.shape) != (cfg.vocab, cfg.side_dim * len(cfg.layers)):
                raise VoxB200Error("side embedding shape does not match the configuration")
        self.layers: List[Dict[str, Any]] = []
        for i, L in enumerate(cfg.layers):
            p = f"l{i}."
            m = L.mixer
            if cfg.block == "gated":
                self.layers.append(self._load_gated_layer(sd, p, i, L, norm))
                continue
            if cfg.block == "post":
                self.layers.append(self._load_post_layer(sd, p, i, L, norm))
                continue
            if cfg.block == "parallel":
                w: Dict[str, Any] = {"norm1": vec(p + "norm1")}
                if L.mlp is not None:
                    w["norm2"] = vec(p + "norm2")
                if cfg.side_dim:
                    w["side_gate"], w["side_proj"], w["side_norm"] = mat(p + "side.gate"), mat(p + "side.proj"), vec(p + "side.norm")
                    if tuple(w["side_gate"].shape) != (cfg.side_dim, cfg.width) or tuple(w["side_proj"].shape) != (cfg.width, cfg.side_dim):
                        raise VoxB200Error(f"layer {i}: side input shapes do not match the configuration")
            else:
                w = {"norm1": norm(p + "norm1"), "norm1b": norm(p + "norm1b")}
            if L.kind == "latent":
                self._load_latent(sd, p, i, m, w)
            elif L.kind == "attention":
                w["qkvg"] = mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g")
                w["o"] = mat(p + "mix.o")
                if m.v_mix:
                    w["vmix"] = sd[p + "mix.vmix"].reshape(1).to(device=dev, dtype=F32).contiguous()
                want = m.heads * m.dim + m.kv_heads * (m.dim + m.vdim) + m.heads * m.vdim
            else:
                w["qkvg"] = mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g")
                w["o"] = mat(p + "mix.o")
                w["norm"] = vec(p + "mix.norm")
                w["decay"] = torch.tensor(m.decay, dtype=torch.float64).to(device=dev, dtype=F32)
                want = 2 * m.heads * m.dim + 2 * m.heads * m.vdim
            if L.kind != "latent":
                if tuple(w["qkvg"].shape) != (want, cfg.width):
                    raise VoxB200Error(f"layer {i}: projection shapes {tuple(w['qkvg'].shape)} do not match the configuration")
                w["qkvg"], w["o"] = dense(w["qkvg"]), dense(w["o"])
            if isinstance(L.mlp, DenseMLPConfig):
                w["up"], w["down"] = mat(p + "mlp.up"), mat(p + "mlp.down")
                if tuple(w["up"].shape) != (L.mlp.ff, cfg.width) or tuple(w["down"].shape) != (cfg.width, L.mlp.ff):
                    raise VoxB200Error(f"layer {i}: feed-forward shapes do not match the configuration")
                w["up"], w["down"] = dense(w["up"]), dense(w["down"])
            elif L.mlp is not None and L.mlp.act != "silu_glu":
                self._load_plain_moe(sd, p, i, L.mlp, w)
            elif L.mlp is not None:
                f = L.mlp
                if cfg.block != "parallel":
                    w["norm2"], w["norm2b"] = norm(p + "norm2"), norm(p + "norm2b")
                self._load_gated_moe(sd, p, f, w)
            self.layers.append(w)
        del self._mat, self._vec, self._dense, self._gate_up

    def _load_gated_moe(self, sd, p: str, f: "MoEConfig", w: Dict[str, Any]) -> None:
        """Experts with a gate and an up matrix (``l<i>.mlp.{router[, router.b], e<j>.{gate,up,down}[, shared.{gate,up,down}]}``):
        on tensor-core projections all experts and the shared expert stacked into ONE interleaved gate/up matrix (along N) and
        ONE down matrix (along K), with the per-expert offsets of the grouped form where tiles do not straddle experts;
        otherwise [E, ...] stacks for the grouped linear kernel."""
        mat, vec, dense, gate_up, cfg = self._mat, self._vec, self._dense, self._gate_up, self.cfg
        w["router"] = vec(p + "mlp.router")
        w["router_b"] = vec(p + "mlp.router.b") if (p + "mlp.router.b") in sd else None
        n_all = f.experts * f.ff + f.shared_ff
        if self.tensor_core and cfg.width % 8 == 0 and n_all % 8 == 0 and f.experts <= self.DENSE_MOE_MAX_RATIO * f.top:
            # dense form (vb_moe_scale_dense): all experts and the shared expert as one gate/up and one down matrix
            names = [f"e{e}" for e in range(f.experts)] + (["shared"] if f.shared_ff else [])
            gate = torch.cat([mat(p + f"mlp.{n}.gate") for n in names], 0)
            up = torch.cat([mat(p + f"mlp.{n}.up") for n in names], 0)
            # a gate/up tile height that divides every expert keeps tiles from straddling experts: the stacked
            # buffer is then also the per-expert buffers one after the other, which the grouped form indexes
            fit = [hh for hh in (64, 48, 32, 16) if f.ff % hh == 0 and f.shared_ff % hh == 0]
            half = fit[0] if fit else ops.gate_up_tile_half(n_all)
            w["gu_all"] = ops.pack_weight(ops.interleave_gate_up(gate, up, half), 2 * half)
            del gate, up
            w["down_all"] = ops.pack_weight(torch.cat([mat(p + f"mlp.{n}.down") for n in names], 1).contiguous(), 128)
            if fit and f.ff % 64 == 0:
                gb = ops.weight_tiles_bytes(2 * f.ff, cfg.width, 2 * half)
                w["grouped"] = {"group_bytes": gb, "kb_total": (n_all + 63) // 64, "group_kb": f.ff // 64}
                if f.shared_ff:
                    w["s_gu_view"] = ops.PackedWeight(w["gu_all"].data[f.experts * gb:], 2 * f.shared_ff, cfg.width,
                                                      2 * half)
        else:
            w["gu"] = torch.stack([mat(p + f"mlp.e{e}.gate", p + f"mlp.e{e}.up") for e in range(f.experts)]).contiguous()
            w["down"] = torch.stack([mat(p + f"mlp.e{e}.down") for e in range(f.experts)]).contiguous()
            if f.shared_ff:
                w["s_gu"] = gate_up(p + "mlp.shared.gate", p + "mlp.shared.up")
                w["s_down"] = dense(mat(p + "mlp.shared.down"))

    def _load_post_layer(self, sd, p: str, i: int, L: "HybridLayerConfig", norm) -> Dict[str, Any]:
        """A layer of a stack that norms sublayer OUTPUTS only: ``l<i>.norm1`` / ``norm2``, ``l<i>.canon1`` (the input
        convolution [width, taps]), ``l<i>.mix.*``, ``l<i>.mlp.{router, e<j>.{gate,up,down}}``.
          latent attention with direct queries: in = q | dkv | g (no dkv in a layer that reads another layer's cached rows);
            uk per head transposed, uv per head
          mixer pair: in = left.q | left.k | left.v | right.in -- ONE projection for both mixers; the three short convolutions
            of the left mixer stacked into one [nq + nk + nv, taps]; A = -exp(A_log) formed here in fp32; o = [left.o | right.o]
            side by side along K, so ONE output projection sums both mixers (their scales go on its input)."""
        mat, vec, dense, cfg, W, m = self._mat, self._vec, self._dense, self.cfg, self.cfg.width, L.mixer
        w: Dict[str, Any] = {"norm1": norm(p + "norm1")[0]}
        if cfg.input_conv:
            w["canon"] = vec(p + "canon1")
            if tuple(w["canon"].shape) != (W, cfg.input_conv):
                raise VoxB200Error(f"layer {i}: input convolution shape does not match the configuration")
        if L.kind == "latent":
            own = m.kv_from is None
            if m.q_rank or m.head_gate:
                raise VoxB200Error(f"layer {i}: post-norm blocks take latent attention with direct queries and no per-head gate")
            if not own:
                src = cfg.layers[m.kv_from] if 0 <= m.kv_from < i else None
                if (src is None or src.kind != "latent" or src.mixer.kv_from is not None or src.mixer.kv_rank != m.kv_rank or
                        src.mixer.rot_dim != m.rot_dim or (src.mixer.rotary.key() if src.mixer.rotary else None) !=
                        (m.rotary.key() if m.rotary else None)):
                    raise VoxB200Error(f"layer {i}: kv_from {m.kv_from} must name an earlier latent-attention layer that projects "
                                       "its own latents, of the same rank, rotated part and rotation")
            if m.value_gate and (p + "mix.g") not in sd:       # (a checkpoint without the gate's matrix: no gate)
                m.value_gate = False
            dq = m.dim + m.rot_dim
            parts = [mat(p + "mix.q")] + ([mat(p + "mix.dkv")] if own else []) + ([mat(p + "mix.g")] if m.value_gate else [])
            uk, uv, o = mat(p + "mix.uk"), mat(p + "mix.uv"), mat(p + "mix.o")
            if (tuple(parts[0].shape) != (m.heads * dq, W) or (own and tuple(parts[1].shape) != (m.kv_rank + m.rot_dim, W)) or
                    (m.value_gate and tuple(parts[-1].shape) != (m.heads * m.vdim, W)) or
                    tuple(uk.shape) != (m.heads * m.dim, m.kv_rank) or tuple(uv.shape) != (m.heads * m.vdim, m.kv_rank) or
                    tuple(o.shape) != (W, m.heads * m.vdim)):
                raise VoxB200Error(f"layer {i}: latent attention shapes do not match the configuration")
            w["in"] = dense(torch.cat(parts, 0).contiguous())
            if own:
                w["dkv_norm"] = vec(p + "mix.dkv.norm")
            w["uk_t"] = uk.view(m.heads, m.dim, m.kv_rank).transpose(1, 2).contiguous()
            w["uv"] = uv.view(m.heads, m.vdim, m.kv_rank).contiguous()
            w["o"] = dense(o)
        elif L.kind == "mixer_pair":
            a, r = m.left, m.right
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            lp, rp = p + "mix.left.", p + "mix.right."
            q, k, v, xin = mat(lp + "q"), mat(lp + "k"), mat(lp + "v"), mat(rp + "in")
            lo, ro = mat(lp + "o"), mat(rp + "o")
            xp, dtp = mat(rp + "x"), mat(rp + "dt")
            if (tuple(q.shape) != (nq, W) or tuple(k.shape) != (nk, W) or tuple(v.shape) != (nv, W) or
                    tuple(lo.shape) != (W, a.heads * a.vdim)):
                raise VoxB200Error(f"layer {i}: attention shapes do not match the configuration")
            if (tuple(xin.shape) != (2 * r.inner, W) or tuple(ro.shape) != (W, r.inner) or
                    tuple(xp.shape) != (r.dt_rank + 2 * r.state, r.inner) or tuple(dtp.shape) != (r.inner, r.dt_rank) or
                    tuple(sd[rp + "A_log"].shape) != (r.inner, r.state)):
                raise VoxB200Error(f"layer {i}: selective-scan shapes do not match the configuration")
            w["in"] = dense(torch.cat([q, k, v, xin], 0).contiguous())
            if a.conv >= 1:
                w["qkv_conv"] = torch.cat([vec(lp + n + ".conv") for n in ("q", "k", "v")], 0).contiguous()
                if tuple(w["qkv_conv"].shape) != (nq + nk + nv, a.conv):
                    raise VoxB200Error(f"layer {i}: short convolution shapes do not match the configuration")
            if a.qk_norm:
                w["q_norm"], w["k_norm"] = vec(lp + "q.norm"), vec(lp + "k.norm")
            w["head_bias"] = vec(lp + "pb")
            if w["head_bias"].numel() != a.heads:
                raise VoxB200Error(f"layer {i}: one score bias per head")
            w["x_conv"], w["x_conv_b"] = vec(rp + "conv"), vec(rp + "conv.b")
            if tuple(w["x_conv"].shape) != (r.inner, r.conv):
                raise VoxB200Error(f"layer {i}: selective-scan convolution shape does not match the configuration")
            w["x_proj"], w["dt_proj"], w["dt_b"] = dense(xp), dense(dtp), vec(rp + "dt.b")
            w["A"] = (-torch.exp(vec(rp + "A_log"))).contiguous()
            w["D"] = vec(rp + "D")
            w["o"] = dense(torch.cat([lo, ro], 1).contiguous())
        else:
            raise VoxB200Error(f"layer {i}: mixer '{L.kind}' is not available in post-norm blocks")
        f = L.mlp
        if f is not None:
            if not isinstance(f, MoEConfig) or f.act not in ("silu_glu", "clamped_glu"):
                raise VoxB200Error(f"layer {i}: post-norm blocks take a mixture of gated experts")
            w["norm2"] = norm(p + "norm2")[0]
            self._load_gated_moe(sd, p, f, w)
            if tuple(w["router"].shape) != (f.experts, W):
                raise VoxB200Error(f"layer {i}: router shape does not match the configuration")
        return w

    def _load_gated_layer(self, sd, p: str, i: int, L: "HybridLayerConfig", norm) -> Dict[str, Any]:
        """A pre-norm layer with gated residuals: ``l<i>.norm1`` / ``norm2``, ``l<i>.rg1[.b]`` / ``rg2[.b]`` (the gates of the
        mixer's and the feed-forward's residual), ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``.  The mixer's gate reads the
        mixer's input, so its matrix is stacked under the mixer's own input projections ("in": ONE projection per mixer).
          latent attention without a query latent: in = q | dkv | rg1; uk per head transposed, uv per head
          attention with two score maps: in = q | k | v | g | rg1, the query heads reordered per key/value group as
            [map 1 of the group's heads | map 2 of them] so that a query head's key head is (head index) / (heads per group)
          minGRU: in = z | x | g | rg1, biases of z and x in fp32"""
        mat, vec, dense, cfg, W, m = self._mat, self._vec, self._dense, self.cfg, self.cfg.width, L.mixer
        w: Dict[str, Any] = {"norm1": norm(p + "norm1")[0], "rg1_b": vec(p + "rg1.b")}
        rg1 = mat(p + "rg1")
        if tuple(rg1.shape) != (W, W):
            raise VoxB200Error(f"layer {i}: residual gate shape does not match the configuration")
        if L.kind == "latent":
            if m.q_rank or m.kv_from is not None or m.head_gate:
                raise VoxB200Error(f"layer {i}: gated blocks take latent attention with direct queries, own latents and no head gate")
            dq = m.dim + m.rot_dim
            q, dkv = mat(p + "mix.q"), mat(p + "mix.dkv")
            uk, uv, o = mat(p + "mix.uk"), mat(p + "mix.uv"), mat(p + "mix.o")
            if (tuple(q.shape) != (m.heads * dq, W) or tuple(dkv.shape) != (m.kv_rank + m.rot_dim, W) or
                    tuple(uk.shape) != (m.heads * m.dim, m.kv_rank) or tuple(uv.shape) != (m.heads * m.vdim, m.kv_rank) or
                    tuple(o.shape) != (W, m.heads * m.vdim)):
                raise VoxB200Error(f"layer {i}: latent attention shapes do not match the configuration")
            w["in"] = dense(torch.cat([q, dkv, rg1], 0).contiguous())
            w["dkv_norm"] = vec(p + "mix.dkv.norm")
            w["uk_t"] = uk.view(m.heads, m.dim, m.kv_rank).transpose(1, 2).contiguous()
            w["uv"] = uv.view(m.heads, m.vdim, m.kv_rank).contiguous()
            w["o"] = dense(o)
        elif L.kind == "diff_attention":
            H, G, D, V = m.heads, m.kv_heads, m.dim, m.vdim
            q, k, v, o = mat(p + "mix.q"), mat(p + "mix.k"), mat(p + "mix.v"), mat(p + "mix.o")
            if (tuple(q.shape) != (H * 2 * D, W) or tuple(k.shape) != (G * 2 * D, W) or tuple(v.shape) != (G * V, W) or
                    tuple(o.shape) != (W, H * V)):
                raise VoxB200Error(f"layer {i}: attention shapes do not match the configuration")
            q = q.view(G, H // G, 2, D, W).permute(0, 2, 1, 3, 4).reshape(H * 2 * D, W)
            parts = [q, k, v]
            if m.gate:
                g = mat(p + "mix.g")
                if tuple(g.shape) != (H * V, W):
                    raise VoxB200Error(f"layer {i}: attention gate shape does not match the configuration")
                parts.append(g)
            w["in"] = dense(torch.cat(parts + [rg1], 0).contiguous())
            w["o"] = dense(o)
            if m.qk_norm:
                w["q_norm"], w["k_norm"] = vec(p + "mix.q.norm"), vec(p + "mix.k.norm")
            lam = [sd[p + "mix." + n].to(torch.float64) for n in ("lq1", "lk1", "lq2", "lk2")]
            w["lambda"] = float(torch.exp((lam[0] * lam[1]).sum()) - torch.exp((lam[2] * lam[3]).sum()) + m.diff)
        elif L.kind == "mingru":
            z, x, g, o = mat(p + "mix.z"), mat(p + "mix.x"), mat(p + "mix.g"), mat(p + "mix.o")
            if any(tuple(t.shape) != (m.width, W) for t in (z, x, g)) or tuple(o.shape) != (W, m.width):
                raise VoxB200Error(f"layer {i}: minGRU shapes do not match the configuration")
            w["in"] = dense(torch.cat([z, x, g, rg1], 0).contiguous())
            w["z_b"], w["x_b"] = vec(p + "mix.z.b"), vec(p + "mix.x.b")
            w["o"] = dense(o)
        else:
            raise VoxB200Error(f"layer {i}: mixer '{L.kind}' is not available in gated blocks")
        f = L.mlp
        if f is not None:
            if not isinstance(f, GluMLPConfig):
                raise VoxB200Error(f"layer {i}: gated blocks take the clamped gated feed-forward")
            w["norm2"], w["rg2_b"] = norm(p + "norm2")[0], vec(p + "rg2.b")
            if (tuple(sd[p + "mlp.gate"].shape) != (f.ff, W) or tuple(sd[p + "mlp.up"].shape) != (f.ff, W) or
                    tuple(sd[p + "mlp.down"].shape) != (W, f.ff) or tuple(sd[p + "rg2"].shape) != (W, W)):
                raise VoxB200Error(f"layer {i}: feed-forward shapes do not match the configuration")
            w["gu"] = self._gate_up(p + "mlp.gate", p + "mlp.up")
            w["down"], w["rg2"] = dense(mat(p + "mlp.down")), dense(mat(p + "rg2"))
        return w

    def _load_latent(self, sd, p: str, i: int, m: "LatentAttentionConfig", w: Dict[str, Any]) -> None:
        """``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}``: dq | dkv | g become one projection (a layer that
        reads another layer's latents has no dkv); uk is kept per head and transposed ([H, kv_rank, dim]: it carries a
        head's query into latent space), uv per head ([H, vdim, kv_rank]: it expands a head's latent-space output)."""
        mat, vec, dense, W = self._mat, self._vec, self._dense, self.cfg.width
        own = m.kv_from is None
        if not own:
            src = self.cfg.layers[m.kv_from] if 0 <= m.kv_from < i else None
            if src is None or src.kind != "latent" or src.mixer.kv_from is not None or src.mixer.kv_rank != m.kv_rank:
                raise VoxB200Error(f"layer {i}: kv_from {m.kv_from} must name an earlier latent-attention layer that "
                                   "projects its own latents of the same rank")
        names = [p + "mix.dq"] + ([p + "mix.dkv"] if own else []) + [p + "mix.g"]
        down = mat(*names)
        if tuple(down.shape) != (m.q_rank + (m.kv_rank if own else 0) + m.heads, W):
            raise VoxB200Error(f"layer {i}: latent projection shapes do not match the configuration")
        uq, uk, uv, o = mat(p + "mix.uq"), mat(p + "mix.uk"), mat(p + "mix.uv"), mat(p + "mix.o")
        if (tuple(uq.shape) != (m.heads * m.dim, m.q_rank) or tuple(uk.shape) != (m.heads * m.dim, m.kv_rank) or
                tuple(uv.shape) != (m.heads * m.vdim, m.kv_rank) or tuple(o.shape) != (W, m.heads * m.vdim)):
            raise VoxB200Error(f"layer {i}: latent attention shapes do not match the configuration")
        w["lat_in"], w["uq"], w["o"] = dense(down), dense(uq), dense(o)
        w["dq_norm"] = vec(p + "mix.dq.norm")
        if own:
            w["dkv_norm"] = vec(p + "mix.dkv.norm")
        w["uk_t"] = uk.view(m.heads, m.dim, m.kv_rank).transpose(1, 2).contiguous()
        w["uv"] = uv.view(m.heads, m.vdim, m.kv_rank).contiguous()

    def _load_plain_moe(self, sd, p: str, i: int, f: "MoEConfig", w: Dict[str, Any]) -> None:
        """Experts of the form down(act(up h)): ``l<i>.mlp.{router, correction, e<j>.{up, down}, shared.{up, down, sg}}``.
        On tensor-core projections every expert and the shared expert are stacked into ONE up matrix (along N) and ONE down
        matrix (along K); otherwise the experts are [E, ...] stacks for the grouped linear kernel."""
        mat, vec, dense, W = self._mat, self._vec, self._dense, self.cfg.width
        w["router"] = vec(p + "mlp.router")
        w["correction"] = vec(p + "mlp.correction") if (p + "mlp.correction") in sd else None
        if tuple(w["router"].shape) != (f.experts, W):
            raise VoxB200Error(f"layer {i}: router shape does not match the configuration")
        if f.shared_ff and f.shared_gate:
            w["sg"] = vec(p + "mlp.shared.sg").reshape(-1)
        names = [f"e{e}" for e in range(f.experts)] + (["shared"] if f.shared_ff else [])
        n_all = f.experts * f.ff + f.shared_ff
        if self.tensor_core and W % 8 == 0 and n_all % 8 == 0 and f.experts <= self.DENSE_MOE_MAX_RATIO * f.top:
            fit = [r for r in (128, 64, 32, 16) if f.ff % r == 0 and f.shared_ff % r == 0]
            tr = fit[0] if fit else 128
            w["up_all"] = ops.pack_weight(torch.cat([mat(p + f"mlp.{n}.up") for n in names], 0).contiguous(), tr)
            w["down_all"] = ops.pack_weight(torch.cat([mat(p + f"mlp.{n}.down") for n in names], 1).contiguous(), 128)
            if fit and f.ff % 64 == 0:
                gb = ops.weight_tiles_bytes(f.ff, W, tr)
                w["grouped"] = {"group_bytes": gb, "kb_total": (n_all + 63) // 64, "group_kb": f.ff // 64}
                if f.shared_ff:
                    w["s_up_view"] = ops.PackedWeight(w["up_all"].data[f.experts * gb:], f.shared_ff, W, tr)
        else:
            w["up"] = torch.stack([mat(p + f"mlp.e{e}.up") for e in range(f.experts)]).contiguous()
            w["down"] = torch.stack([mat(p + f"mlp.e{e}.down") for e in range(f.experts)]).contiguous()
            if f.shared_ff:
                w["s_up"], w["s_down"] = dense(mat(p + "mlp.shared.up")), dense(mat(p + "mlp.shared.down"))

    # the dense mixture-of-experts form runs experts / top times the FLOPs a token needs: taken up to this ratio
    DENSE_MOE_MAX_RATIO = 8

    def nbytes(self) -> int:
        n = 0

        def walk(o):
            nonlocal n
            if isinstance(o, ops.PackedWeight):
                n += o.logical_bytes()
            elif isinstance(o, torch.Tensor):
                n += o.numel() * o.element_size()
            elif isinstance(o, (tuple, list)):
                for x in o:
                    walk(x)
            elif isinstance(o, dict):
                for x in o.values():
                    walk(x)
        walk([self.embed, None if self.cfg.tied_head and self.head is self.embed else self.head, self.final_norm, self.pos,
              self.side_embed, self.pair_table,
              [{k: v for k, v in L.items() if k not in ("s_gu_view", "s_up_view")} for L in self.layers]])   # (views of other entries)
        return n


# ------------------------------------------------------------------------------------------------------------------
# caches: pages for the attention layers, state slots for the recurrent layers
# ------------------------------------------------------------------------------------------------------------------
class HybridCache:
    """Per attention layer K [pages, page, G, dim] and V [pages, page, G, vdim] in the compute dtype (all layers share
    one page table: page p of every layer belongs to the same request); per latent-attention layer that projects its own
    latents ONE tensor [pages, page, 1, kv_rank (+ rot_dim)] that is both K and V (a layer reading another layer's latents aliases
    that layer's tensor); per attention layer with two score maps K [pages, page, 2 G, dim] and V [pages, page, G, vdim];
    per linear-attention layer a state [slots, H, dim, vdim] and per minGRU layer a state [slots, width] in fp32; per mixer
    pair K / V pages of its attention, fp32 pooled blocks [pages, ceil(page / pool), G, dim / vdim], the scan's state
    [slots, inner, N] and the last inputs of its short convolutions [slots, taps - 1, channels]; per layer of a stack with an
    input convolution its last inputs [slots, taps - 1, width]; with a token-pair embedding the last token of every slot.  A layer
    that a loop runs several times has one of these per pass.  Pages and slots are handed out by the worker; a slot's state is treated as zero by
    the kernels when its request starts at position 0, so nothing is cleared on reuse."""

    def __init__(self, cfg: HybridConfig, num_pages: int, page_size: int, num_slots: int, dtype: torch.dtype, device):
        self.num_pages, self.page_size, self.num_slots, self.dtype = num_pages, page_size, num_slots, dtype
        self.k: Dict[int, torch.Tensor] = {}
        self.v: Dict[int, torch.Tensor] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self.k_pool: Dict[int, torch.Tensor] = {}        # fp32 means of completed key / value blocks (pooled-window attention)
        self.v_pool: Dict[int, torch.Tensor] = {}
        self.conv: Dict[Tuple[int, str], torch.Tensor] = {}     # (run, which) -> the last taps - 1 inputs of a short convolution
        # the last token of every slot's request (stacks with a token-pair embedding)
        self.prev_tok = torch.zeros(num_slots, dtype=I32, device=device) if cfg.pair_embed is not None else None
        # one entry per layer RUN (a layer inside a loop runs several times, each pass with a cache or state of its own);
        # without a loop the run index is the layer index
        for i, (li, _) in enumerate(cfg.runs()):
            L = cfg.layers[li]
            m = L.mixer
            if L.kind == "attention":
                self.k[i] = torch.zeros(num_pages, page_size, m.kv_heads, m.dim, dtype=dtype, device=device)
                self.v[i] = torch.zeros(num_pages, page_size, m.kv_heads, m.vdim, dtype=dtype, device=device)
            elif L.kind == "diff_attention":                      # two key maps per key/value head, one value head
                self.k[i] = torch.zeros(num_pages, page_size, 2 * m.kv_heads, m.dim, dtype=dtype, device=device)
                self.v[i] = torch.zeros(num_pages, page_size, m.kv_heads, m.vdim, dtype=dtype, device=device)
            elif L.kind == "latent":
                if m.kv_from is None:                             # [latent | shared rotated key part]
                    self.k[i] = self.v[i] = torch.zeros(num_pages, page_size, 1, m.kv_rank + m.rot_dim, dtype=dtype, device=device)
                else:
                    self.k[i] = self.v[i] = self.k[m.kv_from]
            elif L.kind == "mingru":
                self.state[i] = torch.zeros(num_slots, m.width, dtype=F32, device=device)
            elif L.kind == "mixer_pair":
                a, r = m.left, m.right
                self.k[i] = torch.zeros(num_pages, page_size, a.kv_heads, a.dim, dtype=dtype, device=device)
                self.v[i] = torch.zeros(num_pages, page_size, a.kv_heads, a.vdim, dtype=dtype, device=device)
                if a.pool > 0:
                    per_page = (page_size + a.pool - 1) // a.pool
                    self.k_pool[i] = torch.zeros(num_pages, per_page, a.kv_heads, a.dim, dtype=F32, device=device)
                    self.v_pool[i] = torch.zeros(num_pages, per_page, a.kv_heads, a.vdim, dtype=F32, device=device)
                if a.conv >= 1:
                    n = a.heads * a.dim + a.kv_heads * (a.dim + a.vdim)
                    self.conv[(i, "qkv")] = torch.zeros(num_slots, max(a.conv - 1, 1), n, dtype=F32, device=device)
                self.conv[(i, "x")] = torch.zeros(num_slots, max(r.conv - 1, 1), r.inner, dtype=F32, device=device)
                self.state[i] = torch.zeros(num_slots, r.inner, r.state, dtype=F32, device=device)
            else:
                self.state[i] = torch.zeros(num_slots, m.heads, m.dim, m.vdim, dtype=F32, device=device)
            if cfg.block == "post" and cfg.input_conv > 1:
                self.conv[(i, "in")] = torch.zeros(num_slots, cfg.input_conv - 1, cfg.width, dtype=F32, device=device)

    def nbytes(self) -> int:
        seen = {t.data_ptr(): t for d in (self.k, self.v, self.state, self.k_pool, self.v_pool, self.conv)
                for t in d.values()}      # (aliases count once)
        return sum(t.numel() * t.element_size() for t in seen.values())


@dataclass
class StepInputs:
    """Device-side description of one step (all int32): ``ids`` / ``pos`` / ``row_req`` per token row, ``qo_indptr``
    [B + 1] rows of every request, ``page_indptr`` [B + 1] + ``page_indices`` its pages, ``slots`` [B] its state slot,
    ``out_rows`` the rows whose logits are computed.  ``multi`` / ``single``: whether any request brings more than one /
    exactly one token (host knowledge: selects the prompt-portion and the single-token kernels; ``single_rows`` lists the latter's
    rows for steps that have both).  ``tiles``: row tiles
    (tile_req, tile_row0, n_tiles) of the requests that bring several tokens, for the tiled attention kernel."""
    ids: torch.Tensor
    pos: torch.Tensor
    row_req: torch.Tensor
    qo_indptr: torch.Tensor
    page_indptr: torch.Tensor
    page_indices: torch.Tensor
    slots: torch.Tensor
    out_rows: torch.Tensor
    B: int
    T: int
    n_out: int
    multi: bool = True
    single: bool = True
    tiles: Optional[Tuple[torch.Tensor, torch.Tensor, int]] = None
    single_rows: Optional[Tuple[torch.Tensor, int]] = None      # the rows of the requests that bring exactly one token


class HybridEngine:
    def __init__(self, weights: HybridWeights, cache: HybridCache, max_rows: int, max_out_rows: int):
        cfg = weights.cfg
        self.w, self.cfg, self.cache, self.dtype = weights, cfg, cache, weights.dtype
        self.max_rows, self.max_out_rows = max_rows, max_out_rows
        dev, R, W, CT = weights.device, max_rows, cfg.width, weights.dtype
        att = [L.mixer for L in cfg.layers if L.kind == "attention"]
        lin = [L.mixer for L in cfg.layers if L.kind == "lightning"]
        lat = [L.mixer for L in cfg.layers if L.kind == "latent"]
        dif = [L.mixer for L in cfg.layers if L.kind == "diff_attention"]
        gru = [L.mixer for L in cfg.layers if L.kind == "mingru"]
        par = [L.mixer for L in cfg.layers if L.kind == "mixer_pair"]
        moe = [L.mlp for L in cfg.layers if isinstance(L.mlp, MoEConfig)]
        dmlp = [L.mlp for L in cfg.layers if isinstance(L.mlp, (DenseMLPConfig, GluMLPConfig))]
        gated = W if cfg.block == "gated" else 0          # the residual gate's columns ride on the mixer's input projection
        p_att = [m.heads * m.dim + m.kv_heads * (m.dim + m.vdim) + m.heads * m.vdim for m in att]
        p_lin = [2 * m.heads * (m.dim + m.vdim) for m in lin]
        p_lat = [(m.q_rank if m.q_rank else m.heads * (m.dim + m.rot_dim)) + m.kv_rank + m.rot_dim +
                 (m.heads * m.vdim if m.value_gate else m.heads) + gated for m in lat]
        p_par = [m.left.heads * m.left.dim + m.left.kv_heads * (m.left.dim + m.left.vdim) + 2 * m.right.inner for m in par]
        p_dif = [2 * (m.heads + m.kv_heads) * m.dim + m.kv_heads * m.vdim + m.heads * m.vdim + gated for m in dif]
        p_gru = [3 * m.width + gated for m in gru]
        hv = max([m.heads * m.vdim for m in att + lin + lat + dif] + [m.width for m in gru] +
                 [m.left.heads * m.left.vdim + m.right.inner for m in par] + [1])
        for m in lat:
            if m.kv_rank > 256:
                raise VoxB200Error(f"latent attention: kv_rank {m.kv_rank} exceeds the 256 dims the attention kernels take per head")
            if m.rot_dim and (m.rotary is not None and (m.rotary.dims > m.rot_dim or m.rotary.dims % 2)):
                raise VoxB200Error(f"rotary dims {m.rotary.dims} do not fit the rotated part of {m.rot_dim} dims")
        for m in dif:
            if m.heads % m.kv_heads or m.vdim > 256:
                raise VoxB200Error(f"attention: {m.heads} heads on {m.kv_heads} key/value heads of {m.vdim} values "
                                   "(heads a multiple of key/value heads, at most 256 values per head)")
        self.x = torch.zeros(R, W, dtype=F32, device=dev)              # residual stream
        self.h = torch.zeros(R, W, dtype=CT, device=dev)               # normed input of the running sublayer
        self.y = torch.zeros(R, W, dtype=F32, device=dev)              # sublayer output
        self.proj = torch.zeros(R * max(p_att + p_lin + p_lat + p_dif + p_gru + p_par + [1]), dtype=F32, device=dev)
        self.q = torch.zeros(R * max([m.heads * m.dim for m in att + lat] + [2 * m.heads * m.dim for m in dif] +
                                     [m.left.heads * m.left.dim for m in par] + [1]), dtype=CT, device=dev)
        for m in par:
            a = m.left
            if a.heads % a.kv_heads or a.dim > 256 or a.vdim > 256:
                raise VoxB200Error(f"attention: {a.heads} heads on {a.kv_heads} key/value heads of {a.dim} / {a.vdim} dims "
                                   "(heads a multiple of key/value heads, at most 256 dims per head)")
            if a.pool > 0 and a.window <= 0:
                raise VoxB200Error("pooled blocks lie before a window: mask.pool needs mask.size")
            if m.right.state > 256 or m.right.conv > 16 or a.conv > 16 or m.right.conv < 1:
                raise VoxB200Error("selective scan: at most 256 states per channel, convolutions of 1 to 16 taps")
        if par:
            # the convolved q | k | v rows, and the scan's operands: x after its convolution (fp32 for the recurrence, compute
            # type for the low-rank projection), [dt | B | C], dt's operand, the step sizes before their bias
            self.proj2 = torch.zeros(R * max(m.left.heads * m.left.dim + m.left.kv_heads * (m.left.dim + m.left.vdim) for m in par),
                                     dtype=F32, device=dev)
            inner = max(m.right.inner for m in par)
            self.scan_x = torch.zeros(R * inner, dtype=F32, device=dev)
            self.scan_xc = torch.zeros(R * inner, dtype=CT, device=dev)
            self.scan_low = torch.zeros(R * max(m.right.dt_rank + 2 * m.right.state for m in par), dtype=F32, device=dev)
            self.scan_dtl = torch.zeros(R * max(m.right.dt_rank for m in par), dtype=CT, device=dev)
            self.scan_dt = torch.zeros(R * inner, dtype=F32, device=dev)
        if cfg.pair_embed is not None:
            self.pair_rows = torch.zeros(R, dtype=I32, device=dev)
        if cfg.input_conv > 16:
            raise VoxB200Error("input convolution: at most 16 taps")
        if cfg.block == "gated":
            self.rg = torch.zeros(R, W, dtype=F32, device=dev)         # the feed-forward's residual gate before its sigmoid
            # the embedding output, added again before every repeated pass over the looped layers
            self.e0 = torch.zeros(R, W, dtype=F32, device=dev) if any(r for _, r in cfg.runs()) else None
        if dif:
            self.pair_o = torch.zeros(R * max(2 * m.heads * m.vdim for m in dif), dtype=F32, device=dev)   # both maps' outputs
        if gru:
            self.gru_scratch = None
        if cfg.block == "parallel":
            self.h2 = torch.zeros(R, W, dtype=CT, device=dev)          # the feed-forward's norm of the same stream
            self.y2 = torch.zeros(R, W, dtype=F32, device=dev)         # the feed-forward's output
        if lat:
            self.cq = torch.zeros(R * max(m.q_rank for m in lat), dtype=CT, device=dev)            # normed query latent
            n_lat = R * max(m.heads * (m.kv_rank + m.rot_dim) for m in lat)
            self.q_lat = torch.zeros(n_lat, dtype=CT, device=dev)      # queries carried into latent space (+ their rotated parts)
            self.o_lat = torch.zeros(n_lat, dtype=CT, device=dev)      # attention output in latent space
        if dmlp:
            self.ff_act = torch.zeros(R * max(f.ff for f in dmlp), dtype=CT, device=dev)
        self.mix_out = torch.zeros(R * hv, dtype=CT, device=dev)       # gated mixer output, input of the o projection
        self.lin_o = torch.zeros(R * hv, dtype=F32, device=dev)        # linear-attention output before its norm
        # scratch of the sequence-parallel linear attention: one state per tile of 64 rows (a step has at most
        # max_rows / 64 full tiles plus one partial tile per request)
        self.lin_tile_rows = ops.window_attn_tile_rows() if dev.type == "cuda" else 64
        self.lin_scratch = None
        tiled = [m for m in lin if ops.decay_attn_tile_rows(m.dim, m.vdim) == self.lin_tile_rows] if dev.type == "cuda" else []
        if tiled:
            n_t = max_rows // self.lin_tile_rows + max_out_rows + 1
            self.lin_scratch = torch.zeros(n_t * max(m.heads * m.dim * m.vdim for m in tiled), dtype=F32, device=dev)
        if gru:
            n_t = max_rows // self.lin_tile_rows + max_out_rows + 1
            self.gru_scratch = torch.zeros(ops.mingru_scratch_floats(n_t, self.lin_tile_rows, max(m.width for m in gru))
                                           if dev.type == "cuda" else 1, dtype=F32, device=dev)
        self.scan_scratch = None
        if par and dev.type == "cuda":
            n_t = max_rows // self.lin_tile_rows + cache.num_slots + 1
            self.scan_scratch = torch.zeros(max(ops.selective_scan_scratch_floats(n_t, self.lin_tile_rows, m.right.inner, m.right.state)
                                                for m in par), dtype=F32, device=dev)
        self.v_first = torch.zeros(R * max([m.kv_heads * m.vdim for m in att if m.v_mix] + [1]), dtype=F32, device=dev)
        # split-key scratch of the per-row attention kernel: steps of up to 256 rows, 8 splits
        self.attn_part = torch.zeros(256 * 8 * max([m.heads * (m.vdim + 2) for m in att] +
                                                   [2 * m.heads * (m.vdim + 2) for m in dif] +
                                                   [m.heads * (m.kv_rank + 2) for m in lat] +
                                                   [m.left.heads * (m.left.vdim + 2) for m in par] + [1]), dtype=F32, device=dev)
        self.freqs: Dict[Tuple, torch.Tensor] = {}
        self.cs: Dict[Tuple, torch.Tensor] = {}
        self.cs_mult: Dict[Tuple, float] = {}
        for m in att + dif + lat:
            rot = getattr(m, "rotary", None)
            if rot is not None and rot.key() not in self.freqs:
                if (m not in lat and rot.dims > m.dim) or rot.dims % 2:
                    raise VoxB200Error(f"rotary dims {rot.dims} do not fit head dim {m.dim}")
                self.freqs[rot.key()] = rot.frequencies().to(dev)
                self.cs[rot.key()] = torch.zeros(R, 2, rot.dims // 2, dtype=F32, device=dev)
                self.cs_mult[rot.key()] = rot.multiplier()
        if moe:
            top, E = max(f.top for f in moe), max(f.experts for f in moe)
            # grouped tensor-core form: row tiles of GROUP_TILE rows, every expert's rows padded to whole tiles
            self.moe_tiles = (R * top + self.GROUP_TILE - 1) // self.GROUP_TILE + E
            rmax = self.moe_tiles * self.GROUP_TILE
            self.moe_tile_group = torch.zeros(self.moe_tiles, dtype=I32, device=dev)
            self.moe_xs = torch.zeros(rmax * W if weights.tensor_core else 8, dtype=CT, device=dev)
            self.moe_idx = torch.zeros(R * top, dtype=I32, device=dev)
            self.moe_wts = torch.zeros(R * top, dtype=F32, device=dev)
            self.moe_row_off = torch.zeros(E + 1, dtype=I32, device=dev)
            self.moe_sorted = torch.zeros(rmax, dtype=I32, device=dev)
            self.moe_pair_row = torch.zeros(R * top, dtype=I32, device=dev)
            self.moe_act = torch.zeros(max(R * max(max(f.top * f.ff, f.experts * f.ff + f.shared_ff) for f in moe),
                                           rmax * max(f.ff for f in moe)), dtype=CT, device=dev)
            self.moe_out = torch.zeros(rmax * W, dtype=F32, device=dev)
            self.s_act = torch.zeros(R * max([f.shared_ff for f in moe] + [1]), dtype=CT, device=dev)
            self.s_out = torch.zeros(R, W, dtype=F32, device=dev)
            self.moe_sgate = torch.zeros(R, dtype=F32, device=dev)     # the shared expert's per-token gate
        self.sms = ops.device_info()[0] if dev.type == "cuda" else 1
        self.partials = torch.zeros(2 * self.sms * 128 * 256 if weights.tensor_core else 4, dtype=F32, device=dev)
        self.hn = torch.zeros(max_out_rows, W, dtype=CT, device=dev)
        self.logits = torch.zeros(max_out_rows, cfg.vocab, dtype=F32, device=dev)
        self.first_vmix = next((i for i, L in enumerate(cfg.layers) if L.kind == "attention" and L.mixer.v_mix), None)
        self.layer_tap = None          # set to a list: the residual stream after every layer is appended (tests)
        self.use_tiled_attention = True
        self.use_tiled_recurrence = True

    GROUP_TILE = 128          # rows per tile of the grouped expert projections
    GROUPED_MIN_ROWS = 512    # steps with at least this many rows run the experts grouped; smaller ones in the dense form

    # ---- projections -----------------------------------------------------------------------------------------
    def _proj(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, alpha: float = 1.0, reduce: bool = True) -> torch.Tensor:
        """out (fp32) = alpha * x @ w^T: the tcgen05 kernel for packed bf16 weights, the fp32-FMA kernel otherwise.
        reduce=False: a split-K projection returns its partial planes [split, T, N] for a consumer that sums them (the
        post-norm kernel can; measured slower than the separate, wider reduction at decode sizes, so it is not the default)."""
        if isinstance(w, ops.PackedWeight):
            assert alpha == 1.0 and out.dtype == F32 and out.is_contiguous()
            T = x.shape[0]
            # skinny problems (few weight tiles x token tiles) are split along k over all SMs into fp32 planes
            split = ops.choose_split_k(w.N, w.K, T, self.sms) if (T * w.N) % 4 == 0 else 1
            if split > 1 and split * T * w.N <= self.partials.numel():
                planes = self.partials[:split * T * w.N].view(split, T, w.N)
                ops.gemm(x, w, mode=1, split_k=split, out=planes)
                return ops.sum_planes_f32(planes, out) if reduce else planes
            ops.gemm(x, w, mode=1, split_k=1, out=out.view(1, T, w.N))
            return out
        return ops.linear(x, w, out, alpha=alpha)

    def _proj_ct(self, x: torch.Tensor, w, out: torch.Tensor, act: Optional[str] = None) -> torch.Tensor:
        """out (compute dtype) = act(x @ w^T): the activation runs in the projection's epilogue on the fp32 sum."""
        if isinstance(w, ops.PackedWeight):
            return ops.gemm(x, w, mode=0, out=out, tile_rows=w.tile_rows, act=act)
        return ops.linear(x, w, out, epilogue=ops.LINEAR_ACTS[act])

    # ---- mixers ----------------------------------------------------------------------------------------------
    def _run_attention(self, s: StepInputs, q, kc, vc, out, gate, H: int, G: int, dim: int, vdim: int, window: int,
                       scale: float, head_rows: bool = False, **kw) -> None:
        """Prompt portions on the tiled kernel and single-token rows on the per-row kernel (split over keys with few rows).
        kw: chunk, k_ld, v_ld, v_share of ``ops.window_attn``."""
        tiles = None
        if s.tiles is not None and self.use_tiled_attention and vdim <= 256:
            tiles = (s.qo_indptr, s.tiles[0], s.tiles[1], s.tiles[2])
        args = (q, kc, vc, out, gate, s.row_req, s.pos, s.page_indptr, s.page_indices, s.T, H, G, dim, vdim, window, scale)
        if tiles is not None and (not s.single or s.single_rows is not None):
            ops.window_attn(*args, tiles=tiles, **kw)
            if s.single:
                ops.window_attn(*args, scratch=self.attn_part, rows=s.single_rows, head_rows=head_rows, **kw)
        else:
            ops.window_attn(*args, scratch=self.attn_part, head_rows=head_rows, **kw)

    def _latent(self, i: int, m: LatentAttentionConfig, w: Dict[str, Any], s: StepInputs) -> torch.Tensor:
        """Latent attention in its absorbed form: a head's score q . (U_k c) equals (U_k^T q) . c and its output
        U_v (sum_j p_j c_j), so the cached latents serve every head directly as one shared key = value head of kv_rank
        dims, and neither keys nor values are ever formed per token."""
        T, H, R = s.T, m.heads, m.kv_rank
        own = m.kv_from is None
        P = m.q_rank + (R if own else 0) + H
        proj = self._proj(self.h[:T], w["lat_in"], self.proj[:T * P].view(T, P))
        cq = self.cq[:T * m.q_rank].view(T, m.q_rank)
        cache = self.cache.k[i]
        ops.latent_norm_append(proj, 0, m.q_rank, m.q_rank, R, w["dq_norm"], w.get("dkv_norm"), cq, cache if own else None,
                               s.row_req, s.pos, s.page_indptr, s.page_indices, T, self.cfg.eps)
        q = self._proj_ct(cq, w["uq"], self.q[:T * H * m.dim].view(T, H * m.dim))
        q_lat = ops.linear_batched(q.view(T, H, m.dim), w["uk_t"], self.q_lat[:T * H * R].view(T, H, R))
        o_lat = self.o_lat[:T * H * R].view(T, H * R)
        self._run_attention(s, q_lat.view(T, H * R), cache, cache, o_lat, None, H, 1, R, R, 0, m.scale, head_rows=True)
        out = self.mix_out[:T * H * m.vdim].view(T, H, m.vdim)
        ops.linear_batched(o_lat.view(T, H, R), w["uv"], out, gate=proj[:, P - H:])
        return self._proj(out.view(T, H * m.vdim), w["o"], self.y[:T])

    def _dense_mlp(self, f: DenseMLPConfig, w: Dict[str, Any], h: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        T = h.shape[0]
        act = self._proj_ct(h, w["up"], self.ff_act[:T * f.ff].view(T, f.ff), act=f.act)
        return self._proj(act, w["down"], out)

    def _attention(self, i: int, m: WindowAttentionConfig, w: Dict[str, Any], s: StepInputs) -> torch.Tensor:
        T, W = s.T, self.cfg.width
        nq, nk, nv = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
        P = nq + nk + nv + m.heads * m.vdim
        proj = self._proj(self.h[:T], w["qkvg"], self.proj[:T * P].view(T, P))
        cs, half = None, 0
        if m.rotary is not None:
            cs, half = self.cs[m.rotary.key()], m.rotary.dims // 2
        q = self.q[:T * nq].view(T, nq)
        vmix = 0 if not m.v_mix else (1 if i == self.first_vmix else 2)
        ops.qkv_rotary_append(proj, 0, nq, nq + nk, cs, half, q, self.cache.k[i], self.cache.v[i], s.row_req, s.pos,
                              s.page_indptr, s.page_indices, T, m.heads, m.kv_heads, m.dim, m.vdim, vmix,
                              self.v_first if m.v_mix else None, w.get("vmix") if vmix == 2 else None)
        out = self.mix_out[:T * m.heads * m.vdim].view(T, m.heads * m.vdim)
        gate = proj[:, nq + nk + nv:] if m.gate else None
        self._run_attention(s, q, self.cache.k[i], self.cache.v[i], out, gate, m.heads, m.kv_heads, m.dim, m.vdim, m.window,
                            m.scale)
        return self._proj(out, w["o"], self.y[:T])

    def _lightning(self, i: int, m: DecayAttentionConfig, w: Dict[str, Any], s: StepInputs) -> torch.Tensor:
        T = s.T
        nq, nv = m.heads * m.dim, m.heads * m.vdim
        P = 2 * nq + 2 * nv
        proj = self._proj(self.h[:T], w["qkvg"], self.proj[:T * P].view(T, P))
        o = self.lin_o[:T * nv].view(T, nv)
        par = (s.multi and s.tiles is not None and self.lin_scratch is not None
               and ops.decay_attn_tile_rows(m.dim, m.vdim) == self.lin_tile_rows
               and s.tiles[2] * m.heads * m.dim * m.vdim <= self.lin_scratch.numel())
        if s.single or (s.multi and not par):
            ops.decay_attn(proj, 0, nq, 2 * nq, self.cache.state[i], w["decay"], o, s.qo_indptr, s.pos, s.slots, s.B, m.heads,
                           m.dim, m.vdim, single_rows=s.single, multi_rows=s.multi and not par)
        if par:
            ops.decay_attn_tiled(proj, 0, nq, 2 * nq, self.cache.state[i], w["decay"], o, self.lin_scratch, s.qo_indptr, s.pos,
                                 s.slots, s.tiles[0], s.tiles[1], s.tiles[2], s.B, m.heads, m.dim, m.vdim)
        out = self.mix_out[:T * nv].view(T, nv)
        ops.gated_rmsnorm(o, w["norm"], proj[:, 2 * nq + nv:], self.cfg.eps, out)
        return self._proj(out, w["o"], self.y[:T])

    def _moe_plain(self, f: MoEConfig, w: Dict[str, Any], s: StepInputs, h: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Experts of the form down(act(up h)) behind the sigmoid router; the shared expert enters times its per-token gate."""
        T, W = s.T, self.cfg.width
        idx, wts = self.moe_idx[:T * f.top], self.moe_wts[:T * f.top]
        sgate = self.moe_sgate[:T] if (f.shared_ff and f.shared_gate) else None
        ops.moe_route_sigmoid(h, w["router"], w.get("correction"), f.top, idx, wts, f.groups, f.groups_keep,
                              w.get("sg") if sgate is not None else None, sgate)
        if "grouped" in w and T >= self.GROUPED_MIN_ROWS:
            g, tt = w["grouped"], self.GROUP_TILE
            n_tiles = (T * f.top + tt - 1) // tt + f.experts
            rows = n_tiles * tt
            ops.moe_group(idx, T, f.experts, f.top, self.moe_row_off, self.moe_sorted, self.moe_pair_row, tile_rows=tt,
                          tile_group=self.moe_tile_group[:n_tiles])
            xs = ops.moe_gather_rows(h, self.moe_sorted, self.moe_xs[:rows * W].view(rows, W))
            act = self.moe_act[:rows * f.ff].view(rows, f.ff)
            ops.gemm_grouped(xs, w["up_all"], act, 0, f.ff, W, tt, self.moe_tile_group, group_bytes=g["group_bytes"], act=f.act)
            eo = self.moe_out[:rows * W].view(rows, W)
            ops.gemm_grouped(act, w["down_all"], eo, 1, W, f.ff, tt, self.moe_tile_group, w_kb_stride=g["kb_total"],
                             group_kb=g["group_kb"])
            shared = None
            if f.shared_ff:
                sa = self.s_act[:T * f.shared_ff].view(T, f.shared_ff)
                ops.gemm(h, w["s_up_view"], mode=0, out=sa, tile_rows=w["s_up_view"].tile_rows, act=f.act)
                shared = ops.gemm_grouped(sa, w["down_all"], self.s_out[:T], 1, W, f.shared_ff, ops.gemm_t_tile(T), None,
                                          w_kb_stride=g["kb_total"], kb_base=f.experts * g["group_kb"])
            return ops.moe_combine(eo, shared, wts, self.moe_pair_row, f.top, out, shared_scale=sgate)
        if "up_all" in w:
            # dense form: every expert on every token as one stacked up and one stacked down projection; in between the
            # columns of an expert take the token's routing weight (or zero), the shared expert's columns its gate
            n_all = f.experts * f.ff + f.shared_ff
            act = self.moe_act[:T * n_all].view(T, n_all)
            ops.gemm(h, w["up_all"], mode=0, out=act, tile_rows=w["up_all"].tile_rows, act=f.act)
            ops.moe_scale_dense(act, idx, wts, f.experts, f.ff, f.top, sgate, f.shared_ff)
            return self._proj(act, w["down_all"], out)
        ops.moe_group(idx, T, f.experts, f.top, self.moe_row_off, self.moe_sorted, self.moe_pair_row)
        act = self.moe_act[:T * f.top * f.ff].view(T * f.top, f.ff)
        ops.linear(h, w["up"], act, epilogue=ops.LINEAR_ACTS[f.act], row_off=self.moe_row_off, gather=self.moe_sorted, rows=T)
        eo = self.moe_out[:T * f.top * W].view(T * f.top, W)
        ops.linear(act, w["down"], eo, row_off=self.moe_row_off, rows=T)
        shared = None
        if f.shared_ff:
            sa = self._proj_ct(h, w["s_up"], self.s_act[:T * f.shared_ff].view(T, f.shared_ff), act=f.act)
            shared = self._proj(sa, w["s_down"], self.s_out[:T])
        return ops.moe_combine(eo, shared, wts, self.moe_pair_row, f.top, out, shared_scale=sgate)

    def _moe(self, f: MoEConfig, w: Dict[str, Any], s: StepInputs, h: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
        T, W = s.T, self.cfg.width
        h = self.h[:T] if h is None else h
        out = self.y[:T] if out is None else out
        if f.act not in ("silu_glu", "clamped_glu"):
            return self._moe_plain(f, w, s, h, out)
        idx, wts = self.moe_idx[:T * f.top], self.moe_wts[:T * f.top]
        if f.router == "softmax_all":
            ops.moe_route_groups(h, w["router"], f.top, idx, wts, f.groups, f.groups_keep, scores="softmax", group_rank="max")
        else:
            ops.moe_route(h, w["router"], w["router_b"], f.top, idx, wts)
        glu = (f.limit, f.slope) if f.act == "clamped_glu" else None
        if "grouped" in w and T >= self.GROUPED_MIN_ROWS:
            # compute-bound steps: tokens sorted by expert into whole row tiles, each tile multiplied by its expert's slice of
            # the same packed buffers the dense form uses (tcgen05, gemm.cu), the shared expert as two plain projections
            g, tt = w["grouped"], self.GROUP_TILE
            n_tiles = (T * f.top + tt - 1) // tt + f.experts
            rows = n_tiles * tt
            ops.moe_group(idx, T, f.experts, f.top, self.moe_row_off, self.moe_sorted, self.moe_pair_row, tile_rows=tt,
                          tile_group=self.moe_tile_group[:n_tiles])
            xs = ops.moe_gather_rows(h, self.moe_sorted, self.moe_xs[:rows * W].view(rows, W))
            act = self.moe_act[:rows * f.ff].view(rows, f.ff)
            if glu:
                ops.gemm_grouped_glu(xs, w["gu_all"], act, 2 * f.ff, W, tt, self.moe_tile_group, g["group_bytes"], *glu)
            else:
                ops.gemm_grouped(xs, w["gu_all"], act, 2, 2 * f.ff, W, tt, self.moe_tile_group, group_bytes=g["group_bytes"],
                                 n_out=f.ff)
            eo = self.moe_out[:rows * W].view(rows, W)
            ops.gemm_grouped(act, w["down_all"], eo, 1, W, f.ff, tt, self.moe_tile_group, w_kb_stride=g["kb_total"],
                             group_kb=g["group_kb"])
            shared = None
            if f.shared_ff:
                sa = self.s_act[:T * f.shared_ff].view(T, f.shared_ff)
                if glu:
                    ops.gemm_glu(h, w["s_gu_view"], sa, *glu)
                else:
                    ops.gemm(h, w["s_gu_view"], mode=2, out=sa, tile_rows=w["s_gu_view"].tile_rows, n_out=f.shared_ff)
                shared = ops.gemm_grouped(sa, w["down_all"], self.s_out[:T], 1, W, f.shared_ff, ops.gemm_t_tile(T), None,
                                          w_kb_stride=g["kb_total"], kb_base=f.experts * g["group_kb"])
            return ops.moe_combine(eo, shared, wts, self.moe_pair_row, f.top, out)
        if "gu_all" in w:
            n_all = f.experts * f.ff + f.shared_ff
            act = self.moe_act[:T * n_all].view(T, n_all)
            if glu:
                ops.gemm_glu(h, w["gu_all"], act, *glu)
            else:
                ops.gemm(h, w["gu_all"], mode=2, out=act, tile_rows=w["gu_all"].tile_rows, n_out=n_all)
            ops.moe_scale_dense(act, idx, wts, f.experts, f.ff, f.top)
            return self._proj(act, w["down_all"], out)
        ops.moe_group(idx, T, f.experts, f.top, self.moe_row_off, self.moe_sorted, self.moe_pair_row)
        act = self.moe_act[:T * f.top * f.ff].view(T * f.top, f.ff)
        ops.linear(h, w["gu"], act, epilogue=1, row_off=self.moe_row_off, gather=self.moe_sorted, rows=T, glu=glu)
        eo = self.moe_out[:T * f.top * W].view(T * f.top, W)
        ops.linear(act, w["down"], eo, row_off=self.moe_row_off, rows=T)
        shared = None
        if f.shared_ff:
            sa = self.s_act[:T * f.shared_ff].view(T, f.shared_ff)
            if isinstance(w["s_gu"], ops.PackedWeight):
                if glu:
                    ops.gemm_glu(h, w["s_gu"], sa, *glu)
                else:
                    ops.gemm(h, w["s_gu"], mode=2, out=sa, tile_rows=w["s_gu"].tile_rows, n_out=f.shared_ff)
            else:
                ops.linear(h, w["s_gu"], sa, epilogue=1, glu=glu)
            shared = self._proj(sa, w["s_down"], self.s_out[:T])
        return ops.moe_combine(eo, shared, wts, self.moe_pair_row, f.top, out)

    # ---- the step --------------------------------------------------------------------------------------------
    def forward(self, s: StepInputs) -> torch.Tensor:
        """Runs the step's rows through every layer, appending to the pages and advancing the slots' states; returns the
        logits of ``s.out_rows`` as fp32 [n_out, vocab] (a view of a static buffer)."""
        cfg, w, T = self.cfg, self.w, s.T
        if T > self.max_rows or s.n_out > self.max_out_rows:
            raise VoxB200Error(f"step of {T} rows / {s.n_out} logit rows exceeds the engine's {self.max_rows} / {self.max_out_rows}")
        if cfg.block == "parallel":
            return self._forward_parallel(s)
        if cfg.block == "gated":
            return self._forward_gated(s)
        if cfg.block == "post":
            return self._forward_post(s)
        x, h, y = self.x[:T], self.h[:T], self.y[:T]
        ops.embed_rows_f32(w.embed, s.ids, x, w.pos, s.pos if w.pos is not None else None, scale=cfg.embed_scale)
        for key, freq in self.freqs.items():
            ops.rotary_table(s.pos, freq, self.cs[key][:T], self.cs_mult[key])
        eps = cfg.eps
        n = len(cfg.layers)
        if n:
            ops.layernorm_f32(x, *w.layers[0]["norm1"], eps, h)
        for i, L in enumerate(cfg.layers):
            lw = w.layers[i]
            # (a sublayer hands back its output [T, W], or the split-K planes of its last projection [split, T, W])
            ym = self._mixer(i, L, lw, s)
            nxt = w.layers[i + 1]["norm1"] if i + 1 < n else None
            if L.mlp is not None:
                ops.postnorm_residual_f32(x, ym, *lw["norm1b"], eps, h, *lw["norm2"])
                yf = self._moe(L.mlp, lw, s)
                ops.postnorm_residual_f32(x, yf, *lw["norm2b"], eps, *((h,) + nxt if nxt else (None, None, None)))
            else:
                ops.postnorm_residual_f32(x, ym, *lw["norm1b"], eps, *((h,) + nxt if nxt else (None, None, None)))
            if self.layer_tap is not None:
                self.layer_tap.append(x.clone())
        return self._head(s)

    def _mixer(self, i: int, L: HybridLayerConfig, lw: Dict[str, Any], s: StepInputs) -> torch.Tensor:
        if L.kind == "attention":
            return self._attention(i, L.mixer, lw, s)
        if L.kind == "latent":
            return self._latent(i, L.mixer, lw, s)
        return self._lightning(i, L.mixer, lw, s)

    def _head(self, s: StepInputs) -> torch.Tensor:
        """Final norm of the rows whose logits are wanted, output head, logit scale, soft cap."""
        cfg, w = self.cfg, self.w
        hn = self.hn[:s.n_out]
        packed = isinstance(w.head, ops.PackedWeight)
        nw, nb = w.final_norm_scaled if packed else w.final_norm
        if cfg.norm != "layernorm":
            ops.rmsnorm2_f32(self.x, nw, cfg.eps, hn, rows=s.out_rows)
        else:
            ops.layernorm_f32(self.x, nw, nb, cfg.eps, hn, rows=s.out_rows)
        logits = self._proj(hn, w.head, self.logits[:s.n_out], alpha=1.0 if packed else cfg.logit_scale)
        if cfg.logit_softcap:
            ops.softcap_f32(logits, cfg.logit_softcap)
        return logits

    def _forward_parallel(self, s: StepInputs) -> torch.Tensor:
        """Blocks whose mixer and feed-forward read two RMS norms of the same stream:
        x += m * (mixer(norm1 x) + ff(norm2 x)), then the per-token side input, fused with the next block's norms."""
        cfg, w, T = self.cfg, self.w, s.T
        x, h1, h2, eps = self.x[:T], self.h[:T], self.h2[:T], cfg.eps
        ops.embed_rows_f32(w.embed, s.ids, x, w.pos, s.pos if w.pos is not None else None, scale=cfg.embed_scale)
        n = len(cfg.layers)
        if n:
            ops.rmsnorm2_f32(x, w.layers[0]["norm1"], eps, h1, w.layers[0].get("norm2"), h2 if "norm2" in w.layers[0] else None)
        for i, L in enumerate(cfg.layers):
            lw = w.layers[i]
            ym = self._mixer(i, L, lw, s)
            yf = None
            if isinstance(L.mlp, DenseMLPConfig):
                yf = self._dense_mlp(L.mlp, lw, h2, self.y2[:T])
            elif L.mlp is not None:
                yf = self._moe(L.mlp, lw, s, h=h2, out=self.y2[:T])
            side = None
            if cfg.side_dim:
                side = (lw["side_gate"], lw["side_proj"], lw["side_norm"], w.side_embed, i * cfg.side_dim, s.ids)
            nxt = w.layers[i + 1] if i + 1 < n else None
            ops.residual_side_f32(x, ym, yf, cfg.residual_mult, eps, side,
                                  out1=h1 if nxt else None, w1=nxt["norm1"] if nxt else None,
                                  out2=h2 if nxt and "norm2" in nxt else None, w2=nxt.get("norm2") if nxt else None)
            if self.layer_tap is not None:
                self.layer_tap.append(x.clone())
        return self._head(s)

    # ---- pre-norm blocks with gated residuals ------------------------------------------------------------------
    def _forward_gated(self, s: StepInputs) -> torch.Tensor:
        """x += sigmoid(W_r h + b) * mixer(h) with h = norm1(x), then the same with the feed-forward on norm2(x).  A layer
        inside the loop runs once per pass on that pass's cache or state; before every pass but the first the embedding
        output is added to the stream.  The residual update, that addition and the norm feeding the next sublayer are one
        kernel (``gated_residual_norm_f32``)."""
        cfg, w, T = self.cfg, self.w, s.T
        x, h, eps = self.x[:T], self.h[:T], cfg.eps
        runs = cfg.runs()
        e0 = self.e0[:T] if self.e0 is not None else None
        ops.embed_rows_f32(w.embed, s.ids, x, scale=cfg.embed_scale, out2=e0)
        for key, freq in self.freqs.items():
            ops.rotary_table(s.pos, freq, self.cs[key][:T], self.cs_mult[key])
        if runs:
            ops.rmsnorm2_f32(x, w.layers[runs[0][0]]["norm1"], eps, h)
        for ri, (i, _) in enumerate(runs):
            L, lw = cfg.layers[i], w.layers[i]
            nxt = runs[ri + 1] if ri + 1 < len(runs) else None
            y, r = self._gated_mixer(ri, L, lw, s)
            if L.mlp is not None:
                ops.gated_residual_norm_f32(x, y, r, lw["rg1_b"], eps, out=h, w=lw["norm2"])
                y, r = self._glu_mlp(L.mlp, lw, h)
            self._gated_tail(x, y, r, lw["rg2_b" if L.mlp is not None else "rg1_b"], nxt, e0, h)
        return self._head(s)

    def _gated_tail(self, x, y, r, bias, nxt, e0, h) -> None:
        """The last residual update of a layer run, the embedding re-entering before a repeated pass, the next run's norm."""
        eps = self.cfg.eps
        nw = self.w.layers[nxt[0]]["norm1"] if nxt is not None else None
        add = e0 if (nxt is not None and nxt[1]) else None
        if self.layer_tap is None or add is None:
            ops.gated_residual_norm_f32(x, y, r, bias, eps, out=h if nw is not None else None, w=nw, add=add)
            if self.layer_tap is not None:
                self.layer_tap.append(x.clone())
            return
        ops.gated_residual_norm_f32(x, y, r, bias, eps)                 # (tapped: the stream as the layer leaves it)
        self.layer_tap.append(x.clone())
        ops.gated_residual_norm_f32(x, add, None, None, eps, out=h, w=nw)

    def _gated_mixer(self, ci: int, L: HybridLayerConfig, lw: Dict[str, Any], s: StepInputs):
        """-> (mixer output fp32 [T, W], the residual gate's pre-activation: the last W columns of the input projection)."""
        T, W, m = s.T, self.cfg.width, L.mixer
        if L.kind == "latent":
            P = m.heads * (m.dim + m.rot_dim) + m.kv_rank + m.rot_dim + W
        elif L.kind == "diff_attention":
            P = 2 * (m.heads + m.kv_heads) * m.dim + m.kv_heads * m.vdim + (m.heads * m.vdim if m.gate else 0) + W
        else:
            P = 3 * m.width + W
        proj = self._proj(self.h[:T], lw["in"], self.proj[:T * P].view(T, P))
        if L.kind == "latent":
            y = self._latent_direct(ci, m, lw, s, proj)
        elif L.kind == "diff_attention":
            y = self._diff_attention(ci, m, lw, s, proj)
        else:
            y = self._mingru(ci, m, lw, s, proj)
        return y, proj[:, P - W:]

    def _latent_direct(self, ci: int, m: LatentAttentionConfig, w: Dict[str, Any], s: StepInputs, proj: torch.Tensor,
                       gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Latent attention whose queries come straight from the input and whose heads have a rotated part, in the absorbed
        form: a head's score q_u . (U_k c) + q_r . k_r equals [U_k^T q_u | q_r] . [c | k_r], so the cached rows [c | k_r]
        serve every head as ONE key head of kv_rank + rot_dim dims whose leading kv_rank dims are also the value; the
        per-head value expansion U_v runs on the latent-space output.  proj: [queries | latent + rotated key part | ...]; a
        layer with ``kv_from`` has no latent columns and attends over the rows the named layer cached (this step's included:
        that layer ran before).  ``window`` limits the visible keys; ``gate`` (an fp32 view [T, H * vdim]): the heads' values
        times its sigmoid."""
        T, H, R, D, Rd = s.T, m.heads, m.kv_rank, m.dim, m.rot_dim
        cache = self.cache.k[ci]
        own = m.kv_from is None
        q = self.q[:T * H * D].view(T, H, D)
        q_lat = self.q_lat[:T * H * (R + Rd)].view(T, H, R + Rd)
        cs, half = (self.cs[m.rotary.key()], m.rotary.dims // 2) if (m.rotary is not None and Rd) else (None, 0)
        ops.latent_rope_append(proj, 0, H * (D + Rd), H, D, Rd, R, w.get("dkv_norm"), cs, half,
                               m.rotary.layout if m.rotary is not None else "interleaved", q, q_lat, cache if own else None,
                               s.row_req, s.pos, s.page_indptr, s.page_indices, T, self.cfg.eps)
        ops.linear_batched(q, w["uk_t"], q_lat[:, :, :R])
        o_lat = self.o_lat[:T * H * R].view(T, H * R)
        self._run_attention(s, q_lat.view(T, H * (R + Rd)), cache, cache, o_lat, None, H, 1, R + Rd, R, m.window, m.scale,
                            head_rows=True, k_ld=R + Rd, v_ld=R + Rd)
        out = self.mix_out[:T * H * m.vdim].view(T, H, m.vdim)
        if gate is not None:
            ops.linear_batched_gated(o_lat.view(T, H, R), w["uv"], out, gate)
        else:
            ops.linear_batched(o_lat.view(T, H, R), w["uv"], out)
        return self._proj(out.view(T, H * m.vdim), w["o"], self.y[:T])

    def _diff_attention(self, ci: int, m: DiffAttentionConfig, w: Dict[str, Any], s: StepInputs, proj: torch.Tensor) -> torch.Tensor:
        """Both score maps of every head run as heads of their own through the attention kernels (2 H query heads on 2 G key
        heads, consecutive key heads sharing a value head), leaving fp32 outputs that ``head_pair_combine`` subtracts,
        norms and gates."""
        T, H, G, D, V = s.T, m.heads, m.kv_heads, m.dim, m.vdim
        nq, nk, nv = 2 * H * D, 2 * G * D, G * V
        cs, half = (self.cs[m.rotary.key()], m.rotary.dims // 2) if m.rotary is not None else (None, 0)
        q = self.q[:T * nq].view(T, nq)
        kc, vc = self.cache.k[ci], self.cache.v[ci]
        ops.qkv_norm_rotary_append(proj, 0, nq, nq + nk, cs, half, m.rotary.layout if m.rotary is not None else "half",
                                   w.get("q_norm"), w.get("k_norm"), self.cfg.eps, q, kc, vc, s.row_req, s.pos, s.page_indptr,
                                   s.page_indices, T, 2 * H)
        pair = self.pair_o[:T * 2 * H * V].view(T, 2 * H * V)
        self._run_attention(s, q, kc, vc, pair, None, 2 * H, 2 * G, D, V, m.window, m.scale, chunk=m.chunk, v_share=2)
        out = self.mix_out[:T * H * V].view(T, H * V)
        gate = proj[:, nq + nk + nv:nq + nk + nv + H * V] if m.gate else None
        ops.head_pair_combine(pair, out, gate, H, H // G, V, w["lambda"], 1.0 - m.diff, self.cfg.eps)
        return self._proj(out, w["o"], self.y[:T])

    def _mingru(self, ci: int, m: MinGRUConfig, w: Dict[str, Any], s: StepInputs, proj: torch.Tensor) -> torch.Tensor:
        T, Wm = s.T, m.width
        out = self.mix_out[:T * Wm].view(T, Wm)
        state = self.cache.state[ci]
        par = (s.multi and s.tiles is not None and self.use_tiled_recurrence
               and ops.mingru_scratch_floats(s.tiles[2], self.lin_tile_rows, Wm) <= self.gru_scratch.numel())
        if s.single or (s.multi and not par):
            ops.mingru(proj, 0, Wm, 2 * Wm, w["z_b"], w["x_b"], state, out, s.qo_indptr, s.pos, s.slots, s.B,
                       single_rows=s.single, multi_rows=s.multi and not par)
        if par:
            ops.mingru_tiled(proj, 0, Wm, 2 * Wm, w["z_b"], w["x_b"], state, out, self.gru_scratch, s.qo_indptr, s.pos, s.slots,
                             s.tiles[0], s.tiles[1], s.tiles[2], self.lin_tile_rows, s.B)
        return self._proj(out, w["o"], self.y[:T])

    def _glu_mlp(self, f: GluMLPConfig, w: Dict[str, Any], h: torch.Tensor):
        """-> (down(g * sigmoid(slope g) * (u + 1)), the residual gate's pre-activation W_r h)."""
        T = h.shape[0]
        act = self.ff_act[:T * f.ff].view(T, f.ff)
        if isinstance(w["gu"], ops.PackedWeight):
            ops.gemm_glu(h, w["gu"], act, f.limit, f.slope)
        else:
            ops.linear(h, w["gu"], act, epilogue=1, glu=(f.limit, f.slope))
        r = self._proj(h, w["rg2"], self.rg[:T])
        return self._proj(act, w["down"], self.y[:T]), r

    # ---- blocks that norm sublayer outputs only ------------------------------------------------------------------
    def _forward_post(self, s: StepInputs) -> torch.Tensor:
        """x += norm1(mixer(c(x))), then x += norm2(ff(x)): the sublayers read the stream itself -- the mixer through the input
        convolution c(h) = h + conv(h) over time (state: a request's last taps - 1 rows of the stream, per layer), the
        feed-forward as it is.  The embedding may add a hashed (previous token, token) row, whose previous token lives in the
        request's slot between steps."""
        cfg, w, T = self.cfg, self.w, s.T
        x, h, eps = self.x[:T], self.h[:T], cfg.eps
        rows = None
        if cfg.pair_embed is not None:
            pe = cfg.pair_embed
            rows = ops.pair_hash_rows(self.pair_rows[:T], self.cache.prev_tok, s.ids, s.qo_indptr, s.row_req, s.pos, s.slots, T,
                                      pe.buckets, pe.mul_prev, pe.mul_cur)
        ops.embed_rows_f32(w.embed, s.ids, x, w.pair_table if rows is not None else None, rows, scale=cfg.embed_scale)
        for key, freq in self.freqs.items():
            ops.rotary_table(s.pos, freq, self.cs[key][:T], self.cs_mult[key])
        for i, L in enumerate(cfg.layers):
            lw = w.layers[i]
            if cfg.input_conv:
                # (a convolution of one tap keeps no inputs: any fp32 tensor stands in for its slot)
                ops.short_conv(x, lw["canon"], None, self.cache.conv.get((i, "in"), self.x), s.qo_indptr, s.row_req, s.pos,
                               s.slots, s.B, out=h, residual=True)
            else:
                ops.cast_rows(x, h)
            if L.kind == "latent":
                m = L.mixer
                nq = m.heads * (m.dim + m.rot_dim)
                nc = m.kv_rank + m.rot_dim if m.kv_from is None else 0
                P = nq + nc + (m.heads * m.vdim if m.value_gate else 0)
                proj = self._proj(h, lw["in"], self.proj[:T * P].view(T, P))
                y = self._latent_direct(i, m, lw, s, proj, gate=proj[:, nq + nc:] if m.value_gate else None)
            else:
                y = self._mixer_pair(i, L.mixer, lw, s)
            ops.rms_postnorm_residual_f32(x, y, lw["norm1"], eps, out=h if L.mlp is not None else None)
            if L.mlp is not None:
                ops.rms_postnorm_residual_f32(x, self._moe(L.mlp, lw, s), lw["norm2"], eps)
            if self.layer_tap is not None:
                self.layer_tap.append(x.clone())
        return self._head(s)

    def _mixer_pair(self, i: int, m: MixerPairConfig, w: Dict[str, Any], s: StepInputs) -> torch.Tensor:
        """Pooled-window sigmoid attention and a selective scan side by side on one fused input projection; both write their
        (scaled) outputs next to each other, so ONE output projection over [W_o left | W_o right] sums them."""
        T, a, r, cache, eps = s.T, m.left, m.right, self.cache, self.cfg.eps
        H, G, D, V = a.heads, a.kv_heads, a.dim, a.vdim
        nq, nk, nv, inner, N, dr = H * D, G * D, G * V, r.inner, r.state, r.dt_rank
        nqkv = nq + nk + nv
        P = nqkv + 2 * inner
        proj = self._proj(self.h[:T], w["in"], self.proj[:T * P].view(T, P))
        conv_args = (s.qo_indptr, s.row_req, s.pos, s.slots, s.B)
        # ---- left: convolutions, whole-projection norms, append, pooled blocks, attention ----
        qkv = proj[:, :nqkv]
        if a.conv >= 1:
            qkv2 = self.proj2[:T * nqkv].view(T, nqkv)
            ops.short_conv(qkv, w["qkv_conv"], None, cache.conv[(i, "qkv")], *conv_args, out_f32=qkv2)
            qkv = qkv2
        q = self.q[:T * nq].view(T, nq)
        kc, vc = cache.k[i], cache.v[i]
        ops.qk_norm_append(qkv, 0, nq, nq + nk, w.get("q_norm"), w.get("k_norm"), eps, q, kc, vc, s.row_req, s.pos, s.page_indptr,
                           s.page_indices, T)
        kp = vp = None
        if a.pool > 0:
            kp, vp = cache.k_pool[i], cache.v_pool[i]
            ops.pool_blocks(kp, vp, kc, vc, a.pool, s.qo_indptr, s.pos, s.page_indptr, s.page_indices, T, s.B)
        mix = self.mix_out[:T * (H * V + inner)].view(T, H * V + inner)
        args = (q, kc, vc, kp, vp, w["head_bias"], mix[:, :H * V], s.row_req, s.pos, s.page_indptr, s.page_indices, T, H, a.window,
                a.pool, a.scale, a.softcap, m.left_scale)
        capacity = cache.num_pages * cache.page_size
        keys = dict(scratch=self.attn_part, max_keys=(min(a.window, capacity) + capacity // max(a.pool, 1)) if a.window > 0 else capacity)
        if s.tiles is not None and self.use_tiled_attention and (not s.single or s.single_rows is not None):
            ops.sigmoid_attn(*args, tiles=(s.qo_indptr, s.tiles[0], s.tiles[1], s.tiles[2], self.lin_tile_rows))
            if s.single:
                ops.sigmoid_attn(*args, rows=s.single_rows, **keys)
        else:
            ops.sigmoid_attn(*args, **keys)
        # ---- right: convolution + silu, low-rank projection, step sizes, scan ----
        xc32, xc = self.scan_x[:T * inner].view(T, inner), self.scan_xc[:T * inner].view(T, inner)
        ops.short_conv(proj[:, nqkv:nqkv + inner], w["x_conv"], w["x_conv_b"], cache.conv[(i, "x")], *conv_args, out=xc, out_f32=xc32,
                       act="silu")
        low = self._proj(xc, w["x_proj"], self.scan_low[:T * (dr + 2 * N)].view(T, dr + 2 * N))
        dtl = ops.cast_rows(low[:, :dr], self.scan_dtl[:T * dr].view(T, dr))
        dt = self._proj(dtl, w["dt_proj"], self.scan_dt[:T * inner].view(T, inner))
        z = proj[:, nqkv + inner:]
        scan = (xc32, dt, w["dt_b"], low, dr, dr + N, z, w["A"], w["D"], cache.state[i], mix[:, H * V:], s.qo_indptr, s.pos, s.slots, s.B)
        par = (s.multi and s.tiles is not None and self.use_tiled_recurrence and self.scan_scratch is not None and
               ops.selective_scan_scratch_floats(s.tiles[2], self.lin_tile_rows, inner, N) <= self.scan_scratch.numel())
        if s.single or (s.multi and not par):
            ops.selective_scan(*scan, out_scale=m.right_scale, single_rows=s.single, multi_rows=s.multi and not par)
        if par:
            ops.selective_scan(*scan, out_scale=m.right_scale, tiles=(s.tiles[0], s.tiles[1], s.tiles[2], self.lin_tile_rows),
                               scratch=self.scan_scratch)
        return self._proj(mix, w["o"], self.y[:T])
