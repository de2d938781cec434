"""Prefill and decode throughput of the Bobavik design (hybrid engine) beside the Llama-shaped engine of the speech LMs at
equal size: same width, layer count, head count and head size, and a dense feed-forward as wide as the experts a token
uses (top * ff + shared ff).  Random weights, a few layers of a real model's shape.

    python bench.py --arch bobavik [--arch-sizes 2048,3072] [--steps K] [--warmup W]

``--arch razevik``: the Razevik design (latent attention, parallel blocks, sigmoid group router, side input) beside its
closest relative on the same engine, Bobavik with softmax-attention layers only, at equal width, heads, head size and
expert sizes.

``--arch fovunex``: the Fovunex design (gated pre-norm blocks; latent attention with a shared rotated key part, attention with
two score maps per head in chunks, minGRU, clamped gated dense feed-forward) beside Bobavik (softmax attention and linear
attention with a recurrent state, mixture of experts) at equal width, head count and feed-forward width per token.

``--arch nadevik``: the Nadevik design (post-norm blocks with an input convolution; windowed latent attention with a shared
rotated key part, own and shared cached rows; pooled-window sigmoid attention beside a selective scan; group-limited softmax
router over clamped gated experts; tied head) beside Bobavik (window attention, linear attention with a recurrent state,
mixture of experts) at equal width, head count, head size and expert width per token.

Per size and engine: prefill of one 1024-token prompt (eager launches) and one decode step of 32 requests at context 512
(a CUDA-graph replay, as served), timed with CUDA events after warm-up; an L2-sized buffer is overwritten between timed
iterations.  Output: one JSON line per size.
"""
from __future__ import annotations

import json

import torch

PROMPT, BATCH, CONTEXT, LAYERS, VOCAB = 1024, 32, 512, 4, 32000


def razevik_config(width: int, ff: int, experts: int = 8, top: int = 2) -> dict:
    """four blocks: own latents + dense feed-forward, then (shared, own, shared) with experts, as small models of the
    design are laid out; 128-wide heads, a key/value latent of 128 dims, a query latent of 3/8 of the width"""
    heads = width // 128
    mix = {"heads": heads, "dim": 128, "vdim": 128, "kv_rank": 128, "q_rank": width * 3 // 8, "scale": 128 ** -0.5}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}, "expert": {"ff": ff},
           "shared": {"ff": ff}}
    layers = []
    for i in range(LAYERS):
        m = dict(mix)
        if i % 2:
            m["kv_from"] = i - 1
        layers.append({"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": 3 * ff} if i == 0 else dict(moe)})
    return {"architecture": "Razevik", "width": width, "vocab": VOCAB, "max_positions": 2048, "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "token_side": {"dim": 32}, "logit_softcap": 30.0, "layers": layers}


def fovunex_config(width: int, ff: int) -> dict:
    """four layers: latent attention + feed-forward, minGRU, two-map attention + feed-forward, latent attention + feed-forward;
    128-wide heads (latent attention: 128 unrotated + 64 rotated dims on a latent of 128; two-map attention: two maps of 64
    dims on 128-wide values, a quarter as many key/value heads), chunks of 4096 positions, a dense feed-forward as wide as the
    experts a Bobavik token uses"""
    heads = width // 128
    lat = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 128, "scale": 192 ** -0.5,
           "rot": {"base": 1e4, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    att = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 64, "vdim": 128, "scale": 64 ** -0.5, "diff": 0.5,
           "mask": {"size": 4096}, "rot": {"dims": 64, "base": 1e6}}
    mlp = {"kind": "dense", "ff": 3 * ff, "limit": 7.0}
    layers = [{"type": "latent_attention", "mixer": dict(lat), "mlp": dict(mlp)},
              {"type": "mingru", "mixer": {"width": width}, "mlp": None},
              {"type": "attention", "mixer": dict(att), "mlp": dict(mlp)},
              {"type": "latent_attention", "mixer": dict(lat), "mlp": dict(mlp)}]
    return {"architecture": "Fovunex", "width": width, "vocab": VOCAB, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "layers": layers}


def nadevik_config(width: int, ff: int, experts: int = 8, top: int = 3) -> dict:
    """four layers: latent attention (own cached rows), two mixer pairs, latent attention reading the first layer's rows; every
    layer with experts.  128-wide heads (latent attention: 128 unrotated + 64 rotated dims on a latent of 128, window 4096;
    sigmoid attention: a quarter as many key/value heads, window 512 with pooled blocks of 16, convolutions of 3 taps; scan:
    twice the width, 16 states, step sizes of rank width / 16, convolution of 4 taps); 8 experts in 4 groups (keep 3), top 3 --
    the expert width a Bobavik token uses (top 2 + shared)"""
    heads = width // 128
    lat = {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 128, "scale": 192 ** -0.5, "mask": {"size": 4096},
           "rot": {"base": 1e4, "dims": 64}}
    left = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 30.0,
            "conv": 3, "mask": {"size": 512, "pool": 16}}
    right = {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}
    pair = {"left": left, "right": right, "left_scale": 0.7, "right_scale": 0.7}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 3}}}
    layers = [{"type": "latent_attention", "mixer": dict(lat), "mlp": dict(mlp)},
              {"type": "parallel", "mixer": dict(pair), "mlp": dict(mlp)},
              {"type": "parallel", "mixer": dict(pair), "mlp": dict(mlp)},
              {"type": "latent_attention", "mixer": dict(lat, kv_from=0), "mlp": dict(mlp)}]
    return {"architecture": "Nadevik", "width": width, "vocab": VOCAB, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
            "embedding": {"scale": 1.0, "bigram": {"buckets": 8191, "mul_prev": 31, "mul_cur": 7}}, "layers": layers}


def bobavik_config(width: int, ff: int, experts: int = 8, top: int = 2, window: int = 4096,
                   kinds=("attention", "lightning", "lightning", "attention")) -> dict:
    heads = width // 128
    att = {"heads": heads, "kv_heads": max(1, heads // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "v_mix": True,
           "mask": {"size": window}, "rot": {"dims": 64, "base": 1e6,
                                             "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    lin = {"heads": heads, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** -(5 + 3 * h / heads) for h in range(heads)]}
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": {"ff": ff}}
    kinds = list(kinds)
    return {"architecture": "Bobavik", "width": width, "vocab": VOCAB, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": [{"type": k, "mixer": dict(att if k == "attention" else lin), "mlp": dict(mlp)}
                       for k in (kinds * LAYERS)[:LAYERS]]}


def _timed(fn, steps: int, warmup: int, flush: torch.Tensor) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(steps):
        flush.add_(1)                                   # > L2: evicts what the last iteration left there
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / steps


def _graph(fn):
    torch.cuda.synchronize()
    g, s = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            fn()
    torch.cuda.current_stream().wait_stream(s)
    return g.replay


def bench_bobavik(width: int, ff: int, steps: int, warmup: int, flush, kinds=None, design: str = "bobavik") -> dict:
    from vox_serve_b200 import ops
    from vox_serve_b200.hybrid_engine import StepInputs
    from vox_serve_b200.model.bobavik import BobavikModel
    from vox_serve_b200.model.fovunex import FovunexModel
    from vox_serve_b200.model.nadevik import NadevikModel
    from vox_serve_b200.model.razevik import RazevikModel

    if design == "nadevik":
        model = NadevikModel("nadevik-synthetic:1", config=nadevik_config(width, ff), device="cuda:0")
    elif design == "fovunex":
        model = FovunexModel("fovunex-synthetic:1", config=fovunex_config(width, ff), device="cuda:0")
    elif design == "razevik":
        model = RazevikModel("razevik-synthetic:1", config=razevik_config(width, ff), device="cuda:0")
    else:
        cfg = bobavik_config(width, ff, **({"kinds": kinds} if kinds else {}))
        model = BobavikModel("bobavik-synthetic:1", config=cfg, device="cuda:0")
    page = 64
    pages_per_req = (CONTEXT + page) // page + 1
    n_pages = max(BATCH * pages_per_req, PROMPT // page + 1)
    cache = model.make_cache(n_pages, page, BATCH)
    eng = model.make_engine(cache, max(PROMPT, BATCH), BATCH)
    dev, I32 = "cuda", torch.int32

    def step(n_req: int, rows_per_req: int, pos0: int, per_req_pages: int, tiled: bool):
        T = n_req * rows_per_req
        ids = torch.randint(0, VOCAB, (T,), device=dev, dtype=I32)
        pos = (torch.arange(rows_per_req, device=dev, dtype=I32) + pos0).repeat(n_req)
        row_req = torch.arange(n_req, device=dev, dtype=I32).repeat_interleave(rows_per_req)
        qo = torch.arange(n_req + 1, device=dev, dtype=I32) * rows_per_req
        indptr = torch.arange(n_req + 1, device=dev, dtype=I32) * per_req_pages
        indices = torch.arange(n_req * per_req_pages, device=dev, dtype=I32)
        tiles = None
        if tiled:
            R = ops.window_attn_tile_rows()
            r0 = torch.arange(0, T, R, device=dev, dtype=I32)
            tiles = (torch.div(r0, rows_per_req, rounding_mode="floor").to(I32), r0, r0.numel())
        return StepInputs(ids=ids, pos=pos, row_req=row_req, qo_indptr=qo, page_indptr=indptr, page_indices=indices,
                          slots=torch.arange(n_req, device=dev, dtype=I32), out_rows=(qo[1:] - 1).contiguous(), B=n_req, T=T,
                          n_out=n_req, multi=rows_per_req > 1, single=rows_per_req == 1, tiles=tiles)

    pre = step(1, PROMPT, 0, PROMPT // page + 1, True)
    t_pre = _timed(lambda: eng.forward(pre), steps, warmup, flush)
    dec = step(BATCH, 1, CONTEXT, pages_per_req, False)
    eng.forward(dec)
    t_dec = _timed(_graph(lambda: eng.forward(dec)), steps, warmup, flush)
    return {"prefill_ms": t_pre, "prefill_tok_s": PROMPT / t_pre * 1e3, "decode_ms": t_dec,
            "decode_tok_s": BATCH / t_dec * 1e3, "weight_gb": model.weights.nbytes() / 1e9}


def bench_llama(width: int, inter: int, steps: int, warmup: int, flush) -> dict:
    from vox_serve_b200 import ops
    from vox_serve_b200.engine import LlamaDims, LlamaEngine, LlamaWeights
    from vox_serve_b200.model.orpheus import synthetic_state_dict

    heads = width // 128
    dims = LlamaDims(width, LAYERS, heads, max(1, heads // 4), 128, inter, VOCAB)
    w = LlamaWeights.from_state_dict(synthetic_state_dict(dims, 1, "cuda"), dims, "cuda")
    page = 64
    pages_per_req = (CONTEXT + page) // page + 1
    n_pages = max(BATCH * pages_per_req, PROMPT // page + 1)
    kv = torch.zeros(LAYERS, n_pages, 2, page, dims.num_key_value_heads, 128, dtype=torch.bfloat16, device="cuda")
    eng = LlamaEngine(w, kv, page, max_rows=PROMPT + 64)
    dev, I32 = "cuda", torch.int32

    def prefill():
        ids = torch.randint(0, VOCAB, (PROMPT,), device=dev, dtype=I32)
        pos = torch.arange(PROMPT, device=dev, dtype=I32)
        qo = torch.tensor([0, PROMPT], device=dev, dtype=I32)
        indptr = torch.tensor([0, PROMPT // page], device=dev, dtype=I32)
        indices = torch.arange(PROMPT // page, device=dev, dtype=I32)
        last = torch.tensor([page], device=dev, dtype=I32)
        last_rows = torch.tensor([PROMPT - 1], device=dev, dtype=I32)

        def run():
            ops.plan_rows(eng.plan, qo, indptr, indices, last, 1, PROMPT, page, eng.chunk)
            eng.forward(ids, pos, PROMPT, last_rows=last_rows)
        return run

    def decode():
        ids = torch.randint(0, VOCAB, (BATCH,), device=dev, dtype=I32)
        pos = torch.full((BATCH,), CONTEXT, device=dev, dtype=I32)
        indptr = torch.arange(BATCH + 1, device=dev, dtype=I32) * pages_per_req
        indices = torch.arange(BATCH * pages_per_req, device=dev, dtype=I32)
        last = torch.full((BATCH,), (CONTEXT + 1) % page or page, device=dev, dtype=I32)

        def run():
            ops.plan_rows(eng.plan, None, indptr, indices, last, BATCH, BATCH, page, eng.chunk)
            eng.forward(ids, pos, BATCH)
        return run

    t_pre = _timed(prefill(), steps, warmup, flush)
    d = decode()
    d()
    t_dec = _timed(_graph(d), steps, warmup, flush)
    return {"prefill_ms": t_pre, "prefill_tok_s": PROMPT / t_pre * 1e3, "decode_ms": t_dec,
            "decode_tok_s": BATCH / t_dec * 1e3, "weight_gb": w.nbytes() / 1e9}


def run(sizes, steps: int, warmup: int, only: str = "", arch: str = "bobavik") -> None:
    flush = torch.zeros(192 << 20, dtype=torch.uint8, device="cuda")
    for width in sizes:
        ff = width                     # expert width; a token uses top (2) experts + the shared one
        if arch == "fovunex":
            line = {"bench": "fovunex_vs_bobavik", "width": width, "layers": LAYERS, "prompt": PROMPT, "decode_batch": BATCH,
                    "context": CONTEXT, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic",
                    "l2": "192 MiB buffer overwritten between timed iterations"}
            if only in ("", "fovunex"):
                line["fovunex"] = bench_bobavik(width, ff, steps, warmup, flush, design="fovunex")
            if only in ("", "bobavik"):
                line["bobavik"] = bench_bobavik(width, ff, steps, warmup, flush)
            print(json.dumps(line), flush=True)
            torch.cuda.empty_cache()
            continue
        if arch == "nadevik":
            line = {"bench": "nadevik_vs_bobavik", "width": width, "layers": LAYERS, "prompt": PROMPT, "decode_batch": BATCH,
                    "context": CONTEXT, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic",
                    "l2": "192 MiB buffer overwritten between timed iterations"}
            if only in ("", "nadevik"):
                line["nadevik"] = bench_bobavik(width, ff, steps, warmup, flush, design="nadevik")
            if only in ("", "bobavik"):
                line["bobavik"] = bench_bobavik(width, ff, steps, warmup, flush)
            print(json.dumps(line), flush=True)
            torch.cuda.empty_cache()
            continue
        if arch == "razevik":
            line = {"bench": "razevik_vs_bobavik_attention", "width": width, "layers": LAYERS, "prompt": PROMPT,
                    "decode_batch": BATCH, "context": CONTEXT, "steps": steps, "warmup": warmup, "dtype": "bf16",
                    "data": "synthetic", "l2": "192 MiB buffer overwritten between timed iterations"}
            if only in ("", "razevik"):
                line["razevik"] = bench_bobavik(width, ff, steps, warmup, flush, design="razevik")
            if only in ("", "bobavik"):
                line["bobavik_attention"] = bench_bobavik(width, ff, steps, warmup, flush, kinds=("attention",) * LAYERS)
            print(json.dumps(line), flush=True)
            torch.cuda.empty_cache()
            continue
        line = {"bench": "bobavik_vs_llama", "width": width, "layers": LAYERS, "prompt": PROMPT, "decode_batch": BATCH,
                "context": CONTEXT, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic",
                "l2": "192 MiB buffer overwritten between timed iterations"}
        if only in ("", "bobavik"):
            line["bobavik"] = bench_bobavik(width, ff, steps, warmup, flush)
        if only in ("", "llama"):
            line["llama"] = bench_llama(width, 3 * ff, steps, warmup, flush)
        print(json.dumps(line), flush=True)
        torch.cuda.empty_cache()
