"""Fovunex on the hybrid engine against the plain float64 oracle (tests/fovunex_oracle.py): every mechanism alone, whole
prompts against token-by-token decoding, portions of several sizes, batches against single requests, reuse of pages and
slots, keys far away / at page borders / just inside and outside a chunk with inputs built so that a wrong key shows,
recurrent state on reused slots, other sizes, looped layers, and greedy generation through ModelWorker + Scheduler.
Small configurations with random weights; float32 is compared tightly, bfloat16 loosely.
"""
import json
import os
import tempfile

import pytest
import torch

from tests import fovunex_oracle as O

F32, BF16, I32, F64 = torch.float32, torch.bfloat16, torch.int32, torch.float64
DEV = "cuda"


# ---- CPU: configuration, registry, layer runs, cache -----------------------------------------------------------------
def test_config_reader_covers_every_branch():
    from vox_serve_b200._lib import VoxB200Error
    from vox_serve_b200.hybrid_engine import DiffAttentionConfig, GluMLPConfig, LatentAttentionConfig, MinGRUConfig
    from vox_serve_b200.model.fovunex import fovunex_config

    cfg = O.make_config(layers=("latent", "gru-", "attention", "latent-", "gru"), loop=(1, 4, 3))
    c = fovunex_config(cfg)
    assert c.block == "gated" and c.norm == "rmsnorm_scalar" and c.embed_scale == 2.0 and c.eps == 1e-5
    assert [L.kind for L in c.layers] == ["latent", "mingru", "diff_attention", "latent", "mingru"]
    assert (c.loop_start, c.loop_stop, c.loop_times) == (1, 4, 3)
    lat, gru, att = c.layers[0].mixer, c.layers[1].mixer, c.layers[2].mixer
    assert isinstance(lat, LatentAttentionConfig) and isinstance(gru, MinGRUConfig) and isinstance(att, DiffAttentionConfig)
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.q_rank, lat.scale, lat.head_gate) == (3, 8, 6, 10, 12, 0, 0.27, False)
    assert lat.rotary.layout == "interleaved" and lat.rotary.scaling == "yarn" and lat.rotary.dims == 6
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.scale, att.diff, att.chunk) == (4, 2, 12, 6, 0.29, 0.4, 9)
    assert att.rotary.layout == "half" and att.rotary.factor is None and att.rotary.dims == 8 and gru.width == 28
    assert isinstance(c.layers[0].mlp, GluMLPConfig) and c.layers[1].mlp is None and c.layers[3].mlp is None
    assert (c.layers[4].mlp.ff, c.layers[4].mlp.limit, c.layers[4].mlp.slope) == (24, 1.2, 1.702)
    # what a configuration may leave out
    c2 = fovunex_config(O.make_config(layers=("attention", "latent"), loop=None, chunk=0, a_rot=None, yarn=None, rot_dim=0))
    assert c2.layers[0].mixer.chunk == 0 and c2.layers[0].mixer.rotary is None and c2.layers[1].mixer.rotary is None
    assert c2.runs() == [(0, False), (1, False)]
    bad = O.make_config()
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(VoxB200Error):
        fovunex_config(bad)
    with pytest.raises(VoxB200Error):
        fovunex_config(O.make_config(a_heads=3, a_kv_heads=2))
    with pytest.raises(VoxB200Error):
        fovunex_config(O.make_config(loop=(1, 9, 2)))


def test_layer_runs_and_rotary_frequencies_match_the_oracle():
    from vox_serve_b200.model.fovunex import fovunex_config

    for loop in (None, (0, 4, 2), (1, 3, 3), (2, 4, 2), (0, 1, 4), (1, 1, 5), (1, 3, 1)):
        cfg = O.make_config(loop=loop)
        assert fovunex_config(cfg).runs() == O.layer_runs(cfg), loop
    for yarn, base, dims in (((4.0, 64, 8.0, 1.0), 500.0, 6), ((6.0, 1024, 24.0, 2.0), 15000.0, 24), ((2.5, 300, 3.0, 0.5), 90.0, 10),
                             (None, 1e4, 16), ((16.0, 4096, 1.0, 1.0), 1e6, 64)):
        cfg = O.make_config(layers=("latent",), loop=None, rot_dim=dims, yarn=yarn, lat_base=base)
        rot = fovunex_config(cfg).layers[0].mixer.rotary
        f, mult = O.rotary_frequencies(cfg["layers"][0]["mixer"]["rot"])
        assert torch.allclose(rot.frequencies(), torch.tensor(f, dtype=F64), rtol=1e-14, atol=0) and rot.multiplier() == mult


def test_registry_and_cache_per_layer_run():
    from vox_serve_b200.hybrid_engine import HybridCache
    from vox_serve_b200.model import get_model_class
    from vox_serve_b200.model.fovunex import FovunexModel, fovunex_config

    cfg = O.make_config()                         # latent, (gru, attention) x 2, latent
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        assert get_model_class(d) is FovunexModel
    assert get_model_class("fovunex-synthetic:3") is FovunexModel
    cache = HybridCache(fovunex_config(cfg), 5, 8, 3, torch.float32, "cpu")
    assert sorted(cache.k) == [0, 2, 4, 5] and sorted(cache.state) == [1, 3]
    assert tuple(cache.k[0].shape) == (5, 8, 1, 18) and cache.k[0].data_ptr() == cache.v[0].data_ptr()
    assert tuple(cache.k[2].shape) == (5, 8, 4, 12) and tuple(cache.v[2].shape) == (5, 8, 2, 6)
    assert cache.k[2].data_ptr() != cache.k[4].data_ptr() and tuple(cache.state[1].shape) == (3, 28)
    assert cache.state[1].data_ptr() != cache.state[3].data_ptr()


# ---- helpers ---------------------------------------------------------------------------------------------------------
def _worker(cfg, sd, dtype, slots=3, pages=24, page_size=8, max_rows=256, **kw):
    from vox_serve_b200.model.fovunex import FovunexModel
    from vox_serve_b200.worker import ModelWorker

    model = FovunexModel("fovunex-test", dtype=dtype, device="cuda:0", state_dict=sd, config=cfg, max_tokens=512, **kw)
    return ModelWorker("fovunex-test", max_batch_size=slots, max_num_pages=pages, page_size=page_size, model=model,
                       max_prefill_tokens=max_rows, max_logit_rows=max_rows)


def _replay(worker, seqs, steps, free=True):
    """steps: [[(id, count), ...], ...]; every token's logits are tapped.  Returns id -> [len, vocab] fp32 (CPU)."""
    from vox_serve_b200.requests import Request

    live, at, out = {}, {k: 0 for k in seqs}, {k: [] for k in seqs}
    for step in steps:
        reqs = []
        for rid, n in step:
            toks = seqs[rid][at[rid]:at[rid] + n]
            if rid not in live:
                live[rid] = Request(request_id=rid, prompt=list(toks))
            else:
                live[rid].pending_tokens = (live[rid].pending_tokens or []) + list(toks)
            live[rid].step_tokens, live[rid].logit_rows = n, list(range(n))
            at[rid] += n
            reqs.append(live[rid])
        inp = worker.prepare_lm_inputs(reqs, [])
        assert inp is not None and len(reqs) == len(step), [r.finish_reason for r in live.values()]
        task = (worker.run_lm_prefill if inp["is_prefill"] else worker.run_lm_decode)(reqs, inp)
        try:
            while True:
                task.send(None)
        except StopIteration:
            pass
        for rid, _ in step:
            out[rid].append(worker.step_logits(rid))
        for rid, _ in step:
            if free and at[rid] == len(seqs[rid]):
                live[rid].done_all = True
                worker.free_kv_cache(live.pop(rid))
    return {k: torch.cat(v, 0) for k, v in out.items() if v}


def _err(got, ref):
    """difference over the vocabulary (mean removed), rms, relative to the rms of the reference logits; the worst position"""
    d = got.double() - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / r.pow(2).mean().sqrt()).max().item()


TOL = {F32: 2e-4, BF16: 8e-2}


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ---- whole models ----------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_layers_and_logits_whole_prompt(dtype):
    cfg = O.make_config(layers=("latent", "gru-", "attention", "latent-", "gru"), loop=(1, 4, 2))
    sd = O.random_weights(cfg, 3)
    toks = _tokens(45, cfg["vocab"], 5)
    w = _worker(cfg, sd, dtype)
    w.engine.layer_tap = []
    got = _replay(w, {"a": toks}, [[("a", 45)]])["a"]
    taps, w.engine.layer_tap = w.engine.layer_tap, None
    ref, layers = O.forward(cfg, sd, toks)
    assert len(taps) == len(layers) == 8
    for i, (x, r) in enumerate(zip(taps, layers)):
        rel = ((x.cpu().double() - r).pow(2).mean().sqrt() / r.pow(2).mean().sqrt()).item()
        assert rel < (2e-5 if dtype == F32 else 6e-2), (i, rel)
    assert _err(got, ref) < TOL[dtype]


@pytest.mark.gpu
@pytest.mark.parametrize("layers", [("latent",), ("latent-",), ("attention",), ("attention-",), ("gru",), ("gru-",),
                                    ("gru", "gru"), ("attention", "attention")])
def test_each_mixer_alone(layers):
    for loop in (None, (0, len(layers), 3)):
        cfg = O.make_config(layers=layers, loop=loop)
        sd = O.random_weights(cfg, 11)
        toks = _tokens(30, cfg["vocab"], 2)
        got = _replay(_worker(cfg, sd, F32), {"a": toks}, [[("a", 30)]])["a"]
        assert _err(got, O.forward(cfg, sd, toks)[0]) < TOL[F32], loop


@pytest.mark.gpu
def test_other_sizes():
    """sizes and constants that differ between layers and from the defaults: one head and five, as many key/value heads as
    heads and one, key sizes that are no multiple of 8 and odd value sizes, rotation on the whole head / a slice / absent,
    no rotated part, rotated part wider than the unrotated one, YaRN on / off, chunk of 1 / 5 / larger than the prompt /
    absent, latent ranks that are no multiple of 8, recurrence wider and narrower than the model, feed-forward sizes that
    are odd, limits, loops from the first layer / to the last / three times, widths that rule the tensor-core projections
    out in bfloat16; fed in portions and token by token."""
    rot_b = {"base": 77.0, "dims": 4, "scaling": {"factor": 3.0, "original": 40, "fast": 6.0, "slow": 0.7}}
    L = [{"kind": "attention", "heads": 1, "kv_heads": 1, "dim": 10, "vdim": 7, "scale": 0.4, "diff": 0.15, "mask": {"size": 5},
          "rot": {"dims": 10, "base": 50.0}, "ff": 9, "limit": 0.6},
         {"kind": "latent", "heads": 5, "dim": 4, "rot_dim": 10, "vdim": 3, "kv_rank": 11, "scale": 0.5, "rot": rot_b},
         {"kind": "gru-", "width": 61},
         {"kind": "attention-", "heads": 6, "kv_heads": 6, "dim": 4, "vdim": 12, "scale": 0.7, "diff": 0.8, "mask": {"size": 1}},
         {"kind": "latent-", "heads": 1, "dim": 16, "rot_dim": 0, "vdim": 16, "kv_rank": 24, "scale": 0.2},
         {"kind": "attention", "heads": 6, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.3, "diff": 0.5, "mask": {"size": 1000},
          "rot": {"dims": 2, "base": 9.0}, "ff": 31, "limit": 3.0},
         {"kind": "gru", "width": 5, "ff": 16, "limit": 0.1},
         {"kind": "attention-", "heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "diff": 0.0, "mask": None, "rot": None}]
    for width, loop, scale, dtype in ((52, (0, 3, 2), 1.0, F32), (36, (5, 8, 3), 0.5, F32), (44, (2, 6, 2), 3.0, F32),
                                      (52, (3, 4, 2), 2.0, BF16)):
        cfg = O.make_config(width=width, vocab=37, layers=L, loop=loop, embed_scale=scale, eps=1e-6, a_rot=None, chunk=0)
        sd = O.random_weights(cfg, 7)
        toks = _tokens(40, 37, 1)
        ref = O.forward(cfg, sd, toks)[0]
        got = _replay(_worker(cfg, sd, dtype), {"a": toks}, [[("a", 17)], [("a", 2)], [("a", 14)]] + [[("a", 1)]] * 7)["a"]
        assert _err(got, ref) < TOL[dtype], (width, dtype)


# ---- prompts, portions, batches, reuse ----------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_prefill_decode_portions_and_batches(dtype):
    cfg = O.make_config(layers=("latent", "gru-", "attention", "gru", "latent-"), loop=(1, 4, 2), chunk=11)
    sd = O.random_weights(cfg, 5)
    V = cfg["vocab"]
    seqs = {"a": _tokens(75, V, 1), "b": _tokens(9, V, 2), "c": _tokens(40, V, 3), "d": _tokens(1, V, 4), "e": _tokens(26, V, 6)}
    ref = {k: O.forward(cfg, sd, v)[0] for k, v in seqs.items()}
    w = _worker(cfg, sd, dtype, slots=3, pages=20, page_size=8)
    # whole prompts, one at a time
    for k in ("a", "b", "d"):
        assert _err(_replay(w, {k: seqs[k]}, [[(k, len(seqs[k]))]])[k], ref[k]) < TOL[dtype], k
    # token by token from the first token on
    assert _err(_replay(w, {"c": seqs["c"]}, [[("c", 1)]] * 40)["c"], ref["c"]) < TOL[dtype]
    # portions of changing size, down to two tokens, ending inside and at page, chunk and tile borders
    for cuts in ((2, 3, 11, 8, 16, 2, 33), (64, 2, 2, 7), (7, 1, 1, 8, 58), (11, 11, 22, 31), (65, 10)):
        assert sum(cuts) == 75
        got = _replay(w, {"a": seqs["a"]}, [[("a", n)] for n in cuts])["a"]
        assert _err(got, ref["a"]) < TOL[dtype], cuts
    # the sequence-parallel recurrence against the sequential one
    w.engine.use_tiled_recurrence = False
    assert _err(_replay(w, {"a": seqs["a"]}, [[("a", 70)], [("a", 5)]])["a"], ref["a"]) < TOL[dtype]
    w.engine.use_tiled_recurrence = True
    # five unequal requests on three slots: portions beside single tokens, requests left out of steps, pages and slots
    # given back and taken again (20 pages of 8 hold 160 tokens; the five need 151 in all, never more than 3 live)
    steps = [[("a", 30), ("b", 4), ("d", 1)],
             [("a", 2), ("b", 1), ("c", 12)],
             [("b", 1), ("c", 1)],
             [("a", 40), ("b", 3), ("c", 20)],
             [("a", 1), ("c", 7)],
             [("a", 1), ("e", 13)],
             [("a", 1), ("e", 2)],
             [("e", 11)]]
    got = _replay(w, seqs, steps)
    for k in seqs:
        assert got[k].shape[0] == len(seqs[k])
        assert _err(got[k], ref[k]) < TOL[dtype], k
    assert w.empty_pages.qsize() == 20 and len(w.free_slots) == 3
    # batch against alone, bit for bit in float32: a row's result does not depend on what else is in the step
    if dtype == F32:
        alone = _replay(w, {"e": seqs["e"]}, [[("e", 13)], [("e", 2)], [("e", 11)]])["e"]
        assert torch.equal(alone, got["e"])


@pytest.mark.gpu
def test_long_decoding_across_pages_and_chunks():
    cfg = O.make_config(layers=("latent", "attention-", "gru"), loop=(0, 2, 2), chunk=37)
    sd = O.random_weights(cfg, 9)
    toks = _tokens(260, cfg["vocab"], 8)
    ref = O.forward(cfg, sd, toks)[0]
    w = _worker(cfg, sd, F32, slots=2, pages=34, page_size=8)
    got = _replay(w, {"a": toks}, [[("a", 20)]] + [[("a", 1)]] * 240)["a"]
    assert _err(got, ref) < TOL[F32]
    # the same with CUDA-graph replay of the single-token steps switched off
    w.use_cuda_graph = False
    got2 = _replay(w, {"a": toks}, [[("a", 20)]] + [[("a", 1)]] * 240)["a"]
    assert torch.equal(got, got2)


@pytest.mark.gpu
def test_bfloat16_tensor_core_sizes():
    """sizes the tcgen05 projections and the tensor-core attention tiles take: a 600-token prompt whole against the same
    prompt in portions and token by token, and the oracle."""
    cfg = O.make_config(width=128, vocab=200, layers=("latent", "gru-", "attention", "latent-"), loop=(1, 3, 2), heads=4, dim=32,
                        rot_dim=16, vdim=32, kv_rank=48, yarn=(8.0, 256, 16.0, 1.0), lat_base=10000.0, a_heads=4, a_kv_heads=2,
                        a_dim=32, a_vdim=48, chunk=150, a_rot=(32, 10000.0), gru_width=192, ff=256)
    sd = O.random_weights(cfg, 21)
    toks = _tokens(600, 200, 4)
    ref = O.forward(cfg, sd, toks)[0]
    w = _worker(cfg, sd, BF16, slots=2, pages=24, page_size=64, max_rows=640)
    from vox_serve_b200 import ops
    assert isinstance(w.engine.w.layers[0]["in"], ops.PackedWeight) and isinstance(w.engine.w.layers[0]["gu"], ops.PackedWeight)
    whole = _replay(w, {"a": toks}, [[("a", 600)]])["a"]
    parts = _replay(w, {"a": toks}, [[("a", 130)], [("a", 2)], [("a", 300)], [("a", 160)]] + [[("a", 1)]] * 8)["a"]
    assert _err(whole, ref) < TOL[BF16] and _err(parts, ref) < TOL[BF16]
    assert _err(whole, parts.double()) < TOL[BF16]


# ---- attention alone: far keys, page borders, chunk edges, the first tokens --------------------------------------------
def _pages(T, page_size, g, dtype, *shape):
    n_pages = (T + page_size - 1) // page_size
    perm = torch.randperm(n_pages + 3, generator=g)[:n_pages].to(I32)           # scattered pages
    return n_pages, perm, torch.full((n_pages + 3, page_size) + shape, float("nan"), dtype=dtype, device=DEV)


def _tiles(T):
    from vox_serve_b200 import ops

    rows = ops.window_attn_tile_rows()
    r0 = torch.arange(0, T, rows, dtype=I32, device=DEV)
    return (torch.tensor([0, T], dtype=I32, device=DEV), torch.zeros_like(r0), r0, r0.numel())


def _pair_case(T, page_size, hot, chunk, dtype, tiled, H=4, G=2, D=8, V=4):
    """One request of T positions through the attention kernels as the two-map attention uses them: 2H query heads on 2G key
    heads in the [group][map][head] order, two key heads per value head, chunk mask, fp32 output.  The key at position `hot`
    is large along axis 0 in map 1 only, all queries share that axis, and its value is 1000 in value dim 0 of every head: so
    `hot` dominates map 1 of exactly the queries that may see it.  Returns (got [T, 2H, V], ref)."""
    from vox_serve_b200 import ops

    g = torch.Generator().manual_seed(0)
    R = H // G
    q = torch.randn(T, 2 * H, D, generator=g) * 0.1
    q[:, :, 0] = 6.0
    k = torch.randn(T, 2 * G, D, generator=g) * 0.1
    k[hot, 0::2] = 0.0
    k[hot, 0::2, 0] = 6.0
    v = torch.randn(T, G, V, generator=g) * 0.1
    v[hot, :, 0] = 1000.0
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    n_pages, perm, kc = _pages(T, page_size, g, dtype, 2 * G, D)
    vc = torch.full((n_pages + 3, page_size, G, V), float("nan"), dtype=dtype, device=DEV)
    for j in range(T):
        kc[int(perm[j // page_size]), j % page_size] = k[j].to(dtype)
        vc[int(perm[j // page_size]), j % page_size] = v[j].to(dtype)
    row_req = torch.zeros(T, dtype=I32, device=DEV)
    pos = torch.arange(T, dtype=I32, device=DEV)
    indptr = torch.tensor([0, n_pages], dtype=I32, device=DEV)
    out = torch.full((T, 2 * H * V), float("nan"), dtype=F32, device=DEV)
    scratch = torch.full((T * 2 * H * 8 * (V + 2),), float("nan"), dtype=F32, device=DEV)
    ops.window_attn(q.view(T, -1).to(DEV, dtype).contiguous(), kc, vc, out, None, row_req, pos, indptr, perm.to(DEV), T, 2 * H,
                    2 * G, D, V, 0, 1.0, tiles=_tiles(T) if tiled else None, scratch=scratch if T < 100 else None, chunk=chunk,
                    v_share=2)
    ref = torch.zeros(T, 2 * H, V, dtype=F64)
    for a in range(2 * H):
        kh = a // R                                     # query heads are ordered [group][map][head]
        ref[:, a] = O.softmax_attention(q[:, a].double(), k[:, kh].double(), v[:, kh // 2].double(), 1.0, chunk)
    return out.view(T, 2 * H, V).cpu(), ref


@pytest.mark.gpu
@pytest.mark.parametrize("tiled", [False, True])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_chunked_attention_edges_far_keys_and_page_borders(tiled, dtype):
    """the hot key is seen from its own position to the end of its chunk and by nothing else: hot at the first and the last
    position of a chunk, at the first token, at page borders, chunks larger than / equal to / smaller than a page and a tile;
    no chunk (seen hundreds of positions away)."""
    tol = 2e-3 if dtype == F32 else 4e-2
    sizes = dict(H=4, G=2, D=8, V=4) if dtype == F32 else dict(H=4, G=2, D=16, V=16)
    cases = ((0, 40, 8, 0), (7, 300, 8, 0), (64, 131, 64, 0), (0, 50, 8, 13), (12, 50, 8, 13), (13, 50, 8, 13), (25, 70, 8, 13),
             (63, 200, 64, 64), (64, 200, 64, 64), (127, 200, 16, 64), (70, 300, 64, 120), (239, 300, 64, 120), (5, 20, 8, 1),
             (96, 260, 32, 100))
    for hot, T, ps, chunk in cases:
        got, ref = _pair_case(T, ps, hot, chunk, dtype, tiled, **sizes)
        assert torch.allclose(got.double(), ref, rtol=tol, atol=tol * 10), (hot, T, ps, chunk)
        for a in range(got.shape[1]):
            first_map = (a // (sizes["H"] // sizes["G"])) % 2 == 0
            sees = got[:, a, 0] > 500
            for i in range(T):
                # (the second map's key at `hot` is ordinary: it only dominates where it is the one visible key)
                want = O.visible(i, hot, chunk) if first_map else bool(ref[i, a, 0] > 500)
                assert bool(sees[i]) == want, (hot, chunk, a, i)


def _latent_rot_case(T, page_size, hot, dtype, mode, H=3, D=8, Rd=4, V=4, R=12):
    """One request through the latent-attention steps with a rotated part: cached rows [latent | rotated key part], queries
    [latent-space part | rotated part], values = the leading `R` dims of the cached rows.  Position `hot` dominates through
    its latent (axis 0) from its own position on.  Returns (got [T, H, V], ref)."""
    from vox_serve_b200 import ops

    g = torch.Generator().manual_seed(1)
    q = torch.randn(T, H, D, generator=g) * 0.1
    q[:, :, 0] = 6.0
    qr = torch.randn(T, H, Rd, generator=g) * 0.3
    kr = torch.randn(T, Rd, generator=g) * 0.3
    c = torch.randn(T, R, generator=g) * 0.1
    c[hot] = 0.0
    c[hot, 0] = 6.0
    uk = torch.randn(H * D, R, generator=g) * 0.05
    uv = torch.randn(H * V, R, generator=g) * 0.05
    for a in range(H):
        uk[a * D, 0] = 1.0
        uv[a * V, 0] = 1000.0 / 6.0
    q, qr, kr, c, uk, uv = (t.to(torch.bfloat16).float() for t in (q, qr, kr, c, uk, uv))
    n_pages, perm, cache = _pages(T, page_size, g, dtype, 1, R + Rd)
    for j in range(T):
        cache[int(perm[j // page_size]), j % page_size, 0] = torch.cat([c[j], kr[j]]).to(dtype)
    row_req = torch.zeros(T, dtype=I32, device=DEV)
    pos = torch.arange(T, dtype=I32, device=DEV)
    indptr = torch.tensor([0, n_pages], dtype=I32, device=DEV)
    q_lat = torch.zeros(T, H, R + Rd, dtype=dtype, device=DEV)
    q_lat[:, :, R:] = qr.to(DEV, dtype)
    ops.linear_batched(q.to(DEV, dtype).contiguous(), uk.view(H, D, R).transpose(1, 2).contiguous().to(DEV, dtype), q_lat[:, :, :R])
    o_lat = torch.zeros(T, H * R, dtype=dtype, device=DEV)
    scratch = torch.full((T * H * 8 * (R + 2),), float("nan"), dtype=F32, device=DEV)
    ops.window_attn(q_lat.view(T, -1), cache, cache, o_lat, None, row_req, pos, indptr, perm.to(DEV), T, H, 1, R + Rd, R, 0, 1.0,
                    tiles=_tiles(T) if mode == "tiles" else None, scratch=scratch if T < 100 else None,
                    head_rows=mode == "heads", k_ld=R + Rd, v_ld=R + Rd)
    out = ops.linear_batched(o_lat.view(T, H, R), uv.view(H, V, R).to(DEV, dtype).contiguous(),
                             torch.zeros(T, H, V, dtype=dtype, device=DEV))
    k = (c.double() @ uk.double().T).view(T, H, D)
    v = (c.double() @ uv.double().T).view(T, H, V)
    ref = torch.zeros(T, H, V, dtype=F64)
    for a in range(H):
        ref[:, a] = O.softmax_attention(torch.cat([q[:, a], qr[:, a]], 1).double(), torch.cat([k[:, a], kr.double()], 1), v[:, a], 1.0)
    return out.float().cpu(), ref


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["rows", "tiles", "heads"])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_latent_attention_with_rotated_part_far_keys_and_page_borders(mode, dtype):
    tol = 2e-3 if dtype == F32 else 4e-2
    # (bfloat16: rows of 48 and of 192 dims, the two widths of the tensor-core tile kernel's query fragments)
    all_sizes = [dict(H=3, D=8, Rd=4, V=4, R=12)] if dtype == F32 else [dict(H=2, D=16, Rd=16, V=16, R=32),
                                                                         dict(H=3, D=16, Rd=64, V=16, R=128)]
    for sizes in all_sizes:
        for hot, T, ps in ((0, 40, 8), (7, 300, 8), (8, 130, 8), (63, 200, 64), (64, 131, 64), (5, 70, 16)):
            got, ref = _latent_rot_case(T, ps, hot, dtype, mode, **sizes)
            assert torch.allclose(got.double(), ref, rtol=tol, atol=tol * 10), (hot, T, ps)
            sees = got[:, 0, 0] > 500
            for i in range(T):
                assert bool(sees[i]) == (i >= hot), (hot, i)


# ---- the other mechanisms alone ----------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_projection_tails_rotations_and_head_combination(dtype):
    """qkv_norm_rotary_append (both layouts, with and without norm, rotation on a slice), latent_rope_append, head_pair_combine
    against the oracle's functions, on scattered pages."""
    from vox_serve_b200 import ops

    g = torch.Generator().manual_seed(3)
    T, ps, eps = 21, 8, 1e-5
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == F32 else dict(rtol=2e-2, atol=2e-2)
    pos_l = [3 * i + 1 for i in range(T)]
    n_pages = (max(pos_l) + ps) // ps
    perm = torch.randperm(n_pages + 2, generator=g)[:n_pages].to(I32)
    row_req = torch.zeros(T, dtype=I32, device=DEV)
    pos = torch.tensor(pos_l, dtype=I32, device=DEV)
    indptr = torch.tensor([0, n_pages], dtype=I32, device=DEV)

    def table(rot):
        f, mult = O.rotary_frequencies(rot)
        cs = torch.zeros(T, 2, len(f), dtype=F32, device=DEV)
        return ops.rotary_table(pos, torch.tensor(f, dtype=F64, device=DEV), cs, mult)

    for layout, Hq, Gk, Gv, D, V, rdims, normed in (("half", 6, 4, 2, 10, 5, 6, True), ("interleaved", 2, 2, 2, 8, 8, 8, False),
                                                    ("half", 3, 1, 1, 12, 7, 0, True), ("half", 4, 2, 1, 16, 16, 16, True)):
        rot = {"dims": rdims, "base": 100.0} if rdims else None
        ld = (Hq + Gk) * D + Gv * V + 5
        proj = torch.randn(T, ld, generator=g).to(DEV)
        qn = (torch.rand(D, generator=g) + 0.5).to(DEV) if normed else None
        kn = (torch.rand(D, generator=g) + 0.5).to(DEV) if normed else None
        q_out = torch.zeros(T, Hq * D, dtype=dtype, device=DEV)
        kc = torch.zeros(n_pages + 2, ps, Gk, D, dtype=dtype, device=DEV)
        vc = torch.zeros(n_pages + 2, ps, Gv, V, dtype=dtype, device=DEV)
        ops.qkv_norm_rotary_append(proj, 0, Hq * D, (Hq + Gk) * D, table(rot) if rot else None, rdims // 2, layout, qn, kn, eps,
                                   q_out, kc, vc, row_req, pos, indptr, perm.to(DEV), T, Hq)
        pd = proj.double().cpu()
        qr, kr = pd[:, :Hq * D].view(T, Hq, D), pd[:, Hq * D:(Hq + Gk) * D].view(T, Gk, D)
        if normed:
            qr, kr = O.unit_rms(qr, eps) * qn.double().cpu(), O.unit_rms(kr, eps) * kn.double().cpu()
        qr, kr = O.rotate(qr, pos.cpu(), rot, layout), O.rotate(kr, pos.cpu(), rot, layout)
        assert torch.allclose(q_out.double().cpu().view(T, Hq, D), qr, **tol), layout
        for t, p_ in enumerate(pos_l):
            page, slot = int(perm[p_ // ps]), p_ % ps
            assert torch.allclose(kc[page, slot].double().cpu(), kr[t], **tol)
            assert torch.allclose(vc[page, slot].double().cpu().view(-1), pd[t, (Hq + Gk) * D:(Hq + Gk) * D + Gv * V], **tol)
    # latent tail
    for H, D, Rd, R, rdims, yarn in ((3, 8, 6, 12, 6, True), (2, 5, 0, 9, 0, False), (1, 4, 8, 16, 4, False)):
        rot = {"dims": rdims, "base": 300.0} if rdims else None
        if yarn:
            rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
        ld = H * (D + Rd) + R + Rd + 3
        proj = torch.randn(T, ld, generator=g).to(DEV)
        wc = (torch.rand(R, generator=g) + 0.5).to(DEV)
        q_out = torch.zeros(T, H, D, dtype=dtype, device=DEV)
        q_lat = torch.zeros(T, H, R + Rd, dtype=dtype, device=DEV)
        cache = torch.zeros(n_pages + 2, ps, 1, R + Rd, dtype=dtype, device=DEV)
        ops.latent_rope_append(proj, 0, H * (D + Rd), H, D, Rd, R, wc, table(rot) if rot else None, rdims // 2, "interleaved",
                               q_out, q_lat, cache, row_req, pos, indptr, perm.to(DEV), T, eps)
        pd = proj.double().cpu()
        q = pd[:, :H * (D + Rd)].view(T, H, D + Rd)
        dkv = pd[:, H * (D + Rd):H * (D + Rd) + R + Rd]
        c = O.unit_rms(dkv[:, :R], eps) * wc.double().cpu()
        assert torch.allclose(q_out.double().cpu(), q[:, :, :D], **tol)
        if Rd:
            assert torch.allclose(q_lat[:, :, R:].double().cpu(), O.rotate(q[:, :, D:], pos.cpu(), rot, "interleaved"), **tol)
        k_rot = O.rotate(dkv[:, R:], pos.cpu(), rot, "interleaved")
        for t, p_ in enumerate(pos_l):
            row = cache[int(perm[p_ // ps]), p_ % ps, 0].double().cpu()
            assert torch.allclose(row[:R], c[t], **tol) and torch.allclose(row[R:], k_rot[t], **tol)
    # two maps per head -> one output per head
    for H, R_, V, lam, diff in ((4, 2, 6, 0.37, 0.4), (3, 3, 33, -0.2, 0.0), (2, 1, 64, 1.1, 0.9)):
        a = torch.randn(T, 2 * H * V, generator=g).to(DEV)
        gate = torch.randn(T, H * V + 4, generator=g).to(DEV)
        out = ops.head_pair_combine(a, torch.zeros(T, H * V, dtype=dtype, device=DEV), gate[:, 2:2 + H * V], H, R_, V, lam, 1.0 - diff, eps)
        av = a.double().cpu().view(T, H // R_, 2, R_, V)
        o = (av[:, :, 0] - lam * av[:, :, 1]).reshape(T, H, V)
        ref = (O.unit_rms(o, eps) * (1.0 - diff)).reshape(T, H * V) * O.sigmoid(gate[:, 2:2 + H * V].double().cpu())
        assert torch.allclose(out.double().cpu(), ref, **tol)


@pytest.mark.gpu
def test_mingru_state_slots_tiles_and_portions():
    """the recurrence over requests of unequal length on scattered slots that hold garbage: whole, in portions that end
    inside tiles, token by token; sequential and tile-parallel forms; gates made so that a lost or stale state shows (update
    gates near 0 keep the state for hundreds of tokens)."""
    from vox_serve_b200 import ops

    g = torch.Generator().manual_seed(5)
    Wm, ld = 37, 3 * 37 + 6
    lens = [150, 1, 70, 64, 3]
    sd = {"z": torch.eye(Wm), "x": torch.eye(Wm), "g": torch.eye(Wm), "o": torch.eye(Wm),
          "z.b": torch.randn(Wm, generator=g) - 3.0, "x.b": torch.randn(Wm, generator=g)}
    tile = ops.window_attn_tile_rows()
    for cuts in ([None], [64, 64, 22], [1] * 6 + [100, 44], [130, 2, 18], [63, 65, 22]):
        state = torch.full((7, Wm), float("nan"), dtype=F32, device=DEV)
        slots_of = [5, 0, 3, 6, 2]
        at = [0] * len(lens)
        hs = [torch.randn(n, Wm, generator=g) for n in lens]
        outs = [[] for _ in lens]
        n_steps = len(cuts)
        for step in range(n_steps):
            rows, qo, slots, pos, tile_req, tile_row0, present = [], [0], [], [], [], [], []
            for b, n in enumerate(lens):
                k = n - at[b] if cuts[step] is None or step == n_steps - 1 else min(cuts[step], n - at[b])
                if k <= 0:
                    continue
                bi = len(slots)
                if k > 1:
                    for r0 in range(0, k, tile):
                        tile_req.append(bi)
                        tile_row0.append(qo[-1] + r0)
                rows.append(hs[b][at[b]:at[b] + k])
                pos += list(range(at[b], at[b] + k))
                slots.append(slots_of[b])
                qo.append(qo[-1] + k)
                at[b] += k
                present.append((b, bi))
            h = torch.cat(rows)
            T = h.shape[0]
            proj = torch.zeros(T, ld, dtype=F32)
            proj[:, 2:2 + Wm], proj[:, 2 + Wm:2 + 2 * Wm], proj[:, 4 + 2 * Wm:4 + 3 * Wm] = h, 2 * h, 0.5 * h
            dev = lambda x, dt=I32: torch.tensor(x, dtype=dt, device=DEV)
            res = {}
            for par in (False, True):
                st = state.clone()
                out = torch.full((T, Wm), float("nan"), dtype=F32, device=DEV)
                multi = any(qo[i + 1] - qo[i] > 1 for i in range(len(slots)))
                single = any(qo[i + 1] - qo[i] == 1 for i in range(len(slots)))
                if par and tile_req:
                    scratch = torch.full((ops.mingru_scratch_floats(len(tile_req), tile, Wm),), float("nan"), dtype=F32, device=DEV)
                    if single:
                        ops.mingru(proj.to(DEV), 2, 2 + Wm, 4 + 2 * Wm, sd["z.b"].to(DEV), sd["x.b"].to(DEV), st, out, dev(qo), dev(pos),
                                   dev(slots), len(slots), single_rows=True, multi_rows=False)
                    ops.mingru_tiled(proj.to(DEV), 2, 2 + Wm, 4 + 2 * Wm, sd["z.b"].to(DEV), sd["x.b"].to(DEV), st, out, scratch,
                                     dev(qo), dev(pos), dev(slots), dev(tile_req), dev(tile_row0), len(tile_req), tile, len(slots))
                else:
                    ops.mingru(proj.to(DEV), 2, 2 + Wm, 4 + 2 * Wm, sd["z.b"].to(DEV), sd["x.b"].to(DEV), st, out, dev(qo), dev(pos),
                               dev(slots), len(slots), single_rows=single, multi_rows=multi)
                res[par] = (st, out)
            assert torch.allclose(res[False][1], res[True][1], rtol=1e-5, atol=1e-6)
            state = res[True][0]
            for b, bi in present:
                outs[b].append(res[True][1][qo[bi]:qo[bi + 1]].cpu())
        for b, n in enumerate(lens):
            # the projection columns are h, 2 h and h / 2: the oracle's recurrence with those matrices and an identity output
            ref, S = O.mingru(hs[b].double(), {"z": sd["z"], "x": 2 * sd["x"], "g": 0.5 * sd["g"], "o": sd["o"], "z.b": sd["z.b"],
                                               "x.b": sd["x.b"]}, "")
            got = torch.cat(outs[b])
            assert torch.allclose(got.double(), ref, rtol=1e-5, atol=1e-6), (cuts, b)
            assert torch.allclose(state[slots_of[b]].double().cpu(), S, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("W,T", [(44, 19), (42, 7), (384, 130)])
def test_gated_residual_norm_embedding_scale_and_clamped_feed_forward(W, T):
    from vox_serve_b200 import ops

    g = torch.Generator().manual_seed(W)
    eps = 1e-5
    x, y, add = (torch.randn(T, W, generator=g) for _ in range(3))
    r = torch.randn(T, W + 12, generator=g)
    bias, nw = torch.randn(W, generator=g), torch.full((W,), 1.3)
    for use_add, use_gate, dt in ((True, True, F32), (False, True, BF16), (True, False, F32), (False, False, F32)):
        xd = x.clone().to(DEV)
        out = torch.zeros(T, W, dtype=dt, device=DEV)
        ops.gated_residual_norm_f32(xd, y.to(DEV), r.to(DEV)[:, 4:4 + W] if use_gate else None, bias.to(DEV) if use_gate else None,
                                    eps, out=out, w=nw.to(DEV), add=add.to(DEV) if use_add else None)
        gate = O.sigmoid(r[:, 4:4 + W].double() + bias.double()) if use_gate else 1.0
        xr = x.double() + gate * y.double() + (add.double() if use_add else 0.0)
        assert torch.allclose(xd.double().cpu(), xr, rtol=1e-6, atol=1e-6)
        tol = 1e-5 if dt == F32 else 2e-2
        assert torch.allclose(out.double().cpu(), O.scalar_norm(xr, torch.tensor(1.3, dtype=F64), eps), rtol=tol, atol=tol)
    # without a norm output
    xd = x.clone().to(DEV)
    ops.gated_residual_norm_f32(xd, y.to(DEV), None, None, eps)
    assert torch.allclose(xd.cpu(), x + y, rtol=1e-6, atol=1e-6)
    # embedding times a constant, with a second copy
    table = torch.randn(31, W, generator=g).to(torch.bfloat16)
    ids = torch.randint(0, 31, (T,), generator=g).to(I32)
    o1, o2 = torch.zeros(T, W, device=DEV), torch.zeros(T, W, device=DEV)
    ops.embed_rows_f32(table.to(DEV), ids.to(DEV), o1, scale=2.5, out2=o2)
    assert torch.equal(o1.cpu(), table.float()[ids.long()] * 2.5) and torch.equal(o1, o2)
    # the clamped gated form in both projection kernels
    ff, limit = (40, 0.8) if W != 384 else (128, 1.25)
    h = torch.randn(T, W, generator=g).to(torch.bfloat16)
    gw, uw = (torch.randn(ff, W, generator=g) * 2 * W ** -0.5).to(torch.bfloat16), (torch.randn(ff, W, generator=g) * 2 * W ** -0.5).to(torch.bfloat16)
    gg = torch.clamp(h.double() @ gw.double().T, max=limit)
    uu = torch.clamp(h.double() @ uw.double().T, min=-limit, max=limit)
    ref = gg * O.sigmoid(1.702 * gg) * (uu + 1.0)
    assert float((gg == limit).double().mean()) > 0.02 and float((uu.abs() == limit).double().mean()) > 0.04
    out = torch.zeros(T, ff, dtype=F32, device=DEV)
    ops.linear(h.float().to(DEV), torch.cat([gw, uw]).float().to(DEV), out, epilogue=1, glu=(limit, 1.702))
    assert torch.allclose(out.double().cpu(), ref, rtol=1e-4, atol=1e-5)
    if W % 8 == 0:
        half = ops.gate_up_tile_half(ff)
        pw = ops.pack_weight(ops.interleave_gate_up(gw.to(DEV), uw.to(DEV), half), 2 * half)
        ob = torch.zeros(T, ff, dtype=BF16, device=DEV)
        ops.gemm_glu(h.to(DEV), pw, ob, limit, 1.702)
        assert torch.allclose(ob.double().cpu(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_greedy_generation_through_scheduler(dtype):
    """ModelWorker + Scheduler: three requests of unequal prompts, prompts fed in portions of 16 beside decoding requests,
    more requests than slots.  Tokens equal the oracle's greedy tokens wherever the oracle's top-2 margin is clear."""
    from vox_serve_b200.requests import Request
    from vox_serve_b200.sampling import SamplingConfig
    from vox_serve_b200.scheduler import Scheduler

    cfg = O.make_config(layers=("latent", "gru-", "attention", "latent-"), loop=(1, 3, 2))
    sd = O.random_weights(cfg, 13, head_gain=6.0)
    prompts = {"r0": _tokens(41, cfg["vocab"], 1), "r1": _tokens(5, cfg["vocab"], 2), "r2": _tokens(23, cfg["vocab"], 3)}
    n_new = 12
    w = _worker(cfg, sd, dtype, slots=2, pages=40, page_size=8)
    sch = Scheduler(w, prefill_chunk_tokens=16)
    reqs = {}
    for rid, p in prompts.items():
        reqs[rid] = Request(request_id=rid, prompt=p, sampling_config=SamplingConfig(greedy=True, max_tokens=n_new))
        sch.submit(reqs[rid])
    sch.run_until_done(max_steps=400)
    assert len(sch.finished) == 3 and w.empty_pages.qsize() == 40 and len(w.free_slots) == 2
    margin = 0.05 if dtype == F32 else 0.6
    wrong = 0
    for rid, p in prompts.items():
        got = [int.from_bytes(c, "little", signed=True) for c in sch.audio[rid]]
        assert len(got) == n_new and reqs[rid].finish_reason == "max_tokens_reached"
        toks = list(p)
        for t in got:                       # teacher-forced comparison: every step is judged on the framework's own prefix
            z = O.forward(cfg, sd, toks)[0][-1]
            top = torch.topk(z, 2)
            if float(top.values[0] - top.values[1]) > margin:
                wrong += t != int(top.indices[0])
            toks.append(t)
    assert wrong == 0, wrong


def _write_model_dir(d, cfg, sd):
    """config.json + model.safetensors (8-byte length, JSON header, raw little-endian data) of a bfloat16 checkpoint"""
    import struct

    meta, blobs, off = {}, [], 0
    for k, v in sd.items():
        raw = v.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
        meta[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    head = json.dumps(meta).encode()
    with open(os.path.join(d, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)


@pytest.mark.gpu
def test_command_lines_on_a_model_directory(capsys):
    """a checkpoint directory (scalar norm weights as 0-dim tensors) through the trace replay tool (a subprocess: portions,
    two requests, a request ended and its slot taken again) and through the generate command (in process)."""
    import subprocess
    import sys

    import numpy as np

    from vox_serve_b200 import generate

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = O.make_config(layers=("latent", "gru-", "attention", "latent-"), loop=(1, 3, 2))
    sd = O.random_weights(cfg, 17, head_gain=6.0)
    V = cfg["vocab"]
    a, b, c = _tokens(30, V, 1), _tokens(12, V, 2), _tokens(9, V, 3)
    with tempfile.TemporaryDirectory() as d:
        _write_model_dir(d, cfg, sd)
        out = os.path.join(d, "out")
        steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [0, 19]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
                 {"step": 1, "entries": [{"id": "a", "tokens": a[20:21], "want": [0]}, {"id": "b", "tokens": b[2:], "want": [9]}], "end": ["b"]},
                 {"step": 2, "entries": [{"id": "c", "tokens": c, "want": [8]}, {"id": "a", "tokens": a[21:], "want": [8]}], "end": ["a", "c"]}]
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                            "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                           text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
        ra, rb, rc = (O.forward(cfg, sd, t)[0] for t in (a, b, c))
        want = {0: torch.stack([ra[0], ra[19]]), 1: torch.stack([ra[20], rb[11]]), 2: torch.stack([rc[8], ra[29]])}
        for s_, ref in want.items():
            got = torch.from_numpy(np.fromfile(os.path.join(out, f"{s_}.f32"), dtype="<f4").reshape(2, V).copy())
            assert _err(got, ref) < TOL[F32], s_
        capsys.readouterr()
        assert generate.main(["--model", d, "--prompt", " ".join(map(str, a)), "--prompt", " ".join(map(str, b)), "--max-new", "6",
                              "--dtype", "float32", "--prefill-chunk", "16", "--page-size", "8"]) == 0
        lines = capsys.readouterr().out.strip().splitlines()[-2:]
        for line, prompt in zip(lines, (a, b)):
            toks = list(prompt)
            for t in (int(x) for x in line.split()):
                z = O.forward(cfg, sd, toks)[0][-1]
                top = torch.topk(z, 2)
                assert float(top.values[0] - top.values[1]) < 0.05 or t == int(top.indices[0])
                toks.append(t)
            assert len(toks) == len(prompt) + 6
