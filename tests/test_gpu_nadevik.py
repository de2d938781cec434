"""Nadevik on the hybrid engine against the plain float64 oracle (tests/nadevik_oracle.py): every mechanism alone, whole prompts
against token-by-token decoding, portions of several sizes, batches against single requests, reuse of pages and slots, keys
far away / at page borders / just inside and outside a window or a pooled block with inputs built so that a wrong key shows,
recurrent and convolution state on reused slots, other sizes, and greedy generation through ModelWorker + Scheduler.
Small configurations with random weights; float32 is compared tightly, bfloat16 loosely.
"""
import json
import os
import tempfile

import pytest
import torch

from tests import nadevik_oracle as O

F32, BF16, I32, F64 = torch.float32, torch.bfloat16, torch.int32, torch.float64
DEV = "cuda"


# ---- CPU: configuration, registry, cache, the oracle's own rules ------------------------------------------------------
def test_config_reader_covers_every_branch():
    from vox_serve_b200._lib import VoxB200Error
    from vox_serve_b200.hybrid_engine import LatentAttentionConfig, MixerPairConfig, MoEConfig
    from vox_serve_b200.model.nadevik import nadevik_config

    c = nadevik_config(O.make_config())
    assert (c.block, c.norm, c.embed_scale, c.eps, c.tied_head, c.input_conv) == ("post", "rmsnorm_offset", 3.0, 1e-5, True, 3)
    assert (c.pair_embed.buckets, c.pair_embed.mul_prev, c.pair_embed.mul_cur) == (53, 5, 3)
    assert [L.kind for L in c.layers] == ["latent", "mixer_pair", "mixer_pair", "latent", "mixer_pair"]
    lat, pair, shared = c.layers[0].mixer, c.layers[1].mixer, c.layers[3].mixer
    assert isinstance(lat, LatentAttentionConfig) and isinstance(pair, MixerPairConfig)
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.kv_rank, lat.q_rank, lat.scale, lat.window) == (3, 8, 6, 10, 12, 0, 0.27, 11)
    assert lat.value_gate and not lat.head_gate and lat.kv_from is None and shared.kv_from == 0
    assert lat.rotary.layout == "interleaved" and lat.rotary.factor is None and (lat.rotary.dims, lat.rotary.base) == (6, 300.0)
    a, r = pair.left, pair.right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.pool, a.softcap, a.conv) == (4, 2, 12, 6, 0.31, 9, 4, 5.0, 3)
    assert (r.inner, r.state, r.dt_rank, r.conv) == (40, 5, 6, 4) and (pair.left_scale, pair.right_scale) == (0.7, 1.3)
    f = c.layers[0].mlp
    assert isinstance(f, MoEConfig) and c.layers[2].mlp is None
    assert (f.experts, f.top, f.ff, f.act, f.router, f.groups, f.groups_keep, f.limit, f.slope) == (
        6, 2, 24, "clamped_glu", "softmax_all", 3, 2, 1.2, 1.702)
    # what a configuration may leave out
    c2 = nadevik_config(O.make_config(layers=("pair", "latent"), bigram=None, canon=0, l_rot=0, l_window=0, a_pool=0, a_cap=0.0,
                                      a_conv=0, groups=None))
    assert c2.pair_embed is None and c2.input_conv == 0 and c2.layers[1].mixer.rotary is None and c2.layers[1].mixer.window == 0
    assert (c2.layers[0].mixer.left.pool, c2.layers[0].mixer.left.softcap, c2.layers[0].mixer.left.conv) == (0, 0.0, 0)
    assert c2.layers[0].mlp.groups == 0
    bad = O.make_config()
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(VoxB200Error):
        nadevik_config(bad)
    with pytest.raises(VoxB200Error):
        nadevik_config(O.make_config(a_heads=3, a_kv_heads=2))
    with pytest.raises(VoxB200Error):
        nadevik_config(O.make_config(groups=(3, 1), top=3))
    with pytest.raises(VoxB200Error):
        nadevik_config(O.make_config(l_rot=4, l_rot_dims=6))


def test_registry_and_cache():
    from vox_serve_b200.hybrid_engine import HybridCache
    from vox_serve_b200.model import build_profile, get_model_class
    from vox_serve_b200.model.nadevik import NadevikModel, nadevik_config

    cfg = O.make_config()
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        assert get_model_class(d) is NadevikModel and build_profile(d) == "text_conv"
    assert get_model_class("nadevik-synthetic:3") is NadevikModel
    cache = HybridCache(nadevik_config(cfg), 5, 8, 3, torch.float32, "cpu")
    assert sorted(cache.k) == [0, 1, 2, 3, 4] and sorted(cache.state) == [1, 2, 4] and sorted(cache.k_pool) == [1, 2, 4]
    assert tuple(cache.k[0].shape) == (5, 8, 1, 18) and cache.k[0].data_ptr() == cache.v[0].data_ptr() == cache.k[3].data_ptr()
    assert tuple(cache.k[1].shape) == (5, 8, 2, 12) and tuple(cache.v[1].shape) == (5, 8, 2, 6)
    assert tuple(cache.k_pool[1].shape) == (5, 2, 2, 12) and cache.k_pool[1].dtype == torch.float32
    assert tuple(cache.state[1].shape) == (3, 40, 5) and tuple(cache.conv[(1, "qkv")].shape) == (3, 2, 4 * 12 + 2 * 18)
    assert tuple(cache.conv[(1, "x")].shape) == (3, 3, 40) and tuple(cache.conv[(0, "in")].shape) == (3, 2, 48)
    assert tuple(cache.prev_tok.shape) == (3,) and cache.state[1].data_ptr() != cache.state[2].data_ptr()
    # a pool that does not divide the page: blocks are kept per page of their first position
    c2 = HybridCache(nadevik_config(O.make_config(layers=("pair",), a_pool=3)), 5, 8, 3, torch.float32, "cpu")
    assert tuple(c2.k_pool[0].shape) == (5, 3, 2, 12)


def test_oracle_visibility_and_router_by_hand():
    assert O.window_keys(10, 4) == [7, 8, 9, 10] and O.window_keys(2, 4) == [0, 1, 2] and O.window_keys(3, 0) == [0, 1, 2, 3]
    # window 4, pool 3: block 0 = positions 0..2 is seen once 2 <= i - 4
    assert O.pooled_blocks(5, 4, 3) == [] and O.pooled_blocks(6, 4, 3) == [0] and O.pooled_blocks(8, 4, 3) == [0]
    assert O.pooled_blocks(9, 4, 3) == [0, 1] and O.pooled_blocks(100, 0, 3) == [] and O.pooled_blocks(100, 4, 0) == []
    s = torch.tensor([0.05, 0.30, 0.10, 0.11, 0.25, 0.19], dtype=F64)
    assert O.route(s, 2, 0, 0) == [1, 4]
    assert O.route(s, 2, 3, 2) == [1, 4]                  # groups (0,1) (2,3) (4,5): best scores .30 .11 .25 -> groups 0 and 2
    assert O.route(s, 3, 3, 2) == [1, 4, 5]               # expert 3 (.11) is outside the kept groups although it beats .05
    assert O.route(s, 2, 3, 1) == [1, 0] and O.route(s, 1, 2, 1) == [1]
    assert O.bigram_rows([4, 9, 9], {"buckets": 7, "mul_prev": 3, "mul_cur": 5}) == [7, (12 + 45) % 7, (27 + 45) % 7]


# ---- helpers ---------------------------------------------------------------------------------------------------------
def _worker(cfg, sd, dtype, slots=3, pages=24, page_size=8, max_rows=256, **kw):
    from vox_serve_b200.model.nadevik import NadevikModel
    from vox_serve_b200.worker import ModelWorker

    model = NadevikModel("nadevik-test", dtype=dtype, device="cuda:0", state_dict=sd, config=cfg, max_tokens=512, **kw)
    return ModelWorker("nadevik-test", max_batch_size=slots, max_num_pages=pages, page_size=page_size, model=model,
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


def _err50(got, ref):
    """the same, the median over positions.  bfloat16 is judged so: with several routed layers a near-tie in a router chooses
    another expert than the oracle at a few places per sequence, which moves those positions and, through windows and
    recurrent states, some after them by tens of percent, while every other position stays within a few percent; a wrong
    bfloat16 kernel moves them all.  What only shows at single positions (edges, first tokens) is judged in float32."""
    d = got.double() - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return torch.quantile(d.pow(2).mean(-1).sqrt() / r.pow(2).mean().sqrt(), 0.5).item()


TOL = {F32: 2e-4, BF16: 8e-2}


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ---- whole models ----------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_layers_and_logits_whole_prompt(dtype):
    cfg = O.make_config()
    sd = O.make_weights(cfg, 3, calm=dtype == BF16)
    toks = _tokens(45, cfg["vocab"], 5)
    w = _worker(cfg, sd, dtype)
    w.engine.layer_tap = []
    got = _replay(w, {"a": toks}, [[("a", 45)]])["a"]
    taps, w.engine.layer_tap = w.engine.layer_tap, None
    layers = []
    ref = O.forward(cfg, sd, toks, layers)
    assert len(taps) == len(layers) == 5
    for i, (x, r) in enumerate(zip(taps, layers)):
        rel = (x.cpu().double() - r).pow(2).mean(-1).sqrt() / r.pow(2).mean().sqrt()        # per token
        # (bfloat16: the median over tokens, see _err50)
        assert (rel.max().item() < 1e-4) if dtype == F32 else (torch.quantile(rel, 0.5).item() < 6e-2), (i, rel.max().item())
    assert (_err if dtype == F32 else _err50)(got, ref) < TOL[dtype]


@pytest.mark.gpu
@pytest.mark.parametrize("layers", [("latent",), ("latent-",), ("pair",), ("pair-",), ("latent-", "shared:0"), ("pair", "pair"),
                                    ("latent", "pair-", "shared:0-", "latent", "shared:3")])
def test_each_mixer_alone(layers):
    cfg = O.make_config(layers=layers)
    sd = O.make_weights(cfg, 11)
    toks = _tokens(30, cfg["vocab"], 2)
    got = _replay(_worker(cfg, sd, F32), {"a": toks}, [[("a", 30)]])["a"]
    assert _err(got, O.forward(cfg, sd, toks)) < TOL[F32]


OTHER_SIZES = [
    dict(l_heads=1, a_heads=1, a_kv_heads=1, top=1, groups=None),
    dict(l_heads=5, a_heads=6, a_kv_heads=6, a_dim=5, a_vdim=9, experts=4, top=4, groups=(2, 2)),
    dict(a_heads=6, a_kv_heads=1, a_dim=16, a_vdim=16, l_dim=16, l_vdim=4, l_rank=7, width=44, ff=20),
    dict(l_rot=0, l_window=1, a_window=1, a_pool=1, canon=1, a_conv=1, s_conv=1, s_state=1, s_rank=1),
    dict(l_rot=8, l_rot_dims=4, l_window=0, a_window=0, a_pool=0, a_cap=0.0, canon=0, a_conv=0, bigram=None, embed_scale=1.0),
    dict(a_window=5, a_pool=3, s_state=9, s_conv=2, a_conv=5, canon=5, left_scale=1.0, right_scale=1.0, limit=0.3),
    dict(a_window=7, a_pool=11, s_state=20, s_inner=24, experts=8, top=3, groups=(4, 2), bigram=(7, 11, 13)),
    dict(a_window=13, a_pool=8, s_state=40, s_inner=56, s_rank=9, groups=(1, 1), top=6),
    dict(a_window=4, a_pool=2, s_state=70, s_inner=16, width=36, experts=3, top=2, groups=(3, 2), vocab=31),
]


@pytest.mark.gpu
@pytest.mark.parametrize("kw", OTHER_SIZES)
def test_other_sizes(kw):
    """head counts of one and many, key/value heads = heads and = 1, key size != value size, odd sizes that rule tensor-core
    projections out, windows of one / none, pools of one / that do not divide the page / longer than it, convolutions of one
    and five taps, one state and seventy, top = 1 and = all eligible experts, one group and none, no pair embedding."""
    cfg = O.make_config(layers=("latent", "pair", "shared:0-", "pair-"), **kw)
    sd = O.make_weights(cfg, 7)
    toks = _tokens(41, cfg["vocab"], 3)
    ref = O.forward(cfg, sd, toks)
    got = _replay(_worker(cfg, sd, F32), {"a": toks}, [[("a", 41)]])["a"]
    assert _err(got, ref) < TOL[F32]
    got = _replay(_worker(cfg, sd, F32), {"a": toks}, [[("a", 17)], [("a", 2)], [("a", 9)]] + [[("a", 1)]] * 13)["a"]
    assert _err(got, ref) < TOL[F32]
    sd = O.make_weights(cfg, 7, calm=True)
    got = _replay(_worker(cfg, sd, BF16), {"a": toks}, [[("a", 17)], [("a", 2)], [("a", 9)]] + [[("a", 1)]] * 13)["a"]
    assert _err50(got, O.forward(cfg, sd, toks)) < TOL[BF16]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_prefill_decode_portions_and_batches(dtype):
    """whole prompt = token by token from the first token = portions of 1 ... 64 tokens cut inside pages, windows and pooled
    blocks = batches of five unequal requests on three slots with requests left out of steps and reused pages and slots."""
    cfg = O.make_config()
    sd = O.make_weights(cfg, 5, calm=dtype == BF16)
    V = cfg["vocab"]
    seqs = {k: _tokens(n, V, i) for i, (k, n) in enumerate((("a", 70), ("b", 9), ("c", 33), ("d", 1), ("e", 26)))}
    ref = {k: O.forward(cfg, sd, t) for k, t in seqs.items()}
    err = _err if dtype == F32 else _err50
    w = _worker(cfg, sd, dtype, pages=40)
    whole = _replay(w, seqs, [[(k, len(t))] for k, t in seqs.items()])
    ref_all = torch.cat([ref[k] for k in seqs], 0)
    if dtype == F32:
        for k in seqs:
            assert err(whole[k], ref[k]) < TOL[dtype], k
    else:                                   # (the median needs more positions than the short requests have: all of them together)
        assert err(torch.cat([whole[k] for k in seqs], 0), ref_all) < TOL[dtype]
    one = _replay(w, {"a": seqs["a"]}, [[("a", 1)]] * 70)["a"]
    assert err(one, ref["a"]) < TOL[dtype]
    for cuts in ([2, 2, 3, 1, 5, 7, 11, 13, 2, 24], [64, 2, 4], [3, 64, 3], [8, 8, 8, 8, 8, 8, 8, 8, 6], [9, 4, 4, 53]):
        assert sum(cuts) == 70
        got = _replay(w, {"a": seqs["a"]}, [[("a", n)] for n in cuts])["a"]
        assert err(got, ref["a"]) < TOL[dtype], cuts
        if dtype == F32:
            assert (got - whole["a"]).abs().max().item() < 2e-4 * ref["a"].abs().max().item(), cuts
    # five requests on three slots: portions beside single tokens, requests left out of steps, slots and pages taken again
    steps = [[("a", 5), ("b", 2)], [("a", 1), ("b", 1), ("c", 20)], [("b", 6), ("c", 1)], [("a", 30), ("c", 12)],
             [("a", 1)], [("d", 1), ("a", 2)], [("e", 3), ("a", 31)], [("e", 1)], [("e", 22)]]
    got = _replay(w, seqs, steps)
    for k in seqs:
        if dtype == F32:
            assert err(got[k], ref[k]) < TOL[dtype], k
            assert (got[k] - whole[k]).abs().max().item() < 2e-4 * ref[k].abs().max().item(), k
    assert err(torch.cat([got[k] for k in seqs], 0), ref_all) < TOL[dtype]
    assert w.empty_pages.qsize() == 40 and len(w.free_slots) == 3


@pytest.mark.gpu
def test_long_decoding_across_pages_windows_and_pools():
    cfg = O.make_config(layers=("latent", "pair", "shared:0", "pair-"))
    sd = O.make_weights(cfg, 9)
    toks = _tokens(250, cfg["vocab"], 4)
    ref = O.forward(cfg, sd, toks)
    for graph in (True, False):
        w = _worker(cfg, sd, F32, pages=40)
        w.use_cuda_graph = graph
        got = _replay(w, {"a": toks}, [[("a", 10)]] + [[("a", 1)]] * 240)["a"]
        assert _err(got, ref) < TOL[F32], graph


@pytest.mark.gpu
def test_bfloat16_tensor_core_sizes():
    """sizes whose projections run on the tensor-core kernels (multiples of 8 / 16 / 64): a 600-token prompt whole (tiled
    attention, the scan in pieces) against portions (single rows among them) and the oracle"""
    cfg = O.make_config(layers=("latent", "pair", "shared:0", "pair"), width=128, vocab=160, l_heads=4, l_dim=32, l_rot=16, l_vdim=32,
                        l_rank=64, l_window=100, a_heads=4, a_kv_heads=2, a_dim=32, a_vdim=32, a_window=90, a_pool=16, s_inner=192,
                        s_state=16, s_rank=8, experts=8, top=2, ff=64, groups=(4, 2))
    sd = O.make_weights(cfg, 21, calm=True)
    toks = _tokens(600, cfg["vocab"], 6)
    ref = O.forward(cfg, sd, toks)
    w = _worker(cfg, sd, BF16, slots=2, pages=24, page_size=64, max_rows=1024)
    whole = _replay(w, {"a": toks}, [[("a", 600)]])["a"]
    parts = _replay(w, {"a": toks}, [[("a", 130)], [("a", 1)], [("a", 300)], [("a", 2)], [("a", 167)]])["a"]
    # over 600 tokens the experts that roundings re-route add up through the scans' states, so the tensor-core projections are
    # judged against the same bfloat16 arithmetic on the plain projection kernel (same roundings, other summation order), and
    # that against the oracle loosely
    plain = _replay(_worker(cfg, sd, BF16, slots=2, pages=24, page_size=64, max_rows=1024, tensor_core_projections=False),
                    {"a": toks}, [[("a", 600)]])["a"]
    assert _err50(whole, plain.double()) < 3e-2 and _err50(parts, plain.double()) < 3e-2
    assert _err50(plain, ref) < 0.2 and _err50(whole[:40], ref[:40]) < 0.15
    w32 = _worker(cfg, sd, F32, slots=2, pages=24, page_size=64, max_rows=1024)
    assert _err(_replay(w32, {"a": toks}, [[("a", 600)]])["a"], ref) < TOL[F32]
    w32.engine.use_tiled_recurrence = w32.engine.use_tiled_attention = False
    assert _err(_replay(w32, {"a": toks}, [[("a", 333)], [("a", 267)]])["a"], ref) < TOL[F32]


# ---- single mechanisms -----------------------------------------------------------------------------------------------
def _paged(n_req_tokens, page_size, seed=0, spare=3):
    """scattered pages for requests of the given lengths -> (page_indptr, page_indices, number of pages)"""
    need = [(n + page_size - 1) // page_size for n in n_req_tokens]
    total = sum(need) + spare
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).tolist()
    indptr, idx = [0], []
    for n in need:
        idx += perm[len(idx):len(idx) + n]
        indptr.append(len(idx))
    return torch.tensor(indptr, dtype=I32, device=DEV), torch.tensor(idx, dtype=I32, device=DEV), total


def _step_tables(spans):
    """spans: per request (first position, rows) -> qo_indptr, row_req, pos (device int32)"""
    qo, row_req, pos = [0], [], []
    for b, (p0, n) in enumerate(spans):
        row_req += [b] * n
        pos += list(range(p0, p0 + n))
        qo.append(qo[-1] + n)
    mk = lambda v: torch.tensor(v, dtype=I32, device=DEV)
    return mk(qo), mk(row_req), mk(pos)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("window,pool,page", [(9, 4, 8), (6, 3, 8), (16, 16, 8), (5, 1, 4), (7, 0, 8), (0, 0, 8)])
def test_sigmoid_attention_window_and_pool_edges(dtype, window, pool, page):
    """One key is made to dominate (its score far above a strongly negative head bias, every other weight ~ 0), so the output
    says exactly who sees it: from its own position to distance window - 1 as a token, not at all until its block lies wholly
    before the window, then through the block's mean -- in whole prompts (tiles), portions cut at every place, single rows
    (with and without dealing a row's keys to several CTAs), across page borders, and for keys far away."""
    from vox_serve_b200 import ops

    torch.manual_seed(1)
    H, G, D, V, T = 4, 2, 16, 8, 75
    hot = 21
    q = torch.randn(T, H, D, dtype=F64) * 0.05
    k = torch.randn(T, G, D, dtype=F64) * 0.05
    v = torch.randn(T, G, V, dtype=F64)
    k[hot, :, 0] = 6.0 * max(pool, 1)                 # (strong enough to dominate its block's mean too)
    q[:, :, 0] = 4.0
    bias = torch.tensor([-14.0, -13.0, -15.0, -14.5], dtype=F64)
    scale, cap = 0.9, 30.0
    q, k, v = (t.to(dtype).to(F64) for t in (q, k, v))
    ref = O.sigmoid_attend(q, k, v, bias, scale, cap, window, pool)
    # the reference itself shows the pattern the test is after
    mag = ref.abs().sum((1, 2))
    assert mag[hot] > 1.0 and (window == 0 or mag[hot + window - 1] > 1.0)
    if window and not pool:
        assert mag[hot + window] < 1e-3
    if window and pool:
        first_seen = (hot // pool) * pool + pool - 1 + window
        assert mag[hot + window:first_seen].max() < 1e-3 if first_seen > hot + window else True
        if first_seen < T:
            assert mag[first_seen] > 1e-3
    indptr, pages, n_pages = _paged([T], page, seed=3)
    tile_rows = ops.window_attn_tile_rows()
    tol = 1e-5 if dtype == F32 else 2e-2
    for cuts in ([T], [1] * T, [hot + 1, window or 5, 3, 1, 1, 2, T - hot - 8 - (window or 5)], [30, 45]):
        assert sum(cuts) == T
        kc = torch.full((n_pages, page, G, D), float("nan"), dtype=dtype, device=DEV)
        vc = torch.full((n_pages, page, G, V), float("nan"), dtype=dtype, device=DEV)
        per = (page + pool - 1) // pool if pool else 1
        kp = torch.full((n_pages, per, G, D), float("nan"), dtype=F32, device=DEV)
        vp = torch.full((n_pages, per, G, V), float("nan"), dtype=F32, device=DEV)
        scratch = torch.zeros(1 << 16, dtype=F32, device=DEV)
        out = torch.zeros(T, H * V + 3, dtype=dtype, device=DEV)
        p0 = 0
        for n in cuts:
            qo, row_req, pos = _step_tables([(p0, n)])
            proj = torch.cat([q[p0:p0 + n].reshape(n, -1), k[p0:p0 + n].reshape(n, -1), v[p0:p0 + n].reshape(n, -1)], 1).to(F32).to(DEV)
            qd = torch.zeros(n, H * D, dtype=dtype, device=DEV)
            ops.qk_norm_append(proj.contiguous(), 0, H * D, H * D + G * D, None, None, 1e-5, qd, kc, vc, row_req, pos, indptr, pages, n)
            if pool:
                ops.pool_blocks(kp, vp, kc, vc, pool, qo, pos, indptr, pages, n, 1)
            o = out[p0:p0 + n, :H * V]
            args = (qd, kc, vc, kp if pool else None, vp if pool else None, bias.to(F32).to(DEV), o, row_req, pos, indptr, pages, n, H,
                    window, pool, scale, cap, 1.0)
            if n > 1:
                n_tiles = (n + tile_rows - 1) // tile_rows
                tr = torch.zeros(n_tiles, dtype=I32, device=DEV)
                t0 = torch.arange(0, n, tile_rows, dtype=I32, device=DEV)
                ops.sigmoid_attn(*args, tiles=(qo, tr, t0, n_tiles, tile_rows))
                o2 = torch.zeros(n, H * V, dtype=dtype, device=DEV)
                ops.sigmoid_attn(*args[:6], o2, *args[7:])                       # the same rows one by one
                assert (o2.double() - o.double()).abs().max().item() < tol
            else:
                ops.sigmoid_attn(*args, scratch=scratch, max_keys=4096)           # keys dealt to several CTAs
                o2 = torch.zeros(n, H * V, dtype=dtype, device=DEV)
                ops.sigmoid_attn(*args[:6], o2, *args[7:])
                assert (o2.double() - o.double()).abs().max().item() < tol
            p0 += n
        got = out[:, :H * V].double().cpu().view(T, H, V)
        assert (out[:, H * V:] == 0).all()
        assert (got - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item()), cuts


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,H,G,D,V", [(F32, 10, 2, 24, 40), (BF16, 10, 2, 24, 40), (BF16, 8, 2, 32, 48), (BF16, 6, 3, 64, 128),
                                           (BF16, 3, 3, 16, 16), (BF16, 4, 1, 128, 64), (BF16, 6, 2, 32, 32), (BF16, 5, 1, 16, 32)])
def test_sigmoid_attention_far_keys_batches_and_out_scale(dtype, H, G, D, V):
    """three requests of unequal lengths in one launch (tiles and single rows), positions hundreds of keys and dozens of pages
    from their hot key, an output scale, more heads per group than a CTA takes at once; the plain kernel (float32, odd sizes)
    and the tensor-core tiles (bfloat16, head sizes in multiples of 16) with one, two and four heads per key/value head"""
    from vox_serve_b200 import ops

    torch.manual_seed(2)
    page, window, pool = 8, 50, 6
    lens = [300, 1, 77]
    seqs = []
    for n in lens:
        q, k, v = torch.randn(n, H, D, dtype=F64) * 0.05, torch.randn(n, G, D, dtype=F64) * 0.05, torch.randn(n, G, V, dtype=F64)
        k[min(3, n - 1), :, 1] = 7.0 * pool
        q[:, :, 1] = 3.0
        seqs.append(tuple(t.to(dtype).to(F64) for t in (q, k, v)))
    bias = torch.full((H,), -12.0, dtype=F64)
    indptr, pages, n_pages = _paged(lens, page, seed=5)
    kc = torch.zeros(n_pages, page, G, D, dtype=dtype, device=DEV)
    vc = torch.zeros(n_pages, page, G, V, dtype=dtype, device=DEV)
    per = (page + pool - 1) // pool
    kp, vp = torch.zeros(n_pages, per, G, D, dtype=F32, device=DEV), torch.zeros(n_pages, per, G, V, dtype=F32, device=DEV)
    T = sum(lens)
    qo, row_req, pos = _step_tables([(0, n) for n in lens])
    proj = torch.cat([torch.cat([t.reshape(n, -1) for t in s], 1) for s, n in zip(seqs, lens)], 0).to(F32).to(DEV).contiguous()
    qd = torch.zeros(T, H * D, dtype=dtype, device=DEV)
    ops.qk_norm_append(proj, 0, H * D, H * D + G * D, None, None, 1e-5, qd, kc, vc, row_req, pos, indptr, pages, T)
    ops.pool_blocks(kp, vp, kc, vc, pool, qo, pos, indptr, pages, T, 3)
    out = torch.zeros(T, H * V + 2, dtype=dtype, device=DEV)
    tile_rows = ops.window_attn_tile_rows()
    tiles = [(b, r) for b, n in enumerate(lens) if n > 1 for r in range(int(qo[b]), int(qo[b]) + n, tile_rows)]
    tr = torch.tensor([b for b, _ in tiles], dtype=I32, device=DEV)
    t0 = torch.tensor([r for _, r in tiles], dtype=I32, device=DEV)
    args = (qd, kc, vc, kp, vp, bias.to(F32).to(DEV), out[:, :H * V], row_req, pos, indptr, pages, T, H, window, pool, 0.8, 0.0, 0.6)
    ops.sigmoid_attn(*args, tiles=(qo, tr, t0, len(tiles), tile_rows))
    ops.sigmoid_attn(*args, rows=(torch.tensor([300], dtype=I32, device=DEV), 1))
    ref = torch.cat([0.6 * O.sigmoid_attend(q, k, v, bias, 0.8, 0.0, window, pool).reshape(n, -1) for (q, k, v), n in zip(seqs, lens)], 0)
    assert ref[299].abs().max() > 1e-2                       # position 299 still sees its hot key, through block 0
    tol = (1e-5 if dtype == F32 else 2e-2) * max(1.0, ref.abs().max().item())
    assert (out[:, :H * V].double().cpu() - ref).abs().max().item() < tol and (out[:, H * V:] == 0).all()
    # rows as single-token rows: all of them, and a few with their keys dealt to several CTAs
    out2 = torch.zeros(T, H * V, dtype=dtype, device=DEV)
    ops.sigmoid_attn(*args[:6], out2, *args[7:])
    assert (out2.double().cpu() - ref).abs().max().item() < tol
    few = [299, 150, 377, 300, 60]
    out3 = torch.zeros(T, H * V, dtype=dtype, device=DEV)
    ops.sigmoid_attn(*args[:6], out3, *args[7:], rows=(torch.tensor(few, dtype=I32, device=DEV), len(few)),
                     scratch=torch.zeros(1 << 22, dtype=F32, device=DEV), max_keys=4096)
    assert (out3[few].double().cpu() - ref[few]).abs().max().item() < tol and out3.abs().sum() == out3[few].abs().sum()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["rows", "tiles", "heads"])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_latent_attention_window_edges(mode, dtype):
    """softmax attention over cached rows [latent | rotated part] in a window: a key made to dominate is seen to distance
    window - 1 and by nothing further, at page borders and hundreds of positions from the sequence's start"""
    from vox_serve_b200 import ops

    torch.manual_seed(4)
    H, R, Rd, page, window, T = 4, 32, 16, 8, 13, 150
    rows = (torch.randn(T, R + Rd, dtype=F64) * 0.1).to(dtype).to(F64)
    ql = (torch.randn(T, H, R + Rd, dtype=F64) * 0.1)
    hots = [0, 39, 56, 100, 127]                     # (39: the last place of a page, 56: the first of the next)
    for hp in hots:
        rows[hp, 2] = 8.0
    ql[:, :, 2] = 6.0
    ql = ql.to(dtype).to(F64)
    ref = torch.zeros(T, H, R, dtype=F64)
    for i in range(T):
        js = O.window_keys(i, window)
        for h in range(H):
            ref[i, h] = torch.softmax(rows[js] @ ql[i, h] * 0.5, 0) @ rows[js, :R]
    indptr, pages, n_pages = _paged([T], page, seed=9)
    cache = torch.zeros(n_pages, page, 1, R + Rd, dtype=dtype, device=DEV)
    for t in range(T):
        cache[int(pages[t // page]), t % page, 0] = rows[t].to(dtype)
    qo, row_req, pos = _step_tables([(0, T)])
    out = torch.zeros(T, H * R, dtype=dtype, device=DEV)
    scratch = torch.zeros(256 * 8 * H * (R + 2), dtype=F32, device=DEV)
    q = ql.reshape(T, -1).to(dtype).to(DEV).contiguous()
    kw = dict(k_ld=R + Rd, v_ld=R + Rd)
    if mode == "tiles":
        tr_ = ops.window_attn_tile_rows()
        n_tiles = (T + tr_ - 1) // tr_
        tiles = (qo, torch.zeros(n_tiles, dtype=I32, device=DEV), torch.arange(0, T, tr_, dtype=I32, device=DEV), n_tiles)
        ops.window_attn(q, cache, cache, out, None, row_req, pos, indptr, pages, T, H, 1, R + Rd, R, window, 0.5, tiles=tiles, **kw)
    else:
        ops.window_attn(q, cache, cache, out, None, row_req, pos, indptr, pages, T, H, 1, R + Rd, R, window, 0.5, scratch=scratch,
                        head_rows=(mode == "heads"), **kw)
    got = out.double().cpu().view(T, H, R)
    assert (got - ref).abs().max().item() < (2e-5 if dtype == F32 else 4e-2)
    for hp in hots:                                          # the pattern itself: value 8 in coordinate 2 while the key is seen
        assert ref[hp + window - 1, 0, 2] > 4.0 and ref[hp + window, 0, 2] < 4.0


@pytest.mark.gpu
def test_selective_scan_slots_pieces_and_portions():
    """five requests on scattered slots that hold NaNs, cut five ways (single rows, short portions, portions over several
    tiles), sequential and piece-parallel forms, states of 1 ... 70 per channel, fp32 and bfloat16 outputs"""
    from vox_serve_b200 import ops

    tile_rows = ops.window_attn_tile_rows()
    for inner, N, seed in ((40, 5, 0), (16, 1, 1), (24, 20, 2), (50, 40, 3), (8, 70, 4), (200, 16, 5), (130, 12, 6)):
        g = torch.Generator().manual_seed(seed)
        lens = [150, 1, 37, 2, 70]
        A = -(torch.rand(inner, N, generator=g, dtype=F64) * 3 + 0.05)
        Dv = torch.randn(inner, generator=g, dtype=F64)
        dtb = torch.randn(inner, generator=g, dtype=F64) - 1.0
        data, ref = [], []
        for n in lens:
            x, dt, z = (torch.randn(n, inner, generator=g, dtype=F64) for _ in range(3))
            bc = torch.randn(n, 3 + 2 * N, generator=g, dtype=F64)
            data.append((x, dt, z, bc))
            y, _ = O.scan(x, O.softplus(dt + dtb), bc[:, 3:3 + N], bc[:, 3 + N:], A, Dv)
            ref.append(0.7 * y * O.silu(z))
        slots = torch.tensor([4, 0, 6, 2, 5], dtype=I32, device=DEV)
        dev = lambda t: t.to(F32).to(DEV).contiguous()
        for cuts, tiled in (([1000], False), ([1000], True), ([1, 1, 1, 64, 1000], True), ([3, 70, 1, 1000], True), ([65, 1000], False)):
            for out_dt in (F32, BF16):
                state = torch.full((7, inner, N), float("nan"), dtype=F32, device=DEV)
                at = [0] * len(lens)
                outs = [[] for _ in lens]
                for c in cuts:
                    live = [(b, min(c, lens[b] - at[b])) for b in range(len(lens)) if at[b] < lens[b]]
                    qo, row_req, pos = _step_tables([(at[b], n) for b, n in live])
                    T = int(qo[-1])
                    cat = lambda j: dev(torch.cat([data[b][j][at[b]:at[b] + n] for b, n in live], 0))
                    out = torch.zeros(T, inner + 2, dtype=out_dt, device=DEV)
                    sl = slots[[b for b, _ in live]].contiguous()
                    args = (cat(0), cat(1), dev(dtb), cat(3), 3, 3 + N, cat(2), dev(A), dev(Dv), state, out[:, 1:1 + inner], qo, pos, sl,
                            len(live))
                    tl = [(i, r) for i, (b, n) in enumerate(live) if n > 1 for r in range(int(qo[i]), int(qo[i]) + n, tile_rows)]
                    if tiled and tl:
                        ops.selective_scan(*args, out_scale=0.7, single_rows=True, multi_rows=False)
                        scratch = torch.full((ops.selective_scan_scratch_floats(len(tl), tile_rows, inner, N),), float("nan"),
                                             dtype=F32, device=DEV)
                        ops.selective_scan(*args, out_scale=0.7, scratch=scratch,
                                           tiles=(torch.tensor([i for i, _ in tl], dtype=I32, device=DEV),
                                                  torch.tensor([r for _, r in tl], dtype=I32, device=DEV), len(tl), tile_rows))
                    else:
                        ops.selective_scan(*args, out_scale=0.7)
                    assert (out[:, 0] == 0).all() and (out[:, -1] == 0).all()
                    for i, (b, n) in enumerate(live):
                        outs[b].append(out[int(qo[i]):int(qo[i]) + n, 1:1 + inner].double().cpu())
                        at[b] += n
                for b in range(len(lens)):
                    d = (torch.cat(outs[b], 0) - ref[b]).abs().max().item()
                    assert d < (2e-4 if out_dt == F32 else 3e-2) * max(1.0, ref[b].abs().max().item()), (inner, N, cuts, tiled, b, d)


@pytest.mark.gpu
def test_short_convolution_state_first_tokens_and_reuse():
    """taps of 1 ... 6 on strided inputs with bias, silu and the residual form; requests cut into portions of 1, 2, 3 ... tokens
    on slots that hold NaNs; the first tokens of a sequence see zeros, whatever the slot held"""
    from vox_serve_b200 import ops

    for taps, C, act, res, bias, lens in ((4, 37, "silu", False, True, [23, 1, 9]), (3, 256, None, True, False, [23, 1, 9]),
                                          (1, 5, None, False, False, [23, 1, 9]), (2, 300, "silu", True, True, [23, 1, 9]),
                                          (6, 40, None, False, True, [23, 1, 9]),
                                          # long steps: several rows per thread
                                          (4, 70, "silu", False, True, [150, 1, 67]), (3, 33, None, True, False, [90, 2, 131]),
                                          (2, 20, None, False, True, [23, 100, 9])):
        g = torch.Generator().manual_seed(taps)
        w = torch.randn(C, taps, generator=g, dtype=F64)
        bv = torch.randn(C, generator=g, dtype=F64) if bias else None
        xs = [torch.randn(n, C, generator=g, dtype=F64) for n in lens]
        ref = []
        for x in xs:
            y = O.causal_conv(x, w, bv)
            y = O.silu(y) if act else y
            ref.append(y + x if res else y)
        for cuts in ([1000], [1] * 23 + [1000], [2, 1, 3, 1000], [5, 5, 5, 1000], [1, 1000], [66, 3, 1000]):
            state = torch.full((5, max(taps - 1, 1), C), float("nan"), dtype=F32, device=DEV)
            slots = torch.tensor([3, 0, 4], dtype=I32, device=DEV)
            at, outs = [0] * 3, [[] for _ in lens]
            for c in cuts:
                live = [(b, min(c, lens[b] - at[b])) for b in range(3) if at[b] < lens[b]]
                if not live:
                    break
                qo, row_req, pos = _step_tables([(at[b], n) for b, n in live])
                T = int(qo[-1])
                wide = torch.full((T, C + 7), float("nan"), dtype=F32, device=DEV)
                wide[:, 4:4 + C] = torch.cat([xs[b][at[b]:at[b] + n] for b, n in live], 0).to(F32)
                o16 = torch.zeros(T, C, dtype=BF16, device=DEV)
                o32 = torch.zeros(T, C + 1, dtype=F32, device=DEV)
                ops.short_conv(wide[:, 4:4 + C], w.to(F32).to(DEV).contiguous(), bv.to(F32).to(DEV) if bias else None, state, qo,
                               row_req, pos, slots[[b for b, _ in live]].contiguous(), len(live), out=o16, out_f32=o32[:, :C],
                               act=act, residual=res)
                assert (o32[:, C] == 0).all()
                for i, (b, n) in enumerate(live):
                    outs[b].append((o32[int(qo[i]):int(qo[i]) + n, :C].double().cpu(), o16[int(qo[i]):int(qo[i]) + n].double().cpu()))
                    at[b] += n
            for b in range(3):
                r = ref[b]
                assert (torch.cat([a for a, _ in outs[b]], 0) - r).abs().max().item() < 1e-5 * max(1.0, r.abs().max().item()), (taps, cuts)
                assert (torch.cat([a for _, a in outs[b]], 0) - r).abs().max().item() < 1e-2 * max(1.0, r.abs().max().item())


@pytest.mark.gpu
def test_pair_hash_rows_keep_the_previous_token_per_slot():
    from vox_serve_b200 import ops

    b = {"buckets": 11, "mul_prev": 7, "mul_cur": 3}
    seqs = [_tokens(9, 50, 1), _tokens(1, 50, 2), _tokens(6, 50, 3)]
    want = [O.bigram_rows(s, b) for s in seqs]
    prev = torch.full((4,), 12345, dtype=I32, device=DEV)              # what earlier requests left in the slots
    slots = [2, 0, 3]
    at, got = [0, 0, 0], [[], [], []]
    for step in ([(0, 4), (1, 1)], [(0, 1), (2, 2)], [(2, 1)], [(0, 4), (2, 3)]):
        qo, row_req, pos = _step_tables([(at[i], n) for i, n in step])
        ids = torch.tensor(sum((seqs[i][at[i]:at[i] + n] for i, n in step), []), dtype=I32, device=DEV)
        rows = torch.zeros(ids.numel(), dtype=I32, device=DEV)
        ops.pair_hash_rows(rows, prev, ids, qo, row_req, pos, torch.tensor([slots[i] for i, _ in step], dtype=I32, device=DEV),
                           ids.numel(), 11, 7, 3)
        r = rows.tolist()
        for j, (i, n) in enumerate(step):
            got[i] += r[int(qo[j]):int(qo[j]) + n]
            at[i] += n
    assert got == want and want[0][0] == 11


@pytest.mark.gpu
@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (8, 4, 4, 3), (8, 3, 0, 0), (5, 5, 1, 1), (12, 4, 3, 1), (4, 1, 2, 1),
                                                (64, 6, 8, 3)])
def test_router_against_the_oracle(E, top, groups, keep):
    from vox_serve_b200 import ops

    torch.manual_seed(E + top)
    T, W = 50, 44
    h = (torch.randn(T, W) * 1.5).to(DEV)
    wr = torch.randn(E, W).to(DEV)
    idx = torch.zeros(T, top, dtype=I32, device=DEV)
    wts = torch.zeros(T, top, dtype=F32, device=DEV)
    ops.moe_route_groups(h, wr, top, idx, wts, groups, keep)
    s = torch.softmax(h.double().cpu() @ wr.double().cpu().T, -1)
    for t in range(T):
        want = O.route(s[t], top, groups, keep)
        assert idx[t].tolist() == want, t
        assert torch.allclose(wts[t].double().cpu(), s[t][want], rtol=1e-5, atol=1e-7)


@pytest.mark.gpu
@pytest.mark.parametrize("W,T", [(44, 19), (256, 7), (1000, 130)])
def test_output_norm_residual_value_gate_and_row_casts(W, T):
    from vox_serve_b200 import ops

    torch.manual_seed(W)
    x, y, w = torch.randn(T, W, device=DEV), torch.randn(T, W, device=DEV) * 3, torch.randn(W, device=DEV) * 0.2
    ref = x.double() + O.unit_rms(y.double(), 1e-5) * (1.0 + w.double())
    for out_dt in (F32, BF16, None):
        xx = x.clone()
        out = torch.zeros(T, W, dtype=out_dt, device=DEV) if out_dt else None
        ops.rms_postnorm_residual_f32(xx, y, (w + 1.0).contiguous(), 1e-5, out=out)
        assert (xx.double() - ref).abs().max().item() < 1e-5
        if out is not None:
            assert (out.double() - ref).abs().max().item() < (1e-5 if out_dt == F32 else 4e-2)
    wide = torch.randn(T, W + 9, device=DEV)
    for dt in (F32, BF16):
        assert torch.equal(ops.cast_rows(wide[:, 3:3 + W], torch.zeros(T, W, dtype=dt, device=DEV)), wide[:, 3:3 + W].to(dt))
    # per-head projection whose every output value has a gate of its own
    G, K, N = 3, 16, 8
    for dt in (F32, BF16):
        xs = torch.randn(T, G, K, device=DEV).to(dt)
        wg = torch.randn(G, N, K, device=DEV).to(dt)
        gate = torch.randn(T, G * N + 5, device=DEV)
        out = torch.zeros(T, G, N, dtype=dt, device=DEV)
        ops.linear_batched_gated(xs, wg, out, gate[:, 2:2 + G * N])
        ref2 = torch.einsum("tgk,gnk->tgn", xs.double(), wg.double()) * O.sigmoid(gate[:, 2:2 + G * N].double()).view(T, G, N)
        assert (out.double() - ref2).abs().max().item() < (1e-4 if dt == F32 else 8e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_clamped_experts_dense_and_grouped_forms(dtype):
    """the mixture alone (a model whose mixers contribute nothing would hide it: compare a one-layer model's stream)"""
    cfg = O.make_config(layers=("latent",), width=64, ff=64, experts=4, top=2, groups=(2, 1), limit=0.4)
    sd = O.make_weights(cfg, 31, calm=dtype == BF16)
    toks = _tokens(150, cfg["vocab"], 8)
    ref = O.forward(cfg, sd, toks)
    w = _worker(cfg, sd, dtype, pages=30)
    for min_rows in (512, 64):                  # the dense form, and (bfloat16) the experts grouped on row tiles
        w.engine.GROUPED_MIN_ROWS = min_rows
        got = _replay(w, {"a": toks}, [[("a", 150)]])["a"]
        assert (_err if dtype == F32 else _err50)(got, ref) < TOL[dtype], min_rows


# ---- serving ---------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_greedy_generation_through_scheduler(dtype):
    """ModelWorker + Scheduler: three requests of unequal prompts, prompts fed in portions of 16 beside decoding requests,
    more requests than slots.  Tokens equal the oracle's greedy tokens wherever the oracle's top-2 margin is clear."""
    from vox_serve_b200.requests import Request
    from vox_serve_b200.sampling import SamplingConfig
    from vox_serve_b200.scheduler import Scheduler

    cfg = O.make_config(layers=("latent", "pair", "shared:0-", "pair-"))
    sd = O.make_weights(cfg, 13)
    sd["embed"] = (sd["embed"].float() * 3).to(BF16)                   # clearer margins between the two best tokens
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
    margin = 0.05 if dtype == F32 else 0.8
    wrong = 0
    for rid, p in prompts.items():
        got = [int.from_bytes(c, "little", signed=True) for c in sch.audio[rid]]
        assert len(got) == n_new and reqs[rid].finish_reason == "max_tokens_reached"
        toks = list(p)
        for t in got:                       # teacher-forced comparison: every step is judged on the framework's own prefix
            z = O.forward(cfg, sd, toks)[-1]
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
    """a checkpoint directory through the trace replay tool (a subprocess: portions, two requests, a request ended and its
    slot taken again) and through the generate command (in process)."""
    import subprocess
    import sys

    import numpy as np

    from vox_serve_b200 import generate

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = O.make_config(layers=("latent", "pair", "shared:0-", "pair-"))
    sd = O.make_weights(cfg, 17)
    sd["embed"] = (sd["embed"].float() * 3).to(BF16)
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
        ra, rb, rc = (O.forward(cfg, sd, t) for t in (a, b, c))
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
                z = O.forward(cfg, sd, toks)[-1]
                top = torch.topk(z, 2)
                assert float(top.values[0] - top.values[1]) < 0.05 or t == int(top.indices[0])
                toks.append(t)
            assert len(toks) == len(prompt) + 6
