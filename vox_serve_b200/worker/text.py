"""Worker for text-only LMs on the hybrid engine (model/bobavik.py, model/razevik.py, model/fovunex.py, model/nadevik.py): the same five scheduler-facing methods, page pool,
batch slots, packed staging buffer, sampled-id ring and decode CUDA graphs as ``ModelWorker``, with three differences.

  * Prompts are fed in portions.  A request carries ``pending_tokens`` (the rest of its prompt, or continuation tokens a
    client supplies); a step takes ``step_tokens`` of them (default: ``prefill_chunk_tokens``, or all), so portions of
    prompts run in one batch beside single decoded tokens.  Positions count from 0 without gaps.
  * A request owns a state slot besides its pages: the recurrent layers keep one fp32 state per slot (``HybridCache``), and so
    do short convolutions (their last inputs) and a token-pair embedding (the last token).
    The slot index is the request's batch slot, so slot-resident sampling state and recurrent state share one pool.  Pages
    and slots go back to their pools in ``free_kv_cache`` and are handed out again without clearing: the kernels start a
    request at position 0 from a zero state, and no page is read before it is written.
  * Logits can be tapped.  ``logit_rows`` of a request selects places within its step's tokens; the step computes the
    output head for the last row of every request (what the sampler reads) plus those rows, and ``step_logits`` returns them
    in fp32.

There is no codec: ``run_detokenize`` hands each new token id to the client as 4 little-endian bytes.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from .._lib import VoxB200Error
from ..hybrid_engine import StepInputs
from ..requests import LMInputs, Request
from .base import CudaGraphWorker, I32, _Staging


class TextModelWorker(CudaGraphWorker):
    _serves_text = True
    prefill_chunk_tokens: Optional[int] = None      # portion size when a request does not name one (None: all it has)

    def _prepare_attention_wrappers(self):
        m, dev, B = self.model, self.device, self.max_batch_size
        self.max_rows = self.max_prefill_tokens + B
        self.max_logit_rows = max(getattr(self, "max_logit_rows", 0) or 0, B)
        self.cache = m.make_cache(self.max_num_pages, self.page_size, B)
        self.kv_cache = self.cache
        self.engine = m.make_engine(self.cache, self.max_rows, B + self.max_logit_rows)
        self.tile_rows = ops.window_attn_tile_rows()
        self.max_tiles = self.max_rows // self.tile_rows + B + 1
        self.staging = _Staging(B, self.max_rows, self.max_num_pages, dev,
                                extra=(("row_req", self.max_rows), ("out_rows", B + self.max_logit_rows),
                                       ("tile_req", self.max_tiles), ("tile_row0", self.max_tiles), ("single_rows", B)))
        self.free_slots = list(range(B - 1, -1, -1))
        self.slot_of: Dict[str, int] = {}
        cfg = m.default_sampling_config
        self.rep_cache = None
        if m.use_repetition_penalty and cfg.repetition_window is not None:
            W = cfg.repetition_window if cfg.repetition_window > 0 else 1
            self.rep_cache = torch.zeros(B, W, 1, m.vocab_size, dtype=torch.bool, device=dev)
        self.history_cap = 1 << max(6, int(np.ceil(np.log2(m.max_tokens + 64))))
        self.next_input = torch.zeros(B, dtype=I32, device=dev)
        self.history = torch.zeros(B, self.history_cap, dtype=I32, device=dev)
        self.n_out = torch.zeros(B, dtype=I32, device=dev)
        self.input_ids = torch.zeros(self.max_rows, dtype=I32, device=dev)
        self.out_ids = torch.zeros(B, 1, dtype=torch.int64, device=dev)
        self.sample_logits = torch.zeros(B, m.vocab_size, dtype=torch.bfloat16, device=dev)
        self.ring = [(torch.zeros(B, 1, dtype=torch.int64, pin_memory=True), torch.cuda.Event()) for _ in range(4)]
        self.ring_pos = 0
        self.decode_graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_pool = None
        self.use_cuda_graph = True
        self.gpu_launches = 0
        self._graph_nodes: Dict[int, int] = {}
        self._step_meta = (0, False, False, 0, 0)    # (logit rows, any portion, any single row, tiles, single rows) of the staged step
        self._logit_index: Dict[str, List[int]] = {}
        self.prefill_wrapper = self.decode_wrapper = None

    def capture_decode_graphs(self, batch_sizes=None) -> int:
        n = 0
        for B in (batch_sizes or range(1, self.max_batch_size + 1)):
            if B not in self.decode_graphs:
                self._capture_decode(int(B))
                n += 1
        return n

    # ---- step inputs ----------------------------------------------------------------------------------------
    def prepare_lm_inputs(self, lm_requests: List[Request], detokenize_requests: List[Request]) -> Optional[LMInputs]:
        for req in detokenize_requests:
            req.audio_decode_idx = req.next_audio_decode_idx.copy()
        if len(lm_requests) == 0:
            return None
        if len(lm_requests) > self.max_batch_size:
            raise VoxB200Error(f"{len(lm_requests)} LM requests exceed max_batch_size {self.max_batch_size}")
        st, m, ps = self.staging, self.model, self.page_size
        st.wait_consumed()
        qo, ip, slots = st.h("qo"), st.h("indptr"), st.h("slots")
        pos, ids, row_slot, indices = st.h("pos"), st.h("ids"), st.h("row_slot"), st.h("indices")
        row_req, out_rows, tile_req, tile_row0 = st.h("row_req"), st.h("out_rows"), st.h("tile_req"), st.h("tile_row0")
        single_rows = st.h("single_rows")
        # ---- what every request brings ----
        plan = []           # (request, number of rows, ids or None)
        failed: List[Request] = []
        budget = self.max_rows
        for i, req in enumerate(lm_requests):
            if req.kv_pages is None:                     # admission
                out = m.preprocess(prompt=req.prompt, audio_path=req.audio_path, **dict(req.model_kwargs))
                req.input_tokens = out.input_tokens
                req.input_length = int(out.input_tokens.shape[0])
                req.pending_tokens = out.input_tokens[:, 0].tolist() + list(req.pending_tokens or [])
                req.kv_pages, req.kv_token_len, req.kv_last_page_len, req.next_position_id = [], 0, 0, 0
                slot = self._acquire_slot(req)
                self.n_out[slot:slot + 1].zero_()
                if self.rep_cache is not None:
                    self.rep_cache[slot].zero_()
            if req.pending_tokens:
                n = req.step_tokens or self.prefill_chunk_tokens or len(req.pending_tokens)
                n = min(n, len(req.pending_tokens), self.max_prefill_tokens)
                toks = req.pending_tokens[:n]
            else:
                n, toks = 1, None
            others = len(lm_requests) - i - 1
            why = None
            if n > budget - others:
                n = budget - others                       # a smaller portion now, the rest in a later step
                toks = toks[:n] if toks is not None else None
                if n <= 0:
                    why = "error: no room in the step"
            need = (req.kv_token_len + n + ps - 1) // ps - len(req.kv_pages) if why is None else 0
            if why is None and need > self.empty_pages.qsize():
                why = f"error: out of KV pages ({need} needed, {self.empty_pages.qsize()} free)"
            if why is not None:
                self._fail_request(req, why)
                failed.append(req)
                continue
            for _ in range(need):
                req.kv_pages.append(self.empty_pages.get_nowait())
            plan.append((req, n, toks))
            budget -= n
        if failed:
            lm_requests[:] = [r for r in lm_requests if r not in failed]
            if not lm_requests:
                return None
        # ---- the packed tables ----
        B = len(plan)
        t = npg = n_tiles = n_single = 0
        extra = B                     # logit rows: the last row of every request first, tapped rows after them
        qo[0] = ip[0] = 0
        any_multi = any_single = False
        self._logit_index = {}
        for b, (req, n, toks) in enumerate(plan):
            slot = self.slot_of[req.request_id]
            p0 = req.kv_token_len
            pos[t:t + n] = np.arange(p0, p0 + n, dtype=np.int32)
            row_req[t:t + n] = b
            if toks is not None:
                ids[t:t + n] = toks
                row_slot[t:t + n] = -1
                del req.pending_tokens[:n]
            else:
                ids[t] = 0
                row_slot[t] = slot                        # the slot's last sampled token (build_input_ids)
            if n > 1:
                any_multi = True
                for r0 in range(0, n, self.tile_rows):
                    tile_req[n_tiles], tile_row0[n_tiles] = b, t + r0
                    n_tiles += 1
            else:
                any_single = True
                single_rows[n_single] = t
                n_single += 1
            out_rows[b] = t + n - 1
            idx = []
            for r in (req.logit_rows or []):
                if not 0 <= r < n:
                    raise VoxB200Error(f"logit row {r} outside the step's {n} tokens")
                if r == n - 1:
                    idx.append(b)
                else:
                    if extra >= B + self.max_logit_rows:
                        raise VoxB200Error(f"more than {self.max_logit_rows} tapped logit rows in one step")
                    out_rows[extra] = t + r
                    idx.append(extra)
                    extra += 1
            if req.logit_rows is not None:
                self._logit_index[req.request_id] = idx
            req.logit_rows = req.step_tokens = None
            req.kv_token_len = p0 + n
            req.kv_last_page_len = req.kv_token_len % ps or ps
            req.next_position_id = req.kv_token_len
            req.done_lm_prefill = not req.pending_tokens
            k = len(req.kv_pages)
            indices[npg:npg + k] = req.kv_pages
            npg += k
            t += n
            qo[b + 1], ip[b + 1], slots[b] = t, npg, slot
        self._step_meta = (extra, any_multi, any_single, n_tiles, n_single)
        lm_inputs = {"qo_indptr": qo[:B + 1].tolist(), "paged_kv_indptr": ip[:B + 1].tolist(),
                     "paged_kv_indices": indices[:npg].tolist(),
                     "paged_kv_last_page_len": [r.kv_last_page_len for r, _, _ in plan],
                     "input_ids": self.input_ids[:t].view(t, 1), "position_ids": st.d("pos", t), "input_features": None,
                     "input_masks": None, "repetition_cache": self.rep_cache, "is_prefill": any_multi, "n_rows": t,
                     "n_pages": npg}
        if self.early_launch:
            lm_inputs["_launched"] = self._launch_step(B, t, any_multi)
        return lm_inputs

    # ---- the step on the device -------------------------------------------------------------------------------
    def _device_step(self, B: int, T: int, is_prefill: bool):
        st, m = self.staging, self.model
        if is_prefill:
            n_out, multi, single, n_tiles, n_single = self._step_meta
        else:                                            # (also what a decode graph captures: one row per request)
            n_out, multi, single, n_tiles, n_single = B, False, True, 0, 0
        ops.build_input_ids(self.input_ids, st.d("ids"), self.next_input, st.d("row_slot"), T)
        step = StepInputs(ids=self.input_ids[:T], pos=st.d("pos", T), row_req=st.d("row_req", T), qo_indptr=st.d("qo", B + 1),
                          page_indptr=st.d("indptr", B + 1), page_indices=st.d("indices"), slots=st.d("slots", B),
                          out_rows=st.d("out_rows", n_out), B=B, T=T, n_out=n_out, multi=multi, single=single,
                          tiles=(st.d("tile_req"), st.d("tile_row0"), n_tiles) if n_tiles else None,
                          single_rows=(st.d("single_rows"), n_single) if (n_tiles and n_single) else None)
        logits = m.forward(step, engine=self.engine)
        slots = st.d("slots", B)
        out = self.out_ids[:B]
        sl = ops.cast_f32_bf16(logits[:B], self.sample_logits[:B])
        m.sampling_device(sl.view(B, 1, -1), None, self.rep_cache,
                          cache_rows=slots if self.rep_cache is not None else None, out=out.view(-1))
        ops.token_feedback(out.view(-1), slots, self.next_input, self.history, self.n_out, skip_token=m.stop_token_id)

    def step_logits(self, request_id: str) -> torch.Tensor:
        """fp32 [tapped rows, vocab] of the request's ``logit_rows`` in the step that ran last (host tensor)."""
        idx = self._logit_index[request_id]
        buf = self.engine.logits          # (the static buffer, not a step's view of it: decode graphs replay without one)
        if any(not 0 <= i < buf.shape[0] for i in idx):
            raise VoxB200Error("logit row outside the engine's buffer")
        sel = torch.as_tensor(idx, dtype=torch.int64, device=buf.device)
        return buf.index_select(0, sel).cpu()

    # ---- tokens out ---------------------------------------------------------------------------------------------
    def run_detokenize(self, requests: List[Request]):
        for req in requests:
            for d in req.audio_decode_idx:
                if d < len(req.lm_output_audio_tokens):
                    req.output_audio.put(int(req.lm_output_audio_tokens[d][0, 0]).to_bytes(4, "little", signed=True))
            if req.done_lm_generation and req.audio_decode_idx and \
                    req.audio_decode_idx[-1] + 1 >= len(req.lm_output_audio_tokens):
                req.done_all = True

    def run_lm_decode_resident(self, *a, **k):
        raise VoxB200Error("resident multi-step decode is a speech-path loop (it interleaves vocoder passes)")
