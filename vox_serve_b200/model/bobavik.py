"""Bobavik adapter: a text-only decoder-only LM whose layers alternate sliding-window softmax attention (grouped heads,
partial interleaved rotary with wavelength-dependent frequency scaling, cross-layer value mixing, sigmoid output gate) and
lightning attention (per-head decay, recurrent fp32 state), each followed by a mixture-of-experts feed-forward with a
shared expert, with LayerNorm before and after every sublayer around an fp32 residual stream.  Everything a model of this
design can vary (sizes, head counts, layer order, windows, decays, rotary constants, expert counts) is read from its
``config.json``; the arithmetic runs on ``HybridEngine`` (hybrid_engine.py).

The adapter has the same interface as the speech adapters (``BaseLM``) with ``is_text_model`` set: there is no audio
codec, "detokenizing" a token means handing its id to the client, and the worker that serves it (worker/text.py) keeps a
state slot per request next to the KV pages.

Weights: a directory with ``config.json`` + ``model.safetensors`` (bf16 matrices; read without third-party packages), an
explicit ``state_dict=`` + ``config=``, or ``model_name="bobavik-synthetic[:seed]"`` with ``config=`` (seeded random
weights of that configuration, for benchmarks and tests).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .. import ops
from .._lib import VoxB200Error
from ..hybrid_engine import HybridCache, HybridConfig, HybridEngine, HybridWeights, StepInputs
from ..requests import Request
from ..sampling import Sampler, SamplingConfig
from .base import BaseLM, PreprocessOutput

_ST_DTYPES = {"BF16": (np.uint16, torch.bfloat16), "F16": (np.float16, torch.float16), "F32": (np.float32, torch.float32),
              "F64": (np.float64, torch.float64), "I32": (np.int32, torch.int32), "I64": (np.int64, torch.int64)}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """A safetensors file: 8-byte little-endian header length, that many bytes of JSON (name -> dtype, shape,
    data_offsets), then the raw little-endian data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))
        data = np.frombuffer(f.read(), dtype=np.uint8)
    out: Dict[str, torch.Tensor] = {}
    for name, m in meta.items():
        if name == "__metadata__":
            continue
        if m["dtype"] not in _ST_DTYPES:
            raise VoxB200Error(f"{path}: tensor {name} has unsupported dtype {m['dtype']}")
        npdt, tdt = _ST_DTYPES[m["dtype"]]
        a, b = m["data_offsets"]
        arr = data[a:b].view(npdt).copy()
        t = torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16) if tdt == torch.bfloat16 else torch.from_numpy(arr)
        out[name] = t.reshape(m["shape"])
    return out


def synthetic_state_dict(cfg: HybridConfig, seed: int = 0, device="cpu") -> Dict[str, torch.Tensor]:
    """Seeded random weights with the checkpoint's names (bf16 matrices), generated on ``device``."""
    g = torch.Generator(device=device).manual_seed(seed)
    W = cfg.width

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g, device=device) * std + mean).to(torch.bfloat16)

    sd = {"embed": rnd(cfg.vocab, W), "head": rnd(cfg.vocab, W, std=W ** -0.5), "final.norm": rnd(W, std=0.1, mean=1.0),
          "final.norm.b": rnd(W, std=0.1)}
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        for nm in ("norm1", "norm1b") + (("norm2", "norm2b") if L.mlp else ()):
            sd[p + nm], sd[p + nm + ".b"] = rnd(W, std=0.1, mean=1.0), rnd(W, std=0.1)
        s = W ** -0.5
        if L.kind == "attention":
            sd[p + "mix.q"], sd[p + "mix.k"] = rnd(m.heads * m.dim, W, std=s), rnd(m.kv_heads * m.dim, W, std=s)
            sd[p + "mix.v"], sd[p + "mix.g"] = rnd(m.kv_heads * m.vdim, W, std=s), rnd(m.heads * m.vdim, W, std=s)
            sd[p + "mix.o"] = rnd(W, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
            if m.v_mix:
                sd[p + "mix.vmix"] = torch.rand((), generator=g, device=device).to(torch.bfloat16)
        else:
            sd[p + "mix.q"], sd[p + "mix.k"] = rnd(m.heads * m.dim, W, std=s), rnd(m.heads * m.dim, W, std=s)
            sd[p + "mix.v"], sd[p + "mix.g"] = rnd(m.heads * m.vdim, W, std=s), rnd(m.heads * m.vdim, W, std=s)
            sd[p + "mix.o"] = rnd(W, m.heads * m.vdim, std=(m.heads * m.vdim) ** -0.5)
            sd[p + "mix.norm"] = rnd(m.heads * m.vdim, std=0.1, mean=1.0)
        if L.mlp:
            f = L.mlp
            sd[p + "mlp.router"], sd[p + "mlp.router.b"] = rnd(f.experts, W, std=s), rnd(f.experts, std=0.1)
            names = [f"e{e}" for e in range(f.experts)] + (["shared"] if f.shared_ff else [])
            for nm in names:
                ff = f.shared_ff if nm == "shared" else f.ff
                sd[p + f"mlp.{nm}.gate"], sd[p + f"mlp.{nm}.up"] = rnd(ff, W, std=s), rnd(ff, W, std=s)
                sd[p + f"mlp.{nm}.down"] = rnd(W, ff, std=ff ** -0.5)
    return sd


class BobavikModel(BaseLM):
    is_text_model = True
    has_recurrent_state = True
    design = "Bobavik"
    synthetic_name = "bobavik-synthetic"
    build_profile = "text"          # the subset of the CUDA sources (build.PROFILES) a first run of this design compiles

    # what a design built on the hybrid engine supplies: its configuration reader and its seeded random weights
    @staticmethod
    def read_config(config: Dict[str, Any]) -> HybridConfig:
        return HybridConfig.from_json(config)

    @staticmethod
    def synthetic_weights(cfg: HybridConfig, seed: int, device) -> Dict[str, torch.Tensor]:
        return synthetic_state_dict(cfg, seed, device)

    def __init__(self, model_name: str, dtype: torch.dtype = torch.bfloat16, device: str = "cuda:0",
                 enable_torch_compile: bool = False, audio_decoder_device: Optional[str] = None,
                 state_dict: Optional[Dict[str, torch.Tensor]] = None, config: Optional[Dict[str, Any]] = None,
                 max_tokens: Optional[int] = None, stop_token_id: Optional[int] = None,
                 tensor_core_projections: bool = True, **_unused):
        if dtype not in (torch.bfloat16, torch.float32):
            raise VoxB200Error(f"{self.design} runs in bfloat16 or float32, not {dtype}")
        super().__init__(model_name, device, dtype, enable_torch_compile, audio_decoder_device)
        if not torch.cuda.is_available():
            raise VoxB200Error(f"{type(self).__name__} needs a CUDA device: there is no CPU path")
        if state_dict is None:
            if os.path.isdir(model_name):
                with open(os.path.join(model_name, "config.json")) as f:
                    config = json.load(f)
                state_dict = read_safetensors(os.path.join(model_name, "model.safetensors"))
            elif model_name.startswith(self.synthetic_name) and config is not None:
                seed = int(model_name.split(":")[1]) if ":" in model_name else 0
                cfg = self.read_config(config) if isinstance(config, dict) else config
                state_dict = self.synthetic_weights(cfg, seed, device)
            else:
                raise VoxB200Error(f"'{model_name}': pass a directory with config.json + model.safetensors, "
                                   f"state_dict= and config=, or '{self.synthetic_name}[:seed]' with config=")
        if config is None:
            raise VoxB200Error(f"{type(self).__name__} needs its configuration (config=)")
        self.config = self.read_config(config) if isinstance(config, dict) else config
        self.weights = HybridWeights(state_dict, self.config, dtype, device, tensor_core=tensor_core_projections)
        self._max_tokens = max_tokens or 4096
        self.stop_token_id = -1 if stop_token_id is None else stop_token_id
        self.default_sampling_config = SamplingConfig(greedy=True)
        seed64 = torch.cuda.default_generators[torch.device(device).index or 0].initial_seed() & ((1 << 63) - 1)
        self.rng_state = torch.tensor([seed64, 0, 0], dtype=torch.int64, device=device)

    # ---- static facts -------------------------------------------------------------------------------------
    n_codebooks = 1
    detokenize_interval = 1
    detokenize_overlap = 0
    n_channels = 1
    output_audio_length = 0

    def _first_attention(self):
        return next((L.mixer for L in self.config.layers if L.kind in ("attention", "latent")), None)

    @property
    def num_attention_heads(self) -> int:
        m = self._first_attention()
        return m.heads if m else 0

    @property
    def num_key_value_heads(self) -> int:
        m = self._first_attention()
        return getattr(m, "kv_heads", 1) if m else 0

    @property
    def num_hidden_layers(self) -> int:
        return len(self.config.layers)

    @property
    def hidden_size(self) -> int:
        return self.config.width

    @property
    def head_dim(self) -> int:
        m = self._first_attention()
        return m.dim if m else 0

    @property
    def vocab_size(self) -> int:
        return self.config.vocab

    @property
    def max_tokens(self) -> int:
        return self._max_tokens

    @property
    def max_positions(self) -> int:
        """The longest sequence (prompt + generated) the design can address: the rows of a learned position table."""
        return self.config.positions or (1 << 30)

    def is_stop_id(self, token_ids: List[int]) -> bool:
        return self.stop_token_id >= 0 and token_ids[0] == self.stop_token_id

    # ---- caches and engine --------------------------------------------------------------------------------
    def make_cache(self, num_pages: int, page_size: int, num_slots: int) -> HybridCache:
        return HybridCache(self.config, num_pages, page_size, num_slots, self.dtype, self.device)

    def make_engine(self, cache: HybridCache, max_rows: int, max_out_rows: int) -> HybridEngine:
        return HybridEngine(self.weights, cache, max_rows, max_out_rows)

    # ---- per-step work ------------------------------------------------------------------------------------
    def preprocess(self, prompt=None, audio_path: str = None, **kwargs) -> PreprocessOutput:
        """prompt: token ids (a list / tensor of ints, or a string of ids separated by blanks) -- the design has no
        tokenizer of its own."""
        if isinstance(prompt, str):
            prompt = [int(t) for t in prompt.split()]
        ids = torch.as_tensor(prompt, dtype=torch.int64).reshape(-1, 1)
        if ids.numel() == 0:
            raise VoxB200Error("empty prompt")
        if int(ids.min()) < 0 or int(ids.max()) >= self.config.vocab:
            raise VoxB200Error(f"token id outside [0, {self.config.vocab})")
        if ids.numel() > self.max_positions:
            raise VoxB200Error(f"prompt of {ids.numel()} tokens exceeds the model's {self.max_positions} positions")
        return PreprocessOutput(input_tokens=ids)

    def forward(self, step: StepInputs, engine: HybridEngine = None, **kwargs) -> torch.Tensor:
        """logits fp32 [n_out, vocab] of the step's ``out_rows``."""
        return engine.forward(step)

    def sampling_device(self, logits: torch.Tensor, sampling_params: Optional[SamplingConfig] = None,
                        repetition_cache: Optional[torch.Tensor] = None, cache_rows: Optional[torch.Tensor] = None,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits bf16 [B, 1, V] -> ids int64 [B, 1] through the framework's fused sampler."""
        cfg = sampling_params or self.default_sampling_config
        ids = Sampler.sample_fused(logits, cfg, repetition_cache, cache_rows=cache_rows, rng_state=self.rng_state, out=out)
        if repetition_cache is not None:
            Sampler.update_repetition_penalty_cache(repetition_cache, ids, cfg.repetition_window, cache_rows=cache_rows)
        return ids

    def sampling_host(self, output_ids: torch.Tensor, requests: List[Request],
                      repetition_cache: Optional[torch.Tensor] = None, ids_host=None, ready=None,
                      cache_rows_host: Optional[List[int]] = None):
        """The request-state coroutine of a step.  A request that is still in the middle of its prompt (or whose next token
        is given) takes no sampled token."""
        takes = [not r.pending_tokens for r in requests]
        stop_id, max_tokens, max_pos = self.stop_token_id, self.max_tokens, self.max_positions

        async def update_req_states():
            if ids_host is not None:
                ready.synchronize()
                host = ids_host[:len(requests)].clone()
            else:
                host = output_ids.to("cpu")
            col0 = host[:, 0].tolist()
            for i, req in enumerate(requests):
                if not takes[i]:
                    continue
                tok = host[i:i + 1]
                req.input_tokens = tok
                req.lm_output_tokens.append(tok)
                req.lm_output_audio_tokens.append(tok)
                if col0[i] == stop_id:
                    req.lm_output_audio_tokens.pop()
                    req.done_lm_generation, req.finish_reason = True, "stop_id_encountered"
                elif len(req.lm_output_tokens) >= (req.sampling_config.max_tokens if req.sampling_config and
                                                   req.sampling_config.max_tokens else max_tokens):
                    req.done_lm_generation, req.finish_reason = True, "max_tokens_reached"
                elif (req.next_position_id or 0) >= max_pos:
                    req.done_lm_generation, req.finish_reason = True, "max_positions_reached"

        return update_req_states()

    def sampling(self, logits: torch.Tensor, requests: List[Request], sampling_params: Optional[SamplingConfig] = None,
                 repetition_cache: Optional[torch.Tensor] = None, cfg_scale: Optional[float] = None, **kwargs):
        output_ids = self.sampling_device(logits, sampling_params, repetition_cache)
        return output_ids, self.sampling_host(output_ids, requests, repetition_cache)

    def postprocess(self, token_ids: torch.Tensor, **kwargs) -> torch.Tensor:
        return token_ids
