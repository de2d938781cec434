"""Command line for the text-only LMs: generate continuations of token-id prompts through ModelWorker + Scheduler.

    python -m vox_serve_b200.generate --model DIR --prompt "5 17 3" [--prompt "8 9"] [--max-new 32]
                                      [--dtype bfloat16|float32] [--prefill-chunk 256] [--temperature T --top-p P --top-k K]

``DIR`` holds ``config.json`` + ``model.safetensors``; the model class is chosen by the configuration's ``architecture``.
Prompts are token ids separated by blanks (these models ship no tokenizer).  Every prompt is one request; they run as one
continuous batch, prompts in portions of ``--prefill-chunk`` tokens beside the decoding requests.  Output: one line of
generated ids per prompt, in the order given.
"""
from __future__ import annotations

import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt", action="append", required=True, help="token ids separated by blanks; may be repeated")
    ap.add_argument("--max-new", type=int, default=32)
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--prefill-chunk", type=int, default=256)
    ap.add_argument("--max-batch-size", type=int, default=8)
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=None)
    ap.add_argument("--top-p", type=float, default=None)
    ap.add_argument("--top-k", type=int, default=None)
    a = ap.parse_args(argv)

    import torch

    from . import _lib
    from .model import build_profile

    _lib.load(build_if_missing=True, profile=build_profile(a.model))
    from .requests import Request
    from .sampling import SamplingConfig
    from .scheduler import Scheduler
    from .worker import ModelWorker

    prompts = [[int(t) for t in p.split()] for p in a.prompt]
    need = sum((len(p) + a.max_new + a.page_size) // a.page_size + 1 for p in prompts)
    greedy = a.temperature is None and a.top_p is None and a.top_k is None
    worker = ModelWorker(a.model, max_batch_size=min(a.max_batch_size, max(1, len(prompts))), max_num_pages=need,
                         page_size=a.page_size, max_prefill_tokens=max(a.prefill_chunk, 64), dtype=getattr(torch, a.dtype),
                         temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, greedy=greedy)
    if not getattr(worker.model, "is_text_model", False):
        print("this command serves text-only models", file=sys.stderr)
        return 2
    sch = Scheduler(worker, prefill_chunk_tokens=a.prefill_chunk)
    cfg = worker.model.default_sampling_config
    for i, p in enumerate(prompts):
        sc = SamplingConfig(top_p=cfg.top_p, top_k=cfg.top_k, min_p=cfg.min_p, temperature=cfg.temperature,
                            max_tokens=a.max_new, greedy=cfg.greedy)
        sch.submit(Request(request_id=f"p{i}", prompt=p, sampling_config=sc))
    sch.run_until_done()
    for i in range(len(prompts)):
        print(" ".join(str(int.from_bytes(c, "little", signed=True)) for c in sch.audio[f"p{i}"]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
