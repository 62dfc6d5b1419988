"""Command line of the package.

    python -m proxy_inference_engine_b200 generate --model DIR --prompt-ids 5,17,3 [--prompt-ids ...] --max-new-tokens 32
                                                   [--dtype bfloat16|float32] [--temp T --top-p P --top-k K --seed S]
    python -m proxy_inference_engine_b200 trace    --model DIR --dtype ... --out DIR --max-tokens N      (= bin/trace_run)
    python -m proxy_inference_engine_b200 models                                                         (registry)

``generate`` loads the checkpoint by the model type its config.json names (checkpoint.MODEL_REGISTRY) and continues the
prompts -- token ids; tokenisation and chat templating stay with the caller, as on the reference's model surface
(PIE/engine/inference_engine.py:228-297 receives ids too).  One JSON line per prompt is printed."""
from __future__ import annotations

import argparse
import json
import os
import sys


def _generate(a) -> int:
    import torch

    from .checkpoint import load_model, model_kind
    from .samplers import make_sampler
    with open(os.path.join(a.model, "config.json")) as f:
        kind = model_kind(json.load(f))
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    sampler = make_sampler(a.temp, a.top_p, 0.0, 1, a.top_k, seed=a.seed) if a.temp > 0 else None
    if kind == "llama":
        from .decode import DecodeEngine
        model = load_model(a.model)
        outs = []
        for p in prompts:   # the graph-replayed decode engine runs rows of equal length: one prompt at a time
            eng = DecodeEngine(model, batch=1, max_context=len(p) + a.max_new_tokens + 1,
                               sampling=dict(temp=a.temp, top_p=a.top_p, top_k=a.top_k, seed=a.seed) if a.temp > 0 else None)
            outs.append(eng.generate(torch.tensor([p]), a.max_new_tokens)[0].tolist())
    else:
        from .engine import HybridEngine
        model = load_model(a.model, dtype=a.dtype)
        need = sum((len(p) + a.max_new_tokens + 63) // 64 * 64 for p in prompts[: a.max_seqs]) + 64
        eng = HybridEngine(model, max_tokens=max(a.max_tokens or 0, need), max_seqs=a.max_seqs)
        outs = eng.generate(prompts, a.max_new_tokens, sampler=sampler)
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt_ids": p, "generated_ids": o}), flush=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="proxy_inference_engine_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="continue prompts given as token ids")
    g.add_argument("--model", required=True)
    g.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for more prompts")
    g.add_argument("--max-new-tokens", type=int, default=32)
    g.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    g.add_argument("--temp", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--seed", type=int, default=0)
    g.add_argument("--max-seqs", type=int, default=4, help="sequences live at once (hybrid models)")
    g.add_argument("--max-tokens", type=int, default=0, help="tokens the page pool holds (hybrid models; 0: from the prompts)")
    sub.add_parser("trace", help="replay a recorded schedule (see bin/trace_run)", add_help=False)
    sub.add_parser("models", help="list the model types the registry knows")
    if argv is None:
        argv = sys.argv[1:]
    if argv and argv[0] == "trace":
        from .trace import main as trace_main
        return trace_main(argv[1:])
    a = ap.parse_args(argv)
    if a.cmd == "models":
        from .checkpoint import MODEL_REGISTRY
        print("\n".join(sorted(MODEL_REGISTRY)))
        return 0
    return _generate(a)


if __name__ == "__main__":
    sys.exit(main())
