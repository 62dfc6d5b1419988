"""Trace replay: feed recorded token ids through a model step by step and write the logits that are asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   < steps.jsonl

Each input line is one step, ``{"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [...]}``: all
entries run as ONE ragged batch through ``engine.HybridEngine.forward`` (the step the generate loop uses), sequences are
admitted at their first entry and give their pages and state slot back when named in ``end``.  For a step with wanted
rows the logits go to ``<out>/<n>.f32`` (little-endian fp32 [wanted, vocab], entry order); after every step the line
``done <n>`` is printed.  Nothing is sampled.  Exit code 3: the model's family has no float32 mode."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model*.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True, help="folder the logits files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="tokens the live sequences hold at most (each rounded up to whole 64-token pages)")
    ap.add_argument("--max-seqs", type=int, default=4, help="state slots = sequences live at once")
    a = ap.parse_args(argv)

    with open(os.path.join(a.model, "config.json")) as f:
        config = json.load(f)
    from .checkpoint import load_model, model_kind
    kind = model_kind(config)
    if kind == "llama":
        if a.dtype == "float32":
            print("the quantized Llama path runs in bfloat16 only", file=sys.stderr)
            return 3
        print("trace replay is built for the models that step over a HybridCache", file=sys.stderr)
        return 2
    import torch
    from .engine import HybridEngine

    if not torch.cuda.is_available():
        print("trace_run needs a CUDA device (there is no CPU path)", file=sys.stderr)
        return 2
    model = load_model(a.model, device="cuda", dtype=a.dtype)
    eng = HybridEngine(model, max_tokens=a.max_tokens, max_seqs=a.max_seqs, use_graph=False)   # a replay is not a hot loop
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in step.get("entries", [])]
        if entries:
            logits = eng.forward(entries)
            if logits.shape[0]:
                data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4")
                tmp = os.path.join(a.out, f".{step['step']}.f32.part")
                with open(tmp, "wb") as f:
                    f.write(data.tobytes())
                os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
            else:
                torch.cuda.synchronize()
        for sid in step.get("end", []):
            if sid in eng.cache.seqs:
                eng.finish(sid)
        print(f"done {step['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
