"""Run token-ID workloads or a local Llama checkpoint:  python -m cisr_b200 ...

Parity: runtime/__main__.py:11-51.  Option names and meanings follow the reference
where it has them: --dtype, --execution, --checkpoint, --prompt, --tokens,
--max-new-tokens, --requests, --policy, --pages, --page-size, --token-budget,
--prefill-chunk; the printed JSON has the same fields (device, dtype, weights,
requests[key, status, generated, text, ttft_ms]).  Differences: --device accepts only
cuda (there is no CPU path); --dtype has no float16; without --checkpoint the model is
a named shape with seeded random weights (--config, --seed) instead of one fixed toy;
--temperature, --max-active and --reserve are added; several EOS ids are accepted.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def build_parser() -> argparse.ArgumentParser:
    from .config.presets import preset_names

    parser = argparse.ArgumentParser(prog="python -m cisr_b200", description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--device", choices=["cuda"], default="cuda", help="only cuda: the engine has no CPU path")
    parser.add_argument("--dtype", choices=["float32", "bfloat16"], default="bfloat16",
                        help="bfloat16: serving precision; float32: every product and sum in true 32-bit")
    parser.add_argument("--execution", choices=["eager", "buffered", "graph"], default="eager",
                        help="graph replays decode steps from a captured CUDA graph; eager and buffered launch kernels directly")
    parser.add_argument("--checkpoint", type=Path, help="folder with config.json, safetensors and tokenizer.json")
    parser.add_argument("--config", default="tiny-a", choices=preset_names(),
                        help="named shape used with random weights when no --checkpoint is given")
    parser.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    parser.add_argument("--prompt", default="The capital of France is")
    parser.add_argument("--tokens", default="1,2,3", help="token IDs of the prompt when no --checkpoint is given")
    parser.add_argument("--max-new-tokens", type=int, default=16)
    parser.add_argument("--temperature", type=float, default=0.0, help="0 selects greedily")
    parser.add_argument("--requests", type=Path, help="JSON list: key, prompt (IDs), max_new_tokens, arrival_s")
    parser.add_argument("--policy", choices=["serial", "chunked", "decode_first"], default="decode_first")
    parser.add_argument("--reserve", choices=["full", "lazy"], default="full",
                        help="full: admit only what can never run out of pages; lazy: admit by prompt, preempt and recompute when pages run out")
    parser.add_argument("--pages", type=int, default=128)
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--token-budget", type=int, default=32)
    parser.add_argument("--prefill-chunk", type=int, default=8)
    parser.add_argument("--max-active", type=int, default=8)
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    from . import Engine, Model, Request

    tokenizer = None
    raw = {}
    if args.checkpoint:
        from tokenizers import Tokenizer

        model = Model.from_pretrained(args.checkpoint, dtype=args.dtype)
        raw = model.config
        tokenizer = Tokenizer.from_file(str(args.checkpoint / "tokenizer.json"))
        prompt = tokenizer.encode(args.prompt).ids
    else:
        model = Model.from_config(args.config, seed=args.seed, dtype=args.dtype)
        raw = model.config
        prompt = [int(t) for t in args.tokens.split(",")]
    engine = Engine.for_model(model, pages=args.pages, page_size=args.page_size, max_active=args.max_active,
                              token_budget=args.token_budget, prefill_chunk=args.prefill_chunk, policy=args.policy,
                              reserve=args.reserve, graph=args.execution == "graph")
    inputs = json.loads(args.requests.read_text()) if args.requests else [
        {"key": "request-0", "prompt": prompt, "max_new_tokens": args.max_new_tokens}]
    for item in inputs:
        defaults = {"eos_token_id": raw.get("eos_token_id"), "temperature": args.temperature, "seed": args.seed}
        engine.submit(Request(**(defaults | item)))
    result = []
    for r in engine.run():
        result.append({"key": r.key, "status": r.status, "generated": r.generated,
                       "text": tokenizer.decode(r.generated) if tokenizer else None,
                       "ttft_ms": None if r.first_token_at is None else (r.first_token_at - r.submitted_at) * 1000})
    print(json.dumps({"device": args.device, "dtype": args.dtype,
                      "weights": "pretrained-local" if tokenizer else "random-" + args.config,
                      "requests": result}, indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
