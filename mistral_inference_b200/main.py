"""Command line: `python -m mistral_inference_b200.main generate MODEL_DIR --prompt "5 17 3" [--prompt ...] --max-tokens N`.

Loads any model folder through the registry (reference-format `params.json` checkpoints and `config.json` designs alike) and
runs `generate()` on prompts given as token ids (no tokenizer ships with these checkpoints; the reference's `mistral-demo`,
main.py:163-196, does the same job after tokenising).  Prints one line of generated ids per prompt.
"""
import argparse
import sys
from typing import List, Optional


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="mistral_inference_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="greedy or nucleus generation from prompts of token ids")
    g.add_argument("model")
    g.add_argument("--prompt", action="append", required=True, help="token ids separated by spaces; repeat for a batch")
    g.add_argument("--max-tokens", type=int, default=32)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--chunk-size", type=int, default=None)
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default=None)
    a = ap.parse_args(argv)

    import torch

    from .generate import generate
    from .registry import load_model

    prompts = [[int(t) for t in p.split()] for p in a.prompt]
    model = load_model(a.model, max_batch_size=len(prompts), dtype=getattr(torch, a.dtype) if a.dtype else None)
    tokens, _ = generate(prompts, model, max_tokens=a.max_tokens, temperature=a.temperature, chunk_size=a.chunk_size)
    for row in tokens:
        print(" ".join(str(t) for t in row))
    return 0


if __name__ == "__main__":
    sys.exit(main())
