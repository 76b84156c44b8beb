#!/usr/bin/env python
"""Generate text from a checkpoint (same flags as the reference's generate.py:264-326)."""
import argparse
import sys

import torch

from gruboros_b200.runtime.generation import generate, load_model, load_primer_text, decode_tokens
from gruboros_b200.utils.sizes import parse_size_with_suffix


def main(argv=None):
    p = argparse.ArgumentParser(description="Generate text with a trained minLM")
    p.add_argument("--model", type=str, required=True, help="checkpoint file or directory")
    p.add_argument("--device", type=str, default="auto")
    p.add_argument("--cpu", action="store_true")
    p.add_argument("--use-f32", dest="use_f32", action="store_true")
    p.add_argument("--use-fp16", dest="use_fp16", action="store_true")
    p.add_argument("--generation_length", type=str, default="512")
    p.add_argument("--temperature", type=float, default=0.85)
    p.add_argument("--top_p", type=float, default=0.9)
    p.add_argument("--top_k", type=int, default=0)
    p.add_argument("--primer_file", type=str, default=None)
    p.add_argument("--primer_text", type=str, default=None)
    p.add_argument("--primer_length", type=str, default="1k")
    p.add_argument("--force_primer_length", action="store_true")
    p.add_argument("--output_file", type=str, default=None)
    p.add_argument("--no-stream", dest="stream", action="store_false", default=True)
    a = p.parse_args(argv)
    device = "cpu" if a.cpu else a.device
    model, cfg = load_model(a.model, device=device, use_fp16=a.use_fp16, use_f32=a.use_f32)
    device = next(model.parameters()).device
    primer = load_primer_text(a.primer_file, int(parse_size_with_suffix(a.primer_length)), a.primer_text,
                              explicit_length=a.force_primer_length)
    toks = generate(model, primer, int(parse_size_with_suffix(a.generation_length)), a.temperature, a.top_k, a.top_p,
                    device=device, stream=a.stream)
    text = decode_tokens(toks[0].tolist())
    if not a.stream:
        print(text)
    if a.output_file:
        with open(a.output_file, "w", encoding="utf-8") as f:
            f.write(decode_tokens(primer[0].tolist()) + text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
