"""Decode throughput: tokens/s of step-by-step generation for a random-init model on one B200.

    python -m gruboros_b200.tools.bench_decode [--model 1b] [--tokens 256] [--batches 1 8] [--reference]

Ours: ``Decoder.step`` (one CUDA graph per token: 4 weight-streaming kernels per layer).  Each step is followed by a
greedy argmax on the device that feeds the next step, as a generation loop would; time is CUDA events around the
whole loop, after a warm-up loop.  "ours_sampled" is ``Decoder.generate``: the sampling kernel (temperature, top-p)
sits in the same graph as the step, so the host only replays graphs.  Reported with the weight bytes read per token and the fraction of the measured
HBM copy bandwidth that this amounts to.  ``--reference`` also times the reference model (baseline/_ref, cast to
bf16 as its generate.py does, generate.py:141-144) stepping through its module forward with ``prev_hiddens``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from ..models.minlm import minLM
from .bench_ops import peaks

MODELS = {"1b": dict(num_tokens=256, dim=2048, depth=20), "100m": dict(num_tokens=256, dim=512, depth=32),
          "3b": dict(num_tokens=256, dim=3072, depth=26)}


def timed_loop(step, first_tok, n):
    tok = first_tok
    for _ in range(8):
        tok = step(tok).argmax(-1, keepdim=True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        tok = step(tok).argmax(-1, keepdim=True)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="1b", choices=list(MODELS))
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--batches", type=int, nargs="+", default=[1, 8])
    ap.add_argument("--reference", action="store_true")
    a = ap.parse_args(argv)
    hbm, _, _, src = peaks()
    torch.manual_seed(0)
    model = minLM(**MODELS[a.model]).cuda()
    with torch.no_grad():                       # the zero-initialised output projections would make every step trivial
        for p in model.parameters():
            if p.dim() == 2 and float(p.abs().max()) == 0.0:
                p.normal_(0, 0.02 / p.shape[1] ** 0.5)
    eng = model.fused_engine()
    wbytes = 2 * sum(p.numel() for n, p in model.named_parameters() if p.dim() == 2 and not n.startswith("token_emb"))
    res = {"model": a.model, "weight_bytes_per_token": wbytes, "ours": {}, "reference": {}}
    for B in a.batches:
        dec = eng.decoder(B)
        dec.reset()
        dec.prefill(torch.randint(0, 256, (B, 16), device="cuda"))
        ms = timed_loop(dec.step, torch.randint(0, 256, (B, 1), device="cuda"), a.tokens)
        # the whole loop on the device: sampling kernel + step in one graph per token (temperature 0.85, top-p 0.9)
        dec.generate(8, temperature=0.85, top_p=0.9, seed=1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dec.generate(a.tokens, temperature=0.85, top_p=0.9, seed=2)
        e1.record()
        torch.cuda.synchronize()
        ms_gen = e0.elapsed_time(e1) / a.tokens
        res.setdefault("ours_sampled", {})[f"batch{B}"] = {"ms_per_token_step": round(ms_gen, 4),
                                                           "tokens_per_s": round(B * 1e3 / ms_gen, 1)}
        res["ours"][f"batch{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B * 1e3 / ms, 1),
                                    "weight_GBs": round(wbytes / ms / 1e6, 1),
                                    f"frac_of_{src}_hbm": round(wbytes / ms / 1e6 / hbm, 3),
                                    "launches_per_step": dec.launches_per_step}
    if a.reference:
        ref_root = Path(__file__).resolve().parents[2] / "baseline" / "_ref"
        if not (ref_root / "mingru" / "minLM.py").exists():
            res["reference"] = "baseline/_ref not installed"
        else:
            for k in [k for k in sys.modules if k == "mingru" or k.startswith("mingru.")]:
                del sys.modules[k]
            sys.path.insert(0, str(ref_root))
            from mingru.minLM import minLM as RefLM
            ref = RefLM(**MODELS[a.model]).cuda().bfloat16().eval()
            for B in a.batches:
                with torch.no_grad():
                    _, hid = ref(torch.randint(0, 256, (B, 16), device="cuda"), return_prev_hiddens=True)
                    state = {"h": hid}

                    def step(tok):
                        lg, state["h"] = ref(tok, return_prev_hiddens=True, prev_hiddens=state["h"])
                        return lg[:, -1]

                    ms = timed_loop(step, torch.randint(0, 256, (B, 1), device="cuda"), a.tokens)
                res["reference"][f"batch{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B * 1e3 / ms, 1)}
            for B in a.batches:
                res.setdefault("speedup", {})[f"batch{B}"] = round(
                    res["reference"][f"batch{B}"]["ms_per_step"] / res["ours"][f"batch{B}"]["ms_per_step"], 2)
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
