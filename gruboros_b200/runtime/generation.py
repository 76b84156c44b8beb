"""Text generation from a trained minLM (the reference's generate.py:30-326 as a library).

``load_model`` accepts a checkpoint file, a checkpoint directory (``latest.pt``) with ``config.json`` as the
fallback for the model configuration, or a bare ``state_dict``; a ``_orig_mod.`` prefix left by torch.compile
is stripped.  ``generate`` runs the prompt through the parallel scan once, then decodes token by token carrying
the per-layer hidden state (O(1) state per layer).  On a B200 both phases go through the fused engine.
Sampling supports temperature (0 = greedy), top-k and nucleus (top-p) filtering.
"""
from __future__ import annotations

import json
import os
import sys
import time

import torch
import torch.nn.functional as F

from ..models.minlm import minLM


def decode_token(tok: int) -> str:
    return chr(max(32, tok)) if tok < 128 else "?" if tok > 255 else chr(tok)


def decode_tokens(tokens) -> str:
    return bytes(int(t) & 0xFF for t in tokens).decode("utf-8", errors="replace")


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0) -> torch.Tensor:
    """logits [B, V] -> token ids [B, 1]."""
    if temperature == 0.0:
        return logits.argmax(dim=-1, keepdim=True)
    logits = logits.float() / temperature
    if top_k > 0:
        k = min(top_k, logits.size(-1))
        kth = torch.topk(logits, k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p > 0.0:
        srt, idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(F.softmax(srt, dim=-1), dim=-1)
        drop = cum > top_p
        drop[..., 1:] = drop[..., :-1].clone()      # keep the first token that crosses the threshold
        drop[..., 0] = False
        logits = logits.masked_fill(torch.zeros_like(drop).scatter(-1, idx, drop), float("-inf"))
    return torch.multinomial(F.softmax(logits, dim=-1), num_samples=1)


def load_model(path: str, device="auto", use_bf16=True, use_fp16=False, use_f32=False):
    """Returns (model in eval mode on `device`, model_config)."""
    if device == "auto":
        device = "cuda" if torch.cuda.is_available() else "cpu"
    ckpt_dir = path if os.path.isdir(path) else os.path.dirname(path)
    if os.path.isdir(path):
        path = os.path.join(path, "latest.pt")
        if not os.path.exists(path):
            raise FileNotFoundError(f"no latest.pt in {ckpt_dir}")
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    config = ckpt.get("model_config") if isinstance(ckpt, dict) else None
    if config is None:
        cfg_path = os.path.join(ckpt_dir, "config.json")
        if not os.path.exists(cfg_path):
            raise ValueError("checkpoint has no model_config and there is no config.json beside it")
        with open(cfg_path) as f:
            config = json.load(f)
    state = ckpt["model_state_dict"] if isinstance(ckpt, dict) and "model_state_dict" in ckpt else ckpt
    state = {k[len("_orig_mod."):] if k.startswith("_orig_mod.") else k: v for k, v in state.items()}
    model = minLM(**config)
    model.load_state_dict(state)
    model.eval()
    model = model.to(device)
    if torch.device(device).type == "cuda" and not use_f32 and not model._fusable:
        # the fused engine keeps fp32 masters and computes in bf16 itself; only the module path is cast
        model = model.to(torch.float16 if use_fp16 else torch.bfloat16)
    return model, config


@torch.no_grad()
def generate(model, prompt: torch.Tensor, generation_length: int, temperature=1.0, top_k=0, top_p=0.0,
             device="cuda", stream=True, out=sys.stdout):
    """prompt [1, T] token ids -> generated ids [1, generation_length]."""
    model.eval()
    prompt = prompt.to(device)
    t0 = time.time()
    pending = bytearray()

    def emit(t):
        pending.append(int(t) & 0xFF)
        try:
            text = pending.decode("utf-8")
        except UnicodeDecodeError:
            if len(pending) < 4:
                return
            text = pending.decode("utf-8", errors="replace")
        out.write(text)
        out.flush()
        pending.clear()

    if stream:
        out.write("PROMPT: '" + decode_tokens(prompt[0].tolist()) + "'\nGENERATED: '")
    # On a B200 the fused decoder keeps the recurrent state on the device and replays one CUDA graph per token that
    # holds the sampling kernel and the decode step (models/decode.py); everywhere else each step goes through the
    # module with the state carried by the caller and PyTorch sampling.
    fused = (prompt.is_cuda and getattr(model, "_fusable", False) and getattr(model, "use_fused", False)
             and prompt.shape[0] <= 8 and model.num_tokens <= 256)
    if fused:
        dec = model.fused_engine().decoder(prompt.shape[0])
        dec.reset()
        dec.prefill(prompt)
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())          # follows torch.manual_seed
        result = dec.generate(generation_length, temperature, top_k, top_p, seed=seed,
                              on_token=(lambda t: emit(t[0])) if stream else None)
    else:
        logits, hidden = model(prompt, return_prev_hiddens=True)
        tok = sample(logits[:, -1, :], temperature, top_k, top_p)
        tokens = [tok]
        if stream:
            emit(tok.item())
        for _ in range(1, generation_length):
            logits, hidden = model(tok, return_prev_hiddens=True, prev_hiddens=hidden)
            tok = sample(logits[:, -1, :], temperature, top_k, top_p)
            tokens.append(tok)
            if stream:
                emit(tok.item())
        result = torch.cat(tokens, dim=1)
    if stream:
        dt = time.time() - t0
        out.write(f"'\n\nINFO: Generation complete! ({generation_length / dt if dt > 0 else 0:.2f} tokens/sec)\n")
    return result


def load_primer_text(primer_file=None, primer_length=None, primer_text=None, explicit_length=False) -> torch.Tensor:
    if primer_text:
        toks = list(primer_text.encode("utf-8"))
        if explicit_length and primer_length and len(toks) > primer_length:
            toks = toks[:primer_length]
    elif primer_file:
        with open(primer_file, encoding="utf-8") as f:
            toks = list(f.read().encode("utf-8"))
        if primer_length and len(toks) > primer_length:
            toks = toks[:primer_length]
    else:
        toks = list(b"The ")
    return torch.tensor(toks, dtype=torch.long)[None, :]
