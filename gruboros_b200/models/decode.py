"""Token-by-token decoding on the fused path: device-resident recurrent state and one CUDA graph per step.

Generation with a minGRU model keeps O(1) state per layer (the reference carries it through
``prev_hiddens``, generate.py:201-212, and recomputes ``nn.Linear`` GEMVs plus a dozen small ATen kernels per
layer and token).  Here a step is 4 launches per layer of a weight-streaming kernel, captured once in a CUDA
graph, so a step costs one graph launch and reads every weight exactly once.  Two kernel chains exist:

  "tc"    (default) ``csrc/decode_tc.cu``: split-K products on the tcgen05 tensor cores that accumulate with atomics
          into the residual stream or a pre-activation buffer; RMSNorm, the minGRU step and GELU are the input
          transforms of the consuming product.
  "gemv"  ``csrc/decode.cu``: one warp per weight row on the CUDA cores, RMSNorm in the prologue and the
          non-linearities in the epilogue (bit-reproducible; slower).

    dec = model.fused_engine().decoder(batch=1)
    logits = dec.prefill(prompt)            # [B, V] logits after the prompt (parallel scan kernels)
    logits = dec.step(next_token)           # [B, V]; the returned tensor is overwritten by the next step
    tokens = dec.generate(256, temperature=0.85, top_p=0.9)   # sampling kernel + step in one graph per token
"""
from __future__ import annotations

import torch

from ..ops import kernels as K


class Decoder:
    MAX_BATCH = 8

    def __init__(self, engine, batch: int = 1, use_graph: bool = True, impl: str = "tc"):
        if not 1 <= batch <= self.MAX_BATCH:
            raise ValueError(f"decode batch must be 1..{self.MAX_BATCH}")
        self.engine, self.B = engine, batch
        dev = next(engine.model.parameters()).device
        if dev.type != "cuda":
            raise ValueError("the fused decoder needs the model on a CUDA device")
        engine.ensure_flat(dev)
        self.device = dev
        f32 = torch.float32
        D, Di, Fh, V, depth = engine.D, engine.Di, engine.F, engine.V, engine.depth
        self.tok = torch.zeros(batch, 1, dtype=torch.uint8, device=dev)
        self.x = torch.zeros(batch, D, dtype=f32, device=dev)
        self.h = torch.zeros(depth, batch, Di, dtype=f32, device=dev)      # recurrent state; zeros = "no previous state"
        self.a = torch.zeros(batch, Fh, dtype=f32, device=dev)             # feed-forward (pre-)activation
        self.ku = torch.zeros(batch, 2 * Di, dtype=f32, device=dev)        # candidate | gate pre-activations ("tc" chain)
        self.hn = torch.zeros(batch, Di, dtype=f32, device=dev)            # new state of the layer in flight ("tc" chain)
        if impl not in ("tc", "gemv"):
            raise ValueError("impl must be 'tc' or 'gemv'")
        self.impl = impl
        self.logits = torch.zeros(batch, V, dtype=f32, device=dev)
        self.steps = 0
        self._graph = None
        self._flat = engine.flat
        self.use_graph = use_graph
        self.overlap = True       # kernels of a step start early and prefetch their weights (see csrc/decode.h)
        self.launches_per_step = 0
        self._gen = None          # (key, graph, history) of the sampling + step graph used by generate()
        self.counter = torch.zeros(2, dtype=torch.int64, device=dev)       # [tokens drawn, seed] read by the sampler

    # ------------------------------------------------------------------ state
    def reset(self) -> None:
        self.h.zero_()
        self.ku.zero_()          # the "tc" chain keeps these two zero between steps; restore that after an aborted step
        self.a.zero_()
        self.steps = 0

    def hiddens(self):
        """Per-layer hidden states as the module API carries them: list of [B, 1, dim_inner] (copies)."""
        out = self.h.clone()
        return [out[i].unsqueeze(1) for i in range(self.engine.depth)]

    def load_hiddens(self, prev_hiddens) -> None:
        if prev_hiddens is None:
            self.reset()
            return
        self.h.copy_(torch.stack([p.reshape(self.B, self.engine.Di) for p in prev_hiddens]))

    # ---------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, continue_state: bool = False) -> torch.Tensor:
        """Run the prompt [B, T] through the parallel (scan) kernels, keep the final hidden state, return the
        logits of the last position [B, V].  With ``continue_state`` the prompt extends the current state."""
        eng = self.engine
        tokens = eng._as_tokens(tokens.to(self.device))
        if tokens.shape[0] != self.B:
            raise ValueError(f"decoder was built for batch {self.B}, got {tokens.shape[0]}")
        T = tokens.shape[1]
        prev = self.hiddens() if continue_state and self.steps > 0 else None
        bufs = eng._forward(tokens, T, prev, train=False, want_loss=False)
        self.h.copy_(bufs.h_last)
        self.steps += T
        self.logits.copy_(bufs.logits.view(self.B, T, eng.V)[:, -1])
        return self.logits.clone()

    # ------------------------------------------------------------------- step
    def _kernels(self) -> None:
        if self.impl == "tc":
            self._kernels_tc()
        else:
            self._kernels_gemv()

    def _kernels_tc(self) -> None:
        """Tensor-core chain (csrc/decode_tc.cu): every product accumulates with atomics into the residual stream or
        into a pre-activation buffer, and its non-linearity is the input transform of the next product."""
        eng = self.engine
        ix, eps, sms, ov = eng._idx, eng.eps, eng._sms, self.overlap
        K.embed_fwd(self.tok, 1, eng._p(ix["emb"]), self.x)
        self.logits.zero_()
        for i, lx in enumerate(ix["layers"]):
            K.decode_tc(K.IN_NORM, self.x, eng._w(lx["wg"]), self.ku, vec=eng._p(lx["n1"]), zero=self.a, eps=eps, sms=sms,
                        overlap=ov)
            K.decode_tc(K.IN_GATE, self.ku, eng._w(lx["wo"]), self.x, state=self.h[i], state_out=self.hn, sms=sms, overlap=ov)
            K.decode_tc(K.IN_NORM, self.x, eng._w(lx["w1"]), self.a, vec=eng._p(lx["n2"]), zero=self.ku,
                        copy=(self.h[i], self.hn), eps=eps, sms=sms, overlap=ov)
            K.decode_tc(K.IN_GELU, self.a, eng._w(lx["w2"]), self.x, vec=eng._p(lx["b1"]), out_bias=eng._p(lx["b2"]), sms=sms,
                        overlap=ov)
        K.decode_tc(K.IN_NORM, self.x, eng._w(ix["logits"]), self.logits, vec=eng._p(ix["normf"]), eps=eps, sms=sms, overlap=ov)

    def _kernels_gemv(self) -> None:
        """CUDA-core chain (csrc/decode.cu): one warp per weight row, non-linearities in the epilogue."""
        eng = self.engine
        ix, eps, sms, ov = eng._idx, eng.eps, eng._sms, self.overlap
        K.embed_fwd(self.tok, 1, eng._p(ix["emb"]), self.x)
        for i, lx in enumerate(ix["layers"]):
            K.decode_gemv(K.DEC_GATE, self.x, eng._w(lx["wg"]), self.h[i], norm_w=eng._p(lx["n1"]), eps=eps, sms=sms, overlap=ov)
            K.decode_gemv(K.DEC_RESID, self.h[i], eng._w(lx["wo"]), self.x, sms=sms, overlap=ov)
            K.decode_gemv(K.DEC_GELU, self.x, eng._w(lx["w1"]), self.a, norm_w=eng._p(lx["n2"]), bias=eng._p(lx["b1"]),
                          eps=eps, sms=sms, overlap=ov)
            K.decode_gemv(K.DEC_RESID, self.a, eng._w(lx["w2"]), self.x, bias=eng._p(lx["b2"]), sms=sms, overlap=ov)
        K.decode_gemv(K.DEC_STORE, self.x, eng._w(ix["logits"]), self.logits, norm_w=eng._p(ix["normf"]), eps=eps, sms=sms, overlap=ov)

    def refresh(self) -> None:
        """Pick up changed weights (call after an optimizer step or a load_state_dict) and re-record the step."""
        self.engine.ensure_flat(self.device)
        self.engine.sync_weights()
        self._capture()

    def _capture(self) -> None:
        """Record one step.  The recording run is preceded by an eager one (first-use set-up of the kernels), and
        both act on a saved copy of the state, which is restored afterwards."""
        saved = self.h.clone()
        cur = torch.cuda.current_stream(self.device)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            n0 = K.LAUNCHES
            self._kernels()
            self.launches_per_step = K.LAUNCHES - n0
        cur.wait_stream(side)
        if self.use_graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._kernels()
            self._graph = g
        self.h.copy_(saved)
        self._flat = self.engine.flat
        self._gen = None          # a recorded sampling + step graph points at the buffers of the previous recording

    @torch.no_grad()
    def step(self, tok: torch.Tensor) -> torch.Tensor:
        """One token per sequence ([B] or [B, 1] integer ids) -> logits [B, V] (a buffer the next step overwrites)."""
        if self.launches_per_step == 0 or self.engine.flat is not self._flat:
            self.refresh()
        self.tok.copy_(tok.reshape(self.B, 1))
        if self._graph is not None:
            self._graph.replay()
            K.LAUNCHES += self.launches_per_step
        else:
            self._kernels()
        self.steps += 1
        return self.logits

    # --------------------------------------------------------------- generate
    @torch.no_grad()
    def generate(self, n: int, temperature: float = 1.0, top_k: int = 0, top_p: float = 0.0, seed: int = 0,
                 on_token=None) -> torch.Tensor:
        """Continue every sequence by ``n`` tokens, starting from the logits of the last ``prefill`` / ``step``.

        Sampling (``csrc/sample.cu``: temperature, top-k, top-p, inverse-CDF draw) and the decode step are captured
        together in one CUDA graph; the drawn token feeds the next step on the device, so the host only replays the
        graph n times.  ``on_token(tokens_uint8_cpu [B])`` is called after every step if given (one small D2H copy
        per token, for streaming output).  Returns int64 [B, n]."""
        if self.launches_per_step == 0 or self.engine.flat is not self._flat:
            self.refresh()
        key = (float(temperature), int(top_k), float(top_p), self.impl, self.overlap)
        if self._gen is None or self._gen[0] != key or self._gen[2].shape[1] < n or self.engine.flat is not self._flat:
            hist = torch.zeros(self.B, max(n, 256), dtype=torch.int64, device=self.device)

            def body():
                K.sample(self.logits, self.tok, temperature=temperature, top_k=top_k, top_p=top_p, counter=self.counter,
                         history=hist)
                self._kernels()

            saved_h, saved_l = self.h.clone(), self.logits.clone()
            cur = torch.cuda.current_stream(self.device)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                body()                                       # eager run first: one-time kernel set-up
            cur.wait_stream(side)
            graph = None
            if self.use_graph:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    body()
            self.h.copy_(saved_h)
            self.logits.copy_(saved_l)
            self._gen = (key, graph, hist, body)
        _, graph, hist, body = self._gen
        self.counter.copy_(torch.tensor([0, int(seed)], dtype=torch.int64))
        for _ in range(n):
            if graph is not None:
                graph.replay()
                K.LAUNCHES += self.launches_per_step + 2
            else:
                body()
            if on_token is not None:
                on_token(self.tok.view(-1).cpu())
        self.steps += n
        return hist[:, :n].clone()
