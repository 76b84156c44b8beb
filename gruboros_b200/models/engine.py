"""Fused sm_100a execution engine for ``minLM``.

A forward (and backward) pass is a fixed sequence of hand-written kernels over
preallocated buffers - no autograd graph, no per-op allocation:

  forward, per layer                              kernel (csrc/)
    ku  = RMSNorm(x) Wg^T          bf16 [M,2Di]   tcgen05 GEMM, rows scaled by rstd in the epilogue   gemm_sm100_2cta.cu
    h   = minGRU scan(k, u, h0)    bf16, fp32 carry  scan_fwd            scan.cu
    x   = x + h Wo^T               fp32           GEMM, residual epilogue (+ x*w bf16 and row sums of x^2 for the next norm)
    g,f = gelu'(a), gelu(a), a = RMSNorm(x) W1^T + b1   bf16   GEMM, row scale + bias + GELU epilogue
    x   = x + f W2^T + b2          fp32           GEMM, bias + residual epilogue (+ next norm's inputs)
  head: one GEMM whose epilogue is the final RMSNorm's row scale and the 256-way cross-entropy
        (per-row loss and d logits straight from tensor memory).

  RMSNorm never runs as a pass of its own: the GEMM (or the embedding gather) that PRODUCES x also writes the
  bf16 operand x * w_norm and per-row partial sums of x^2; the GEMM that CONSUMES the norm multiplies its
  accumulator rows by rsqrt(mean(x^2) + eps), which commutes with the contraction.

  backward mirrors it: wgrad GEMMs read both operands MN-major and accumulate with
  red.add into the flat fp32 gradient buffer (split-K for SM occupancy), dgrad GEMMs read
  the weights MN-major (no transposed copies), GELU' (saved by forward) and the feed-forward bias gradient are a
  dgrad epilogue, the scan has its own reverse kernel, RMSNorm backward also accumulates the residual gradient
  and the bias / norm-weight gradients.  The gradients flowing into a folded norm's consumer are scaled by rstd
  where they are produced, so wgrad and dgrad work on the unnormalised operand.

The residual stream and every reduction are fp32; GEMM operands are bf16 (the precision the
reference trains at under bf16 autocast, mingru/minLM.py:86-155 being the module-level math).
"""
from __future__ import annotations

import math
import os

import torch

from ..ops import kernels as K
from ..ops import _lib as L
from ..utils.flat import FlatParams, lookup

NUM_SMS_DEFAULT = 148


def pick_splitk(n_out: int, k_out: int, m_red: int, sms: int, remote: bool = False) -> int:
    """Split factor for a wgrad GEMM (256 x 256 output tiles, one per pair of SMs) so that tiles * split fills whole
    waves.  Every split adds one more partial tile to the reduction; when the reduction crosses NVLink (`remote`,
    data parallel) that traffic is the scarcer resource, so the smallest split reaching 80 % wave efficiency is
    taken (at most 2) instead of the most efficient one.

    Returns -1 ("stream-K": equal runs of (tile, k-block) units per SM pair) when there are so few output tiles
    that even a deep split leaves SMs idle (the embedding and logits matrices: 8 tiles for 74 pairs).  For the big
    matrices whole-tile waves win although stream-K balances perfectly: pairs that march through the same k range
    of neighbouring tiles together share operand panels in L2, while stream-K's staggered runs each pull their
    own panels from DRAM (measured on the 6144 x 2048 x 16376 wgrad: 381 us against 309 us)."""
    pairs = max(1, sms // 2)
    tiles = math.ceil(n_out / 256) * math.ceil(k_out / 256)
    kblocks = math.ceil(m_red / 64)
    if tiles * 4 <= pairs and kblocks * tiles >= 8 * pairs:
        return -1
    best, best_eff = 1, 0.0
    for s in range(1, 3 if remote else 9):
        if kblocks // s < 16 and s > 1:
            break
        t = tiles * s
        eff = t / (math.ceil(t / pairs) * pairs)
        if remote and eff >= 0.8:
            return s
        if eff > best_eff + 0.03:
            best, best_eff = s, eff
    return best


class _Buffers:
    """Activations saved by forward and scratch used by backward for one (B, T)."""

    def __init__(self, eng: "FusedEngine", B: int, T: int, train: bool):
        dev = eng.device
        D, Di, Fh, V, depth = eng.D, eng.Di, eng.F, eng.V, eng.depth
        M = B * T
        bf, f32 = torch.bfloat16, torch.float32
        e = lambda *s, dtype=bf: torch.empty(*s, dtype=dtype, device=dev)
        self.B, self.T, self.M, self.train = B, T, M, train
        nres = 2 * depth + 1 if train else 2
        self.xs = [e(M, D, dtype=f32) for _ in range(nres)]
        nl = depth if train else 1
        P = (D + 127) // 128                      # partial sums of squares per row (one per 128 columns)
        # inputs of each RMSNorm in folded form: bf16 x * w, partial sums of x^2; rstd as its consumer computed it
        self.xw1 = [e(M, D) for _ in range(nl)]
        self.xw2 = [e(M, D) for _ in range(nl)]
        self.ssq1 = [e(M, P, dtype=f32) for _ in range(nl)]
        self.ssq2 = [e(M, P, dtype=f32) for _ in range(nl)]
        self.rstd1 = [e(M, dtype=f32) for _ in range(nl)]
        self.rstd2 = [e(M, dtype=f32) for _ in range(nl)]
        self.ku = [e(M, 2 * Di) for _ in range(nl)]
        self.h = [e(M, Di) for _ in range(nl)]
        self.g1 = [e(M, Fh) for _ in range(nl)]   # gelu'(pre-activation), what backward multiplies by
        self.f1 = [e(M, Fh) for _ in range(nl)]
        self.h0 = e(depth, B, Di, dtype=f32)           # carry used by the last forward
        self.h0_valid = False
        self.h_last = e(depth, B, Di, dtype=f32)
        self.xwf = e(M, D)
        self.ssqf = e(M, P, dtype=f32)
        self.rstdf = e(M, dtype=f32)
        self.labels = e(M, dtype=torch.uint8)
        self.loss_rows = e(M, dtype=f32)
        self.loss = torch.zeros(1, dtype=f32, device=dev)
        if train:
            self.onehot = e(M, V)
            self.dlogits = e(M, V)
            self.dres = [e(M, D, dtype=f32) for _ in range(2)]
            self.dres16 = e(M, D)
            self.dy16 = e(M, D)
            self.da1 = e(M, Fh)
            self.dh = e(M, Di)
            self.dku = e(M, 2 * Di)
        else:
            self.logits = e(M, V, dtype=f32)

    def li(self, i: int) -> int:
        return i if self.train else 0


class FusedEngine:
    def __init__(self, model):
        self.model = model
        self.D = model.dim
        self.depth = model.depth
        self.V = model.num_tokens
        self.Di = model.layers[0][2].dim_inner
        self.F = model.layers[0][4][0].out_features
        if self.V > 256:
            raise ValueError("the fused cross-entropy epilogue handles vocabularies up to 256 (byte-level models)")
        if self.D % 64 or self.Di % 8 or self.F % 8:
            raise ValueError("fused path needs dim % 64 == 0 and inner sizes that are multiples of 8")
        self.flat: FlatParams | None = None
        # fully sharded training installs its own parameter storage here (parallel/fsdp.py): an object with names,
        # device, param(i) / grad(i) fp32 views of the small replicated parameters, weight(i) bf16 views of gathered weights
        # and scatter(i) -> destination of matrix i's gradient; None: everything lives in `flat`
        self.store = None
        self.device = None
        self._bufs: dict = {}
        self._gen = 0
        self._sms = NUM_SMS_DEFAULT
        self.eps = torch.finfo(torch.float32).eps    # nn.RMSNorm(eps=None) on an fp32 residual stream
        self.grad_sink = None   # data parallel: (peer base pointers of the flat grad buffers, elements per owner)
        # sharded parameters (FSDP): object with begin_pass(direction) and prefetch(direction, layer) -> keyword
        # arguments for the GEMM that all-gathers the next unit's bf16 weights with its copy warps ({} when resident)
        self.param_gather = None
        self.launches_last = 0
        self._side = None        # side stream for the optimizer ranges overlapped with backward
        # GRB_NVTX=1 wraps every layer of a pass in an NVTX range (visible in Nsight timelines)
        self.nvtx = os.environ.get("GRB_NVTX", "0") == "1"
        # how a wgrad GEMM's reduction over the M rows is split over the machine: "tiles" (default: equal split-K
        # parts per output tile, factor from pick_splitk, stream-K only for matrices of a few tiles) or "stream"
        self.wgrad_split = os.environ.get("GRB_WGRAD_SPLIT", "tiles")

    # ------------------------------------------------------------- parameters
    def ensure_flat(self, device) -> FlatParams:
        """Parameters live in one flat fp32 buffer; (re)build it if the module was moved or re-assigned."""
        device = torch.device(device)
        self.device = device
        if self.store is not None:
            src = self.store
        else:
            first = next(self.model.parameters())
            owner = lookup(first)
            if owner is not None and owner.intact() and owner.device == device and len(owner.params) == len(list(self.model.parameters())):
                self.flat = owner
            else:
                self.flat = FlatParams(self.model, device)
                self._bufs.clear()
            src = self.flat
        if not hasattr(self, "_idx") or self._idx_owner is not src:
            names = {n: i for i, n in enumerate(src.names)}
            ix = lambda n: names[n]
            self._idx = {
                "emb": ix("token_emb.weight"), "normf": ix("norm.weight"), "logits": ix("to_logits.weight"),
                "layers": [
                    dict(n1=ix(f"layers.{i}.1.weight"), wg=ix(f"layers.{i}.2.to_hidden_and_gate.weight"),
                         wo=ix(f"layers.{i}.2.to_out.weight"), n2=ix(f"layers.{i}.3.weight"),
                         w1=ix(f"layers.{i}.4.0.weight"), b1=ix(f"layers.{i}.4.0.bias"),
                         w2=ix(f"layers.{i}.4.2.weight"), b2=ix(f"layers.{i}.4.2.bias"))
                    for i in range(self.depth)],
            }
            self._idx_owner = src
            self._sms = torch.cuda.get_device_properties(device).multi_processor_count
        return src

    def sync_weights(self) -> None:
        """Refresh the bf16 mirror if any parameter changed since it was last written."""
        if self.store is not None:
            return                      # sharded storage: the optimizer step writes the bf16 shards itself
        f = self.flat
        ver = f.version() + f.data._version
        if f.w16_version != ver:
            K.cast_f32_bf16(f.data, f.w16)
            f.w16_version = ver

    def weights_updated_in_place(self) -> None:
        """Called by the fused optimizer after it rewrote parameters and the bf16 mirror together."""
        f = self.flat
        f.w16_version = f.version() + f.data._version

    def _p(self, i):      # fp32 parameter view
        return self.store.param(i) if self.store is not None else self.flat.view(self.flat.data, i)

    def _w(self, i):      # bf16 mirror view
        return self.store.weight(i) if self.store is not None else self.flat.view(self.flat.w16, i)

    def _g(self, i):      # fp32 gradient view
        return self.store.grad(i) if self.store is not None else self.flat.view(self.flat.grad, i)

    def _wgrad(self, dy16, x16, i, splitk):
        """Gradient of weight matrix i: local accumulate, or the fused reduce-scatter when data parallel."""
        if self.store is not None:
            K.linear_wgrad(dy16, x16, None, splitk=splitk, scatter=self.store.scatter(i))
        elif self.grad_sink is None:
            K.linear_wgrad(dy16, x16, self._g(i), splitk=splitk)
        else:
            peers, shard = self.grad_sink
            K.linear_wgrad(dy16, x16, None, splitk=splitk, scatter=(peers, shard, self.flat.offsets[i], False, self.flat.numel))

    def buffers(self, B, T, train) -> _Buffers:
        key = (B, T, train)
        b = self._bufs.get(key)
        if b is None:
            if len(self._bufs) >= 4:
                self._bufs.clear()
            b = _Buffers(self, B, T, train)
            self._bufs[key] = b
        return b

    # ---------------------------------------------------------------- carry
    def _load_carry(self, bufs: _Buffers, prev_hiddens) -> bool:
        if prev_hiddens is None:
            return False
        prev = list(prev_hiddens)
        if len(prev) != self.depth:
            raise ValueError(f"expected {self.depth} hidden states, got {len(prev)}")
        if any(p.numel() == 0 for p in prev):
            return False                      # empty carry: same as no carry
        for i, p in enumerate(prev):
            if p.numel() != bufs.B * self.Di:
                raise ValueError(f"hidden state {i} has {p.numel()} elements, expected batch {bufs.B} x inner dim {self.Di}")
        bufs.h0.copy_(torch.stack([p.reshape(bufs.B, self.Di) for p in prev]))
        return True

    # -------------------------------------------------------------- forward
    def _forward(self, tokens: torch.Tensor, T: int, prev_hiddens, *, train: bool, want_loss: bool, alpha: float = 1.0):
        """tokens: uint8 [B, >=T(+1)] on the device.  Returns the buffer set holding the results."""
        dev = tokens.device
        self.ensure_flat(dev)
        self.sync_weights()
        B = tokens.shape[0]
        bufs = self.buffers(B, T, train)
        n0 = K.LAUNCHES
        M, D, Di, Fh, V = bufs.M, self.D, self.Di, self.F, self.V
        has_h0 = self._load_carry(bufs, prev_hiddens)
        bufs.h0_valid = has_h0
        ix = self._idx
        pg = self.param_gather
        if pg is not None:
            pg.begin_pass("fwd")
        layers = ix["layers"]
        eps = self.eps
        K.embed_fwd(tokens, T, self._p(ix["emb"]), bufs.xs[0], bufs.labels if want_loss else None,
                    bufs.onehot if train else None, next_norm=(self._p(layers[0]["n1"]), bufs.xw1[0], bufs.ssq1[0]))
        for i, lx in enumerate(layers):
            if self.nvtx:
                torch.cuda.nvtx.range_push(f"fwd layer {i}")
            j = bufs.li(i)
            x_in = bufs.xs[2 * i] if train else bufs.xs[0]
            x_mid = bufs.xs[2 * i + 1] if train else bufs.xs[1]
            x_out = bufs.xs[2 * i + 2] if train else bufs.xs[0]
            K.linear_fwd(bufs.xw1[j], self._w(lx["wg"]), bufs.ku[j], rownorm=(bufs.ssq1[j], D, eps, bufs.rstd1[j]),
                         **(pg.prefetch("fwd", i) if pg is not None else {}))
            ku3 = bufs.ku[j].view(B, T, 2 * Di)
            K.scan_fwd(ku3[..., Di:], ku3[..., :Di], bufs.h[j].view(B, T, Di),
                       h0=bufs.h0[i] if has_h0 else None, h_last=bufs.h_last[i])
            K.linear_fwd(bufs.h[j], self._w(lx["wo"]), x_mid, epi=K.EPI_RESID_F32, aux=x_in,
                         next_norm=(self._p(lx["n2"]), bufs.xw2[j], bufs.ssq2[j]))
            K.linear_fwd(bufs.xw2[j], self._w(lx["w1"]), bufs.g1[j], epi=K.EPI_BIAS_GELU, out1=bufs.f1[j],
                         bias=self._p(lx["b1"]), rownorm=(bufs.ssq2[j], D, eps, bufs.rstd2[j]))
            if i + 1 < self.depth:       # the norm that follows this block: next layer's first, or the final one
                jn = bufs.li(i + 1)
                nxt = (self._p(layers[i + 1]["n1"]), bufs.xw1[jn], bufs.ssq1[jn])
            else:
                nxt = (self._p(ix["normf"]), bufs.xwf, bufs.ssqf)
            K.linear_fwd(bufs.f1[j], self._w(lx["w2"]), x_out, epi=K.EPI_RESID_F32, aux=x_mid, bias=self._p(lx["b2"]),
                         next_norm=nxt)
            if self.nvtx:
                torch.cuda.nvtx.range_pop()
        if want_loss:
            K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_CE, bufs.xwf, self._w(ix["logits"]), M, V, D,
                   out0=bufs.dlogits if train else None, out1=bufs.loss_rows, aux=bufs.labels, ldo=V, alpha=alpha / M,
                   rownorm=(bufs.ssqf, D, eps, bufs.rstdf))
            K.sum_scale(bufs.loss_rows, 1.0 / M, bufs.loss)
        else:
            K.linear_fwd(bufs.xwf, self._w(ix["logits"]), bufs.logits, epi=K.EPI_STORE_F32,
                         rownorm=(bufs.ssqf, D, eps, None))
        self._gen += 1
        bufs.gen = self._gen
        self.launches_last = K.LAUNCHES - n0
        return bufs

    # ------------------------------------------------------------- backward
    def unit_ranges(self):
        """Flat element ranges [lo, hi) of the parameter units in the order backward completes their gradients:
        head (final norm + logits), layers depth-1 .. 0, embedding."""
        f, ix = self.flat, self._idx
        end = lambda i: f.offsets[i] + (f.params[i].numel() + 63) // 64 * 64
        units = [(f.offsets[ix["normf"]], end(ix["logits"]))]
        for lx in reversed(ix["layers"]):
            units.append((f.offsets[lx["n1"]], end(lx["b2"])))
        units.append((f.offsets[ix["emb"]], end(ix["emb"])))
        return units

    def _backward(self, bufs: _Buffers, unit_done=None) -> None:
        """Gradients of the last training forward on `bufs`, accumulated into the flat fp32 gradient buffer.
        `unit_done(j)` is called as soon as every gradient of unit j (see unit_ranges) has been launched."""
        if not bufs.train or bufs.gen != self._gen:
            raise RuntimeError("backward must follow the training forward whose activations it uses")
        n0 = K.LAUNCHES
        if self.grad_sink is None and self.store is None:
            self.flat.reclaim_discarded_grads()     # gradients the caller dropped (p.grad = None) start from zero
        B, T, M = bufs.B, bufs.T, bufs.M
        D, Di, Fh, V = self.D, self.Di, self.F, self.V
        ix = self._idx
        sms = self._sms
        if self.wgrad_split == "stream":
            sk = lambda n, k: -1       # every wgrad dealt as equal runs of (tile, k-block) units per SM pair
        else:
            sk = lambda n, k: pick_splitk(n, k, M, sms, remote=self.grad_sink is not None and len(self.grad_sink[0]) > 2)
        pg = self.param_gather
        if pg is not None:
            pg.begin_pass("bwd")
        # head.  Every gradient that flows into the consumer of a folded norm already carries that norm's rstd
        # (d logits from the cross-entropy epilogue, d(k,u) from the scan, d(pre-activation) from the GELU' epilogue),
        # so wgrad and dgrad run on the saved unnormalised operand and the norm's backward takes the `prescaled` form.
        self._wgrad(bufs.dlogits, bufs.xwf, ix["logits"], sk(V, D))
        K.linear_dgrad(bufs.dlogits, self._w(ix["logits"]), bufs.dy16,
                       **(pg.prefetch("bwd", self.depth) if pg is not None else {}))
        last = ix["layers"][-1]
        dres_a, dres_b = bufs.dres
        K.rmsnorm_bwd(bufs.dy16, bufs.xs[2 * self.depth], bufs.rstdf, self._p(ix["normf"]), None, dres_a, bufs.dres16,
                      self._g(ix["normf"]), self._g(last["b2"]), prescaled=True)
        for i in range(self.depth - 1, -1, -1):
            lx = ix["layers"][i]
            x_in, x_mid = bufs.xs[2 * i], bufs.xs[2 * i + 1]
            # feed-forward: x_out = x_mid + gelu(RMSNorm(x_mid) W1^T + b1) W2^T + b2
            self._wgrad(bufs.dres16, bufs.f1[i], lx["w2"], sk(D, Fh))
            K.linear_dgrad(bufs.dres16, self._w(lx["w2"]), bufs.da1, epi=K.EPI_GELU_BWD, aux=bufs.g1[i],
                           colsum=self._g(lx["b1"]), rowscale=bufs.rstd2[i],
                           **(pg.prefetch("bwd", i) if pg is not None else {}))
            self._wgrad(bufs.da1, bufs.xw2[i], lx["w1"], sk(Fh, D))
            K.linear_dgrad(bufs.da1, self._w(lx["w1"]), bufs.dy16)
            K.rmsnorm_bwd(bufs.dy16, x_mid, bufs.rstd2[i], self._p(lx["n2"]), dres_a, dres_b, bufs.dres16,
                          self._g(lx["n2"]), None, prescaled=True)
            # minGRU: x_mid = x_in + scan(RMSNorm(x_in) Wg^T) Wo^T
            self._wgrad(bufs.dres16, bufs.h[i], lx["wo"], sk(D, Di))
            K.linear_dgrad(bufs.dres16, self._w(lx["wo"]), bufs.dh)
            ku3 = bufs.ku[i].view(B, T, 2 * Di)
            dku3 = bufs.dku.view(B, T, 2 * Di)
            K.scan_bwd(ku3[..., Di:], ku3[..., :Di], bufs.h[i].view(B, T, Di), bufs.dh.view(B, T, Di),
                       dku3[..., Di:], dku3[..., :Di], h0=bufs.h0[i] if bufs.h0_valid else None, rowscale=bufs.rstd1[i])
            self._wgrad(bufs.dku, bufs.xw1[i], lx["wg"], sk(2 * Di, D))
            K.linear_dgrad(bufs.dku, self._w(lx["wg"]), bufs.dy16)
            prev_b2 = self._g(ix["layers"][i - 1]["b2"]) if i > 0 else None
            K.rmsnorm_bwd(bufs.dy16, x_in, bufs.rstd1[i], self._p(lx["n1"]), dres_b, dres_a, bufs.dres16,
                          self._g(lx["n1"]), prev_b2, prescaled=True)
            if unit_done is not None:
                if i == self.depth - 1:
                    unit_done(0)                    # head: its last gradient (final-norm weight) came before this layer
                unit_done(self.depth - i)
        # embedding: dE[v] += sum over rows with token v of dres  ==  onehot^T dres
        self._wgrad(bufs.onehot, bufs.dres16, ix["emb"], sk(V, D))
        if unit_done is not None:
            unit_done(self.depth + 1)
        self._gen += 1          # activations are consumed
        self.launches_last += K.LAUNCHES - n0

    # ----------------------------------------------------------- public API
    @staticmethod
    def _as_tokens(x: torch.Tensor) -> torch.Tensor:
        if x.dtype != torch.uint8:
            x = x.to(torch.uint8)
        if x.stride(-1) != 1:
            x = x.contiguous()
        return x

    def _hiddens_out(self, bufs: _Buffers):
        out = bufs.h_last.clone()
        return [out[i].unsqueeze(1) for i in range(self.depth)]

    def train_step(self, chunk: torch.Tensor, prev_hiddens=None, loss_scale: float = 1.0, optimizer=None, stepper=None):
        """Forward + backward of one TBPTT chunk without autograd.

        chunk: [B, chunk_size] byte tokens (uint8 or integer) on the GPU; the first chunk_size-1 are
        inputs and the last chunk_size-1 the labels, as in the reference (mingru/minLM.py:94-95).
        Gradients of ``loss_scale * mean CE`` are accumulated into the parameters' ``.grad``.
        With ``optimizer`` (a Schedule-Free AdamW covering exactly this model, no gradient accumulation pending) the
        optimizer step is folded in: as soon as backward has produced the last gradient of a layer, that layer's
        flat range is updated on a side stream, so the memory-bound update hides under the remaining GEMMs.
        ``stepper`` generalises that: an object with ``begin(units)``, ``unit_done(j, main, side)`` and
        ``end(main, side)`` (the data-parallel wrapper passes one that also synchronises the ranks per layer).
        Returns (loss [0-dim fp32 tensor, unscaled], next hidden states [list of [B,1,Di]]).
        """
        tokens = self._as_tokens(chunk)
        T = tokens.shape[1] - 1
        bufs = self._forward(tokens, T, prev_hiddens, train=True, want_loss=True, alpha=loss_scale)
        if stepper is None and optimizer is not None:
            stepper = _LocalStepper(optimizer, self.flat)
        if stepper is None:
            self._backward(bufs)
        else:
            units = self.unit_ranges()
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=self.device)
            side = self._side
            stepper.begin(units)
            self._backward(bufs, lambda j: stepper.unit_done(j, main, side))
            stepper.end(main, side)
        if self.store is None:
            self.flat.attach_grads()
        return bufs.loss[0].clone(), self._hiddens_out(bufs)

    def decoder(self, batch: int = 1, use_graph: bool = True, impl: str = "tc"):
        """Token-by-token generation state for `batch` sequences (``models/decode.py``), cached per configuration."""
        from .decode import Decoder
        if not hasattr(self, "_decoders"):
            self._decoders = {}
        key = (batch, use_graph, impl)
        d = self._decoders.get(key)
        if d is None or d.device != next(self.model.parameters()).device:
            d = self._decoders[key] = Decoder(self, batch, use_graph, impl)
        return d

    def module_forward(self, x, return_loss, return_prev_hiddens, prev_hiddens):
        tokens = self._as_tokens(x)
        if return_loss:
            T = tokens.shape[1] - 1
            need_grad = torch.is_grad_enabled() and any(p.requires_grad for p in self.model.parameters())
            if need_grad:
                self.ensure_flat(tokens.device)
                loss = _FusedLoss.apply(next(iter(self.model.parameters())), self, tokens, T, prev_hiddens)
                bufs = self.buffers(tokens.shape[0], T, True)
            else:
                bufs = self._forward(tokens, T, prev_hiddens, train=False, want_loss=True)
                loss = bufs.loss[0].clone()
            return (loss, self._hiddens_out(bufs)) if return_prev_hiddens else loss
        if prev_hiddens is not None:
            tokens = tokens[:, -1:]
        T = tokens.shape[1]
        bufs = self._forward(tokens, T, prev_hiddens, train=False, want_loss=False)
        logits = bufs.logits.view(tokens.shape[0], T, self.V).clone()
        return (logits, self._hiddens_out(bufs)) if return_prev_hiddens else logits


class _LocalStepper:
    """Optimizer step of a single replica folded into backward: unit j's flat range is updated on the side stream as
    soon as its last gradient kernel has been launched on the main stream."""

    def __init__(self, optimizer, flat):
        self.optimizer, self.flat = optimizer, flat

    def begin(self, units):
        self.units = units
        self.hp = self.optimizer.begin_ranged_step(self.flat)

    def unit_done(self, j, main, side):
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ev)
            self.optimizer.step_range(self.flat, self.units[j][0], self.units[j][1], self.hp)

    def end(self, main, side):
        main.wait_stream(side)
        self.optimizer.end_ranged_step(self.flat)


class _FusedLoss(torch.autograd.Function):
    """Autograd node for ``loss = model(x, return_loss=True)`` on the fused path: backward runs the engine's
    backward kernels, which accumulate straight into the flat gradient buffer that every ``p.grad`` views."""

    @staticmethod
    def forward(ctx, anchor, engine, tokens, T, prev_hiddens):
        bufs = engine._forward(tokens, T, prev_hiddens, train=True, want_loss=True, alpha=1.0)
        ctx.engine, ctx.bufs = engine, bufs
        return bufs.loss[0].clone()

    @staticmethod
    def backward(ctx, gloss):
        engine, bufs = ctx.engine, ctx.bufs
        # d logits were written for d(loss) = 1; fold the incoming scale in (device-side, no sync)
        bufs.dlogits.copy_(bufs.dlogits.float() * gloss)
        engine._backward(bufs)
        if engine.store is None:
            engine.flat.attach_grads()
        return None, None, None, None, None
