"""Operator micro-benchmarks on one B200, CUDA-event timed after warm-up, inputs larger than L2.

  scan      minGRU log-space scan, forward and backward, B8 x T8192 x C3072, bf16 in / fp32 accumulate, h0 carry:
            the sm_100a kernels vs. the reference's eager formulation (softplus / cumsum / logcumsumexp, fp32 under
            autocast; mingru/minGRU.py:16-28,56-67) and vs. the HBM roofline.
  gemm      the tcgen05 GEMMs on the 1B model's shapes vs. torch.matmul (cuBLAS).
  gemm_fused the fused-epilogue GEMMs exactly as a 1B layer issues them (residual add, bias + GELU, GELU').
  rmsnorm   RMSNorm backward (+ residual-gradient accumulation): shared-memory ring vs. register version.
  optimizer fused Schedule-Free AdamW vs. the HBM roofline.

    python -m gruboros_b200.tools.bench_ops [scan] [gemm] [gemm_fused] [rmsnorm] [optimizer]   -> one JSON object on stdout
    (no argument: scan, gemm and optimizer)
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch
import torch.nn.functional as F

from ..ops import kernels as K


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


def timeit(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def rnd(*s):
    return torch.randn(*s, device="cuda").bfloat16()


def reference_scan(k, u, h0):
    """The reference's parallel branch, evaluated as bf16 autocast would: fp32 elementwise and scans."""
    k, u = k.float(), u.float()
    log_coeffs = -F.softplus(k)
    log_z = -F.softplus(-k)
    log_tilde_h = torch.where(u >= 0, (F.relu(u) + 0.5).log(), -F.softplus(-u))
    log_values = torch.cat((h0.log().unsqueeze(1), log_z + log_tilde_h), dim=1)
    log_coeffs = F.pad(log_coeffs, (0, 0, 1, 0))
    a_star = log_coeffs.cumsum(dim=1)
    return (a_star + (log_values - a_star).logcumsumexp(dim=1)).exp()[:, 1:]


def bench_scan(B=8, T=8192, C=3072):
    hbm, _, _, src = peaks()
    k, u = rnd(B, T, C), rnd(B, T, C)
    h0 = torch.randn(B, C, device="cuda").abs() + 0.1
    h = torch.empty(B, T, C, device="cuda", dtype=torch.bfloat16)
    hl = torch.empty(B, C, device="cuda")
    g = rnd(B, T, C)
    dk, du, dh0 = torch.empty_like(k), torch.empty_like(k), torch.empty(B, C, device="cuda")
    fwd = timeit(lambda: K.scan_fwd(k, u, h, h0=h0, h_last=hl))
    bwd = timeit(lambda: K.scan_bwd(k, u, h, g, dk, du, h0=h0, dh0=dh0))
    one = B * T * C * 2
    out = {"shape": [B, T, C], "fwd_us": fwd * 1e3, "bwd_us": bwd * 1e3,
           "fwd_GBs": 3 * one / fwd / 1e6, "bwd_GBs": 6 * one / bwd / 1e6,
           "fwd_frac_of_%s_hbm" % src: 3 * one / fwd / 1e6 / hbm, "bwd_frac_of_%s_hbm" % src: 6 * one / bwd / 1e6 / hbm,
           "bytes_model": "fwd reads k,u writes h (3 tensors); bwd reads k,u,h,g writes dk,du (6 tensors)"}
    kr, ur = k.clone().requires_grad_(True), u.clone().requires_grad_(True)

    def ref_fwd():
        with torch.no_grad():
            reference_scan(kr, ur, h0)

    def ref_fwd_bwd():
        kr.grad = ur.grad = None
        reference_scan(kr, ur, h0).backward(g.float())

    try:
        rf = timeit(ref_fwd, iters=3, warm=1)
        rfb = timeit(ref_fwd_bwd, iters=3, warm=1)
        out.update(reference_fwd_us=rf * 1e3, reference_fwd_bwd_us=rfb * 1e3, speedup_fwd=rf / fwd,
                   speedup_fwd_bwd=rfb / (fwd + bwd))
    except torch.cuda.OutOfMemoryError:
        out["reference"] = "out of memory"
    return out


class _ClockSampler:
    """SM clock / power of GPU 0 through NVML (read-only) every 50 ms while a loop runs."""

    def __init__(self):
        import threading
        self.clk, self.pw, self._stop = [], [], False
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv, self._h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        except Exception:
            self._nv = None
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        import time
        while not self._stop and self._nv is not None:
            self.clk.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
            self.pw.append(self._nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            time.sleep(0.05)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop = True
        self._t.join()

    def summary(self):
        c = sorted(self.clk)
        return {"sm_mhz_median": c[len(c) // 2] if c else None, "power_w_max": round(max(self.pw)) if self.pw else None}


def sustained(fn, flops, secs=2.5):
    """Back-to-back launches for `secs` seconds (the power-capped regime a training step runs in), CUDA-event timed."""
    import time
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    with _ClockSampler() as smp:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0, n = time.time(), 0
        a.record()
        while time.time() - t0 < secs:
            for _ in range(20):
                fn()
            n += 20
            torch.cuda.synchronize()
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / n
    return dict(us=round(ms * 1e3, 1), tflops=round(flops / ms / 1e9, 1), **smp.summary())


def bench_gemm(M=16376, secs=2.5):
    """Ours vs torch.matmul (cuBLAS) on the 1B model's projections, every pass, sustained loops with sampled clocks.
    Operand layouts are the ones the engine uses: forward x W^T (both K-major), dgrad dy W (W read MN-major), wgrad
    dy^T x (both MN-major, fp32 accumulate with red.add, split-K as the engine picks it); cuBLAS gets the same
    logical operands (transposed views) and writes bf16."""
    from ..models.engine import pick_splitk
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    _, burst, sust, src = peaks()
    shapes = {"gate": (M, 6144, 2048), "out": (M, 2048, 3072), "ff1": (M, 8192, 2048), "ff2": (M, 2048, 8192)}
    out = {"seconds_per_loop": secs, "peaks": {"bf16_tflops_burst": burst, "bf16_tflops_sustained": sust, "source": src}}
    for name, (m, n, k) in shapes.items():
        a, b, dy = rnd(m, k), rnd(n, k), rnd(m, n)
        o = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        dx = torch.empty(m, k, device="cuda", dtype=torch.bfloat16)
        dw, dw16 = torch.zeros(n, k, device="cuda"), torch.empty(n, k, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * m * n * k
        sk = pick_splitk(n, k, m, sms)
        res = {
            "fwd": sustained(lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_STORE_BF16, a, b, m, n, k, out0=o), fl, secs),
            "fwd_cublas": sustained(lambda: torch.matmul(a, b.t(), out=o), fl, secs),
            "dgrad": sustained(lambda: K.gemm(K.MAJOR_K, K.MAJOR_MN, K.EPI_STORE_BF16, dy, b, m, k, n, out0=dx), fl, secs),
            "dgrad_cublas": sustained(lambda: torch.matmul(dy, b, out=dx), fl, secs),
            "wgrad": sustained(lambda: K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_F32, dy, a, n, k, m, out0=dw, splitk=sk), fl, secs),
            "wgrad_cublas": sustained(lambda: torch.matmul(dy.t(), a, out=dw16), fl, secs),
            "wgrad_splitk": sk,
        }
        for p in ("fwd", "dgrad", "wgrad"):
            res[p + "_vs_cublas"] = round(res[p]["tflops"] / res[p + "_cublas"]["tflops"], 3)
            res[p + "_frac_of_%s_sustained" % src] = round(res[p]["tflops"] / sust, 3)
        out[name] = res
        del a, b, dy, o, dx, dw, dw16
    return out


def bench_wgrad_variants(M=16376, secs=1.5):
    """What the weight-gradient GEMM (both operands MN-major) loses, and where: `red.add` with split-K 1 - 4, a plain
    fp32 store with split-K 1 (no accumulation, no partial tiles) and cuBLAS on the same operands (bf16 output),
    sustained loops, TFLOP/s."""
    out = {}
    for name, (n, k) in {"gate": (6144, 2048), "ff1": (8192, 2048), "out": (2048, 3072)}.items():
        dy, a = rnd(M, n), rnd(M, k)
        dw = torch.zeros(n, k, device="cuda")
        dw16 = torch.empty(n, k, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * n * k
        r = {}
        for sk in (1, 2, 3, 4):
            r[f"red_split{sk}"] = sustained(lambda: K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_F32, dy, a, n, k, M, out0=dw, splitk=sk), fl, secs)["tflops"]
        r["store_f32_split1"] = sustained(lambda: K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_STORE_F32, dy, a, n, k, M, out0=dw), fl, secs)["tflops"]
        r["cublas"] = sustained(lambda: torch.matmul(dy.t(), a, out=dw16), fl, secs)["tflops"]
        out[name] = r
        del dy, a, dw, dw16
    return out


def bench_optimizer_overlap(M=16376, n_gemm=2000, n_opt=120):
    """Does the fused optimizer hide behind GEMMs on a second stream?  n_gemm GEMMs on one stream and n_opt optimizer
    steps of 128 Mi parameters on another, each alone and both together (CUDA events around the whole batch; the
    launches of the two streams are interleaved so that neither queue runs dry)."""
    n = 128 * 1024 * 1024
    y, z, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    w16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    dy, wgt, x = rnd(M, 6144), rnd(6144, 2048), rnd(M, 2048)
    dx = torch.empty(M, 2048, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(6144, 2048, device="cuda")
    gemms = {"dgrad_bf16_store": lambda: K.gemm(K.MAJOR_K, K.MAJOR_MN, K.EPI_STORE_BF16, dy, wgt, M, 2048, 6144, out0=dx),
             "wgrad_red_split3": lambda: K.gemm(K.MAJOR_MN, K.MAJOR_MN, K.EPI_RED_F32, dy, x, 6144, 2048, M, out0=dw, splitk=3)}

    def opt():
        K.sfadamw_step(y, z, v, g, w16, lr=1e-3, beta1=0.9, beta2=0.995, bias2=0.5, eps=1e-8, wd=1e-4, ckp1=0.1)

    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()

    def run(gemm, ng, no):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        s1.wait_stream(torch.cuda.current_stream())
        s2.wait_stream(torch.cuda.current_stream())
        per = max(1, ng // max(1, no)) if no else ng
        gi = oi = 0
        while gi < ng or oi < no:
            with torch.cuda.stream(s1):
                for _ in range(min(per, ng - gi)):
                    gemm()
                    gi += 1
            if oi < no:
                with torch.cuda.stream(s2):
                    opt()
                    oi += 1
        torch.cuda.current_stream().wait_stream(s1)
        torch.cuda.current_stream().wait_stream(s2)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    out = {}
    for name, gemm in gemms.items():
        run(gemm, 200, 10)
        tg, to, tb = run(gemm, n_gemm, 0), run(gemm, 0, n_opt), run(gemm, n_gemm, n_opt)
        out[name] = {"gemm_alone_ms": round(tg, 1), "optimizer_alone_ms": round(to, 1), "both_ms": round(tb, 1),
                     "optimizer_cost_beside_gemm_ms": round(tb - tg, 1)}
    return out


def bench_gemm_fused(M=16376, D=2048, DI=3072, F=8192):
    """The fused-epilogue GEMMs exactly as the 1B layer issues them (TFLOP/s)."""
    out = {}
    h, wo, x = rnd(M, DI), rnd(D, DI), torch.randn(M, D, device="cuda")
    out["out_proj_resid"] = 2.0 * M * D * DI / timeit(lambda: K.linear_fwd(h, wo, x, epi=K.EPI_RESID_F32, aux=x)) / 1e9
    xn, w1, b1 = rnd(M, D), rnd(F, D), torch.randn(F, device="cuda")
    pre, act = (torch.empty(M, F, device="cuda", dtype=torch.bfloat16) for _ in range(2))   # pre: saved GELU derivative
    out["ff1_bias_gelu"] = 2.0 * M * F * D / timeit(
        lambda: K.gemm(K.MAJOR_K, K.MAJOR_K, K.EPI_BIAS_GELU, xn, w1, M, F, D, out0=pre, out1=act, bias=b1)) / 1e9
    w2 = rnd(D, F)
    out["ff2_resid"] = 2.0 * M * D * F / timeit(lambda: K.linear_fwd(act, w2, x, epi=K.EPI_RESID_F32, aux=x)) / 1e9
    dy, dpre = rnd(M, D), torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    out["ff2_dgrad_gelu_bwd"] = 2.0 * M * D * F / timeit(
        lambda: K.gemm(K.MAJOR_K, K.MAJOR_MN, K.EPI_GELU_BWD, dy, w2, M, F, D, out0=dpre, aux=pre)) / 1e9
    return {k: round(v, 1) for k, v in out.items()}


def bench_rmsnorm(M=16376, D=2048):
    """RMSNorm backward fused with the residual-gradient accumulation: 32 bytes per element row-wise
    (x 4 + dres_in 4 + dy 2 read, dres_out 4 + bf16 copy 2 written; the figure counts exactly those)."""
    hbm, _, _, src = peaks()
    n_buf = 6                                           # rotate buffers so that nothing is served from L2
    xs = [torch.randn(M, D, device="cuda") for _ in range(n_buf)]
    ds = [torch.randn(M, D, device="cuda") for _ in range(n_buf)]
    dys = [rnd(M, D) for _ in range(n_buf)]
    w, rstd = torch.ones(D, device="cuda"), torch.rand(M, device="cuda") + 0.5
    out, o16 = torch.empty(M, D, device="cuda"), torch.empty(M, D, device="cuda", dtype=torch.bfloat16)
    dw, dc = torch.zeros(D, device="cuda"), torch.zeros(D, device="cuda")
    it = iter(range(10 ** 9))

    nbytes = M * D * 16.0
    res = {"rows": M, "dim": D}
    for name, ring in (("shared_memory_ring", True), ("register_rows", False)):
        def run():
            i = next(it) % n_buf
            K.rmsnorm_bwd(dys[i], xs[i], rstd, w, ds[i], out, o16, dw, dc, ring=ring)

        t = timeit(run, iters=18)
        res[name] = {"us": round(t * 1e3, 1), "GBs": round(nbytes / t / 1e6, 1),
                     "frac_of_%s_hbm" % src: round(nbytes / t / 1e6 / hbm, 3)}
    return res


def bench_optimizer(n=512 * 1024 * 1024):
    hbm, _, _, src = peaks()
    y, z, v, g = (torch.randn(n, device="cuda") for _ in range(4))
    v.abs_()
    w16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    t = timeit(lambda: K.sfadamw_step(y, z, v, g, w16, lr=1e-3, beta1=0.9, beta2=0.995, bias2=0.5, eps=1e-8, wd=1e-4,
                                      ckp1=0.1), iters=5)
    return {"params": n, "ms": t, "GBs": n * 34 / t / 1e6, "frac_of_%s_hbm" % src: n * 34 / t / 1e6 / hbm,
            "bytes_model": "16 B read + 12 B written + 2 B bf16 mirror + 4 B gradient clear per parameter"}


def main(argv=None):
    which = (argv if argv is not None else sys.argv[1:]) or ["scan", "gemm", "optimizer"]
    res = {}
    if "scan" in which:
        res["scan"] = bench_scan()
    if "gemm" in which:
        res["gemm"] = bench_gemm()
    if "rmsnorm" in which:
        res["rmsnorm_bwd"] = bench_rmsnorm()
        res["rmsnorm_bwd_3b"] = bench_rmsnorm(M=8188, D=3072)
    if "gemm_fused" in which:
        res["gemm_fused"] = bench_gemm_fused()
    if "optimizer_overlap" in which:
        res["optimizer_overlap"] = bench_optimizer_overlap()
    if "wgrad_variants" in which:
        res["wgrad_variants"] = bench_wgrad_variants()
    if "optimizer" in which:
        res["optimizer"] = bench_optimizer()
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
