"""Decode kernels (csrc/decode.cu) and the graph-captured decoder against plain PyTorch fp32 references."""
import io

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from gruboros_b200.ops import _lib as L
from gruboros_b200.ops import kernels as K
from gruboros_b200.runtime.generation import generate
from tests.test_engine_gpu import cos, make_pair
from tests.test_model_cpu import zipf_bytes


def bf(t):
    return t.bfloat16().float()


def ref_gemv(epi, x, w16, out_before, norm_w, bias, eps, has_prev):
    """The op of csrc/decode.h in fp32 on the bf16-rounded operands."""
    xin = x
    if norm_w is not None:
        xin = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * norm_w
    acc = bf(xin) @ w16.float().t()
    if epi == K.DEC_GATE:
        N = out_before.shape[1]
        u, k = acc[:, :N], acc[:, N:]
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        z = torch.sigmoid(k)
        return torch.lerp(out_before, cand, z) if has_prev else cand * z
    if bias is not None:
        acc = acc + bias
    if epi == K.DEC_RESID:
        return out_before + acc
    if epi == K.DEC_GELU:
        return F.gelu(acc)
    return acc


@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("N,Kd", [(384, 512), (200, 1032), (256, 3072), (256, 8192)])
def test_decode_gemv_matches_fp32_reference(B, N, Kd):
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + N)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    eps = 1e-6
    for epi, norm, use_bias, has_prev in [(K.DEC_STORE, True, False, True), (K.DEC_STORE, False, True, True),
                                          (K.DEC_GATE, True, False, True), (K.DEC_GATE, True, False, False),
                                          (K.DEC_RESID, False, True, True), (K.DEC_RESID, False, False, True),
                                          (K.DEC_GELU, True, True, True)]:
        x = rn(B, Kd)
        rows = 2 * N if epi == K.DEC_GATE else N
        w16 = (rn(rows, Kd) / Kd ** 0.5).bfloat16()
        norm_w = 1.0 + 0.1 * rn(Kd) if norm else None
        bias = rn(N) if use_bias else None
        out = rn(B, N).abs() + 0.1
        want = ref_gemv(epi, x, w16, out.clone(), norm_w, bias, eps, has_prev)
        K.decode_gemv(epi, x, w16, out, norm_w=norm_w, bias=bias, eps=eps, has_prev=has_prev)
        torch.cuda.synchronize()
        err = (out - want).abs().max().item()
        assert err < 2e-2 * max(1.0, want.abs().max().item()), (epi, norm, use_bias, has_prev, err)
        assert cos(out, want) > 0.9999
    L.check_device_status()


@pytest.mark.parametrize("B", [1, 3, 8])
@pytest.mark.parametrize("N,Kd", [(384, 512), (200, 1032), (2048, 3072), (256, 8192), (1000, 64)])
def test_decode_tc_matches_fp32_reference(B, N, Kd):
    """Tensor-core chain kernel: every input transform, bias, accumulate-into-output and the housekeeping jobs."""
    g = torch.Generator(device="cuda").manual_seed(B * 77 + N)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    eps = 1e-6
    w16 = (rn(N, Kd) / Kd ** 0.5).bfloat16()
    for mode in (K.IN_NORM, K.IN_GATE, K.IN_GELU):
        out = rn(B, N)
        before = out.clone()
        bias = rn(N)
        dirty, cdst, csrc = rn(5000), rn(B, 77), rn(B, 77)
        if mode == K.IN_NORM:
            x, nw = rn(B, Kd), 1.0 + 0.1 * rn(Kd)
            inp = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * nw
            K.decode_tc(mode, x, w16, out, vec=nw, out_bias=bias, zero=dirty, copy=(cdst, csrc), eps=eps)
        elif mode == K.IN_GATE:
            ku, h = rn(B, 2 * Kd), rn(B, Kd).abs() + 0.1
            u, k = ku[:, :Kd], ku[:, Kd:]
            inp = torch.lerp(h, torch.where(u >= 0, u + 0.5, torch.sigmoid(u)), torch.sigmoid(k))
            hn = torch.full_like(h, float("nan"))
            h_before = h.clone()
            K.decode_tc(mode, ku, w16, out, state=h, state_out=hn, out_bias=bias, zero=dirty, copy=(cdst, csrc))
            torch.cuda.synchronize()
            assert torch.equal(h, h_before)                       # the old state is left alone
            assert torch.allclose(hn, inp, atol=1e-5, rtol=1e-5)  # the new state, in fp32
        else:
            a, b1 = rn(B, Kd), rn(Kd)
            inp = F.gelu(a + b1)
            K.decode_tc(mode, a, w16, out, vec=b1, out_bias=bias, zero=dirty, copy=(cdst, csrc))
        torch.cuda.synchronize()
        want = before + bf(inp) @ w16.float().t() + bias
        err = (out - want).abs().max().item()
        assert err < 2e-2 * max(1.0, want.abs().max().item()), (mode, err)
        assert cos(out - before, want - before) > 0.9999
        assert float(dirty.abs().max()) == 0.0 and torch.equal(cdst, csrc)
    L.check_device_status()


def test_decode_gemv_rejects_bad_shapes():
    x = torch.zeros(9, 64, device="cuda")
    w = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        K.decode_gemv(K.DEC_STORE, x, w, torch.zeros(9, 8, device="cuda"))          # more than 8 sequences
    x = torch.zeros(1, 60, device="cuda")
    w = torch.zeros(8, 60, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        K.decode_gemv(K.DEC_STORE, x, w, torch.zeros(1, 8, device="cuda"))          # K not a multiple of 8


@pytest.mark.parametrize("impl", ["tc", "gemv"])
@pytest.mark.parametrize("B", [1, 2, 5])
def test_decoder_follows_module_path(B, impl):
    fused, ref = make_pair(dim=128, depth=3, seed=4)
    prompt = zipf_bytes(B, 19).cuda()
    follow = zipf_bytes(B, 12).cuda()
    with torch.no_grad():
        lr, hid = ref(prompt.long(), return_prev_hiddens=True)
        dec = fused.fused_engine().decoder(B, impl=impl)
        dec.reset()
        lf = dec.prefill(prompt)
        assert cos(lf, lr[:, -1]) > 0.999
        for t in range(follow.shape[1]):
            tok = follow[:, t:t + 1]
            lr, hid = ref(tok.long(), return_prev_hiddens=True, prev_hiddens=hid)
            lf = dec.step(tok)
            assert lf.shape == (B, 256)
            assert cos(lf, lr[:, -1]) > 0.999, t
            assert (lf - lr[:, -1]).abs().max().item() < 5e-2 * max(1.0, lr.abs().max().item())
        for a, b in zip(dec.hiddens(), hid):
            assert a.shape == b.shape and cos(a, b) > 0.999
    L.check_device_status()


@pytest.mark.parametrize("impl", ["tc", "gemv"])
def test_decoder_without_prompt_and_graph_equals_eager(impl):
    fused, ref = make_pair(dim=128, depth=2, seed=7)
    toks = zipf_bytes(2, 6).cuda()
    eng = fused.fused_engine()
    with torch.no_grad():
        dg, de = eng.decoder(2, use_graph=True, impl=impl), eng.decoder(2, use_graph=False, impl=impl)
        assert dg is not de
        dg.reset(); de.reset()
        hid = None
        for t in range(toks.shape[1]):
            a = dg.step(toks[:, t]).clone()
            b = de.step(toks[:, t]).clone()
            if impl == "gemv":
                assert torch.equal(a, b)                   # same kernels, same order: bit-identical
            else:
                assert torch.allclose(a, b, atol=1e-3, rtol=1e-3)      # split-K atomics: summation order varies
            if hid is None:
                lr, hid = ref(toks[:, t:t + 1].long(), return_prev_hiddens=True)
            else:
                lr, hid = ref(toks[:, t:t + 1].long(), return_prev_hiddens=True, prev_hiddens=hid)
            assert cos(a, lr[:, -1]) > 0.999
        assert dg._graph is not None and dg.launches_per_step == 2 + 4 * 2
    L.check_device_status()


def test_decoder_picks_up_new_weights():
    fused, _ = make_pair(dim=128, depth=2, seed=9)
    dec = fused.fused_engine().decoder(1)
    tok = torch.tensor([65], device="cuda")
    with torch.no_grad():
        dec.reset()
        a = dec.step(tok).clone()
        for p in fused.parameters():
            p.mul_(1.5)
        dec.refresh()
        dec.reset()
        b = dec.step(tok).clone()
        fused.use_fused = False
        want = fused(tok.view(1, 1).long())[:, -1]
    assert not torch.allclose(a, b)
    assert cos(b, want) > 0.999


def test_generate_uses_decoder_and_is_deterministic_when_greedy():
    fused, ref = make_pair(dim=128, depth=2, seed=11)
    prompt = zipf_bytes(1, 8)
    out = io.StringIO()
    a = generate(fused, prompt, 16, temperature=0.0, device="cuda", stream=True, out=out)
    b = generate(fused, prompt, 16, temperature=0.0, device="cuda", stream=False)
    assert a.shape == (1, 16) and torch.equal(a, b)
    assert fused.fused_engine().decoder(1).steps == 8 + 16
    assert "tokens/sec" in out.getvalue()
    c = generate(ref, prompt, 16, temperature=0.0, device="cuda", stream=False)      # module path, fp32
    assert c.shape == (1, 16)


def filtered_probs(logits, temperature, top_k, top_p):
    """The distribution runtime.generation.sample draws from (same filtering, kept as probabilities)."""
    logits = logits.float() / temperature
    if top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.size(-1)), dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p > 0.0:
        srt, idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.cumsum(F.softmax(srt, dim=-1), dim=-1)
        drop = cum > top_p
        drop[..., 1:] = drop[..., :-1].clone()
        drop[..., 0] = False
        logits = logits.masked_fill(torch.zeros_like(drop).scatter(-1, idx, drop), float("-inf"))
    return F.softmax(logits, dim=-1)


@pytest.mark.parametrize("V", [256, 200])
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 0.0), (0.85, 0, 0.9), (1.3, 40, 0.0), (0.7, 17, 0.8), (1.0, 1, 0.0)])
def test_sample_kernel_distribution_and_draw(V, temperature, top_k, top_p):
    g = torch.Generator(device="cuda").manual_seed(V + top_k)
    B = 5
    logits = torch.randn(B, V, device="cuda", generator=g) * 3
    u = torch.rand(B, device="cuda", generator=g)
    tok = torch.zeros(B, dtype=torch.uint8, device="cuda")
    probs = torch.full((B, V), float("nan"), device="cuda")
    K.sample(logits, tok, temperature=temperature, top_k=top_k, top_p=top_p, u=u, probs_out=probs)
    torch.cuda.synchronize()
    want = filtered_probs(logits, temperature, top_k, top_p)
    assert torch.allclose(probs, want, atol=2e-6, rtol=1e-4)
    cdf = torch.cumsum(probs.double(), dim=-1)
    for b in range(B):
        t = int(tok[b])
        assert probs[b, t] > 0
        lo = float(cdf[b, t - 1]) if t > 0 else 0.0
        assert lo - 1e-5 <= float(u[b]) <= float(cdf[b, t]) + 1e-5


def test_sample_kernel_greedy_counter_history_and_seed():
    B, V = 3, 256
    logits = torch.randn(B, V, device="cuda")
    tok = torch.zeros(B, dtype=torch.uint8, device="cuda")
    counter = torch.zeros(2, dtype=torch.int64, device="cuda")
    hist = torch.full((B, 4), -1, dtype=torch.int64, device="cuda")
    K.sample(logits, tok, temperature=0.0, counter=counter, history=hist)
    assert torch.equal(tok.long(), logits.argmax(-1)) and int(counter[0]) == 1
    assert torch.equal(hist[:, 0], logits.argmax(-1)) and bool((hist[:, 1:] == -1).all())
    flat = torch.zeros(1, V, device="cuda")                 # uniform distribution: the draw depends on the generator only
    draws = {}
    for seed in (1, 2):
        counter.copy_(torch.tensor([0, seed]))
        seq = []
        for _ in range(32):
            K.sample(flat, tok[:1], temperature=1.0, counter=counter)
            seq.append(int(tok[0]))
        draws[seed] = seq
    assert draws[1] != draws[2] and len(set(draws[1])) > 16
    counter.copy_(torch.tensor([0, 1]))
    again = []
    for _ in range(32):
        K.sample(flat, tok[:1], temperature=1.0, counter=counter)
        again.append(int(tok[0]))
    assert again == draws[1]


def test_decoder_generate_on_device_matches_stepwise_greedy():
    fused, _ = make_pair(dim=128, depth=2, seed=13)
    prompt = zipf_bytes(2, 10).cuda()
    dec = fused.fused_engine().decoder(2)
    with torch.no_grad():
        dec.reset()
        logits = dec.prefill(prompt)
        want = []
        for _ in range(12):
            t = logits.argmax(-1)
            want.append(t.clone())
            logits = dec.step(t)
        want = torch.stack(want, dim=1)
        dec.reset()
        dec.prefill(prompt)
        seen = []
        got = dec.generate(12, temperature=0.0, on_token=lambda t: seen.append(t.clone()))
    assert got.shape == (2, 12) and got.dtype == torch.int64
    assert (got == want).float().mean().item() > 0.9          # split-K atomics can flip a near-tie
    assert torch.equal(torch.stack(seen, dim=1).long(), got.cpu())
    torch.manual_seed(5)
    a = generate(fused, prompt[:1].cpu(), 24, temperature=0.9, top_p=0.9, device="cuda", stream=False)
    torch.manual_seed(5)
    b = generate(fused, prompt[:1].cpu(), 24, temperature=0.9, top_p=0.9, device="cuda", stream=False)
    assert a.shape == (1, 24) and (a == b).float().mean().item() > 0.9
    L.check_device_status()
