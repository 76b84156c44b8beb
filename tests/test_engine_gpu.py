"""Fused sm_100a engine against the plain PyTorch module path (fp32) on the same weights."""
import copy
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from gruboros_b200.models.minlm import minLM
from gruboros_b200.optim.schedulefree import AdamWScheduleFree
from tests.test_model_cpu import randomize, zipf_bytes


def cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()


def make_pair(dim=128, depth=2, seed=1):
    torch.manual_seed(0)
    ref = minLM(num_tokens=256, dim=dim, depth=depth)
    randomize(ref, seed)
    fused = copy.deepcopy(ref).cuda()
    ref = ref.cuda()
    ref.use_fused = False
    return fused, ref


@pytest.mark.parametrize("B,chunk", [(2, 65), (3, 130)])
def test_loss_and_grads_match_module_path(B, chunk):
    fused, ref = make_pair()
    x = zipf_bytes(B, 2 * chunk).cuda()
    hid_f = hid_r = None
    for c in range(2):
        ck = x[:, c * chunk:(c + 1) * chunk]
        lf, hid_f = fused(ck, return_loss=True, return_prev_hiddens=True, prev_hiddens=hid_f)
        lr, hid_r = ref(ck, return_loss=True, return_prev_hiddens=True, prev_hiddens=hid_r)
        assert abs(lf.item() - lr.item()) < 2e-2 * max(1.0, abs(lr.item())), (lf.item(), lr.item())
        (lf / 2).backward()
        (lr / 2).backward()
        for a, b in zip(hid_f, hid_r):
            assert a.shape == b.shape
            assert cos(a, b) > 0.999
        hid_f = [h.detach() for h in hid_f]
        hid_r = [h.detach() for h in hid_r]
    from gruboros_b200.ops import _lib as L
    L.check_device_status()
    for (n, p), (_, q) in zip(fused.named_parameters(), ref.named_parameters()):
        assert p.grad is not None, n
        c = cos(p.grad, q.grad)
        rel = (p.grad.double().norm() / q.grad.double().norm().clamp_min(1e-30)).item()
        assert c > 0.99 and 0.95 < rel < 1.05, (n, c, rel)


def _rel_errors(got, want):
    got, want = got.double(), want.double()
    d = got - want
    return (d.norm() / want.norm().clamp_min(1e-30)).item(), (d.abs().max() / want.abs().max().clamp_min(1e-30)).item()


def test_loss_and_grads_match_reference_modules_in_fp64():
    """The fused engine against the REFERENCE's own modules evaluated in fp64 on the same weights, at a size where
    every kernel runs many tiles (dim 512, depth 2, T = 2047, two chunks with carry).  The bounds are what bf16
    operands with fp32 accumulation allow: relative L2 error of every gradient tensor <= 1.5e-2, and its largest
    element-wise error <= 6e-2 of the tensor's largest gradient (the maximum, over up to 10^6 elements, of rounding
    noise whose relative rms is about 1e-2)."""
    from tests.refload import load_reference_mingru
    REF = load_reference_mingru()
    if REF is None:
        pytest.skip("reference tree not present")
    _, ref_lm = REF
    torch.manual_seed(0)
    fused = minLM(num_tokens=256, dim=512, depth=2)
    randomize(fused, 3)
    ref = ref_lm.minLM(num_tokens=256, dim=512, depth=2).double()
    ref.load_state_dict({k: v.double() for k, v in fused.state_dict().items()})
    fused, ref = fused.cuda(), ref.cuda()
    chunk = 2048
    x = zipf_bytes(2, 2 * chunk, seed=9).cuda()
    hid_f = hid_r = None
    for c in range(2):
        ck = x[:, c * chunk:(c + 1) * chunk]
        lf, hid_f = fused(ck, return_loss=True, return_prev_hiddens=True, prev_hiddens=hid_f)
        lr, hid_r = ref(ck, return_loss=True, return_prev_hiddens=True, prev_hiddens=hid_r)
        assert abs(lf.item() - lr.item()) < 5e-3 * max(1.0, abs(lr.item())), (c, lf.item(), lr.item())
        (lf / 2).backward()
        (lr / 2).backward()
        for a, b in zip(hid_f, hid_r):
            l2, mx = _rel_errors(a, b)
            assert l2 < 1e-2 and mx < 2e-2, ("hidden", c, l2, mx)
        hid_f = [h.detach() for h in hid_f]
        hid_r = [h.detach() for h in hid_r]
    from gruboros_b200.ops import _lib as L
    L.check_device_status()
    worst = []
    for (n, p), (_, q) in zip(fused.named_parameters(), ref.named_parameters()):
        l2, mx = _rel_errors(p.grad, q.grad)
        worst.append((l2, mx, n))
        assert l2 < 1.5e-2 and mx < 6e-2, (n, l2, mx)
    print("largest gradient errors (rel L2, rel max):", sorted(worst, reverse=True)[:3])


def test_discarded_grads_restart_from_zero_with_a_torch_optimizer():
    """torch.optim.AdamW.zero_grad() and module.zero_grad() drop ``p.grad`` (set_to_none=True is the default).  The
    fused backward ACCUMULATES into one flat buffer, so it must restart dropped gradients from zero: with the
    weights frozen (lr 0) the third backward on the same chunk gives the first one's gradients, not three times them."""
    fused, _ = make_pair(dim=128, depth=2)
    opt = torch.optim.AdamW(fused.parameters(), lr=0.0)
    ck = zipf_bytes(2, 65, seed=4).cuda()
    norms = []
    for c in range(3):
        fused(ck, return_loss=True).backward()
        norms.append(torch.stack([p.grad.double().norm() for p in fused.parameters()]))
        opt.step()
        if c == 1:
            fused.zero_grad()
        else:
            opt.zero_grad()
        assert all(p.grad is None for p in fused.parameters())
    for later in norms[1:]:
        ratio = later / norms[0].clamp_min(1e-30)
        assert (ratio - 1).abs().max().item() < 1e-3, ratio
    # gradients that were NOT dropped keep accumulating (gradient accumulation over chunks relies on it)
    fused(ck, return_loss=True).backward()
    fused(ck, return_loss=True).backward()
    twice = torch.stack([p.grad.double().norm() for p in fused.parameters()])
    assert ((twice / norms[0].clamp_min(1e-30)) - 2).abs().max().item() < 1e-2


def test_resume_then_fused_step_matches_uninterrupted_run(tmp_path):
    """Optimizer state loaded BEFORE the engine moved the parameters into its flat buffer (the order train.py
    resumes in) is adopted by the flat z / exp_avg_sq buffers at the first step."""
    from gruboros_b200.runtime.trainer import Trainer
    a, _ = make_pair(dim=128, depth=2)
    oa = AdamWScheduleFree(a.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4); oa.train()
    ta = Trainer(a, oa, chunk_size=65)
    x = zipf_bytes(2, 4 * 65, seed=11).cuda()
    for c in range(2):
        ta.step_chunk(x[:, c * 65:(c + 1) * 65])
    ckpt = {"model": {k: v.clone() for k, v in a.state_dict().items()}, "opt": copy.deepcopy(oa.state_dict())}
    hidden = [h.clone() for h in ta.hidden]
    # fresh model + optimizer, state loaded before the first fused step
    torch.manual_seed(0)
    b = minLM(num_tokens=256, dim=128, depth=2).cuda()
    ob = AdamWScheduleFree(b.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    b.load_state_dict(ckpt["model"])
    ob.load_state_dict(ckpt["opt"])
    ob.train()
    tb = Trainer(b, ob, chunk_size=65)
    tb.hidden = hidden
    la, lb = [], []
    for c in range(2, 4):
        ck = x[:, c * 65:(c + 1) * 65]
        la.append(ta.step_chunk(ck)); lb.append(tb.step_chunk(ck))
    torch.cuda.synchronize()
    assert tb.last_folded == ta.last_folded
    assert (torch.stack(la) - torch.stack(lb)).abs().max().item() < 1e-3
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert (p - q).abs().max().item() < 1e-4, n
    za, zb = a.fused_engine().flat.sf_z, b.fused_engine().flat.sf_z
    assert (za - zb).abs().max().item() < 1e-4


def test_train_step_equals_autograd_path():
    fused, _ = make_pair()
    other = copy.deepcopy(fused)
    x = zipf_bytes(2, 65).cuda()
    loss_a, hid_a = fused.fused_engine().train_step(x, None, loss_scale=0.5)
    loss_b, hid_b = other(x, return_loss=True, return_prev_hiddens=True)
    (loss_b * 0.5).backward()
    assert abs(loss_a.item() - loss_b.item()) < 1e-5
    for (n, p), (_, q) in zip(fused.named_parameters(), other.named_parameters()):
        assert cos(p.grad, q.grad) > 0.9999, n


def test_inference_logits_and_decode():
    fused, ref = make_pair()
    x = zipf_bytes(1, 24).cuda()
    with torch.no_grad():
        lf = fused(x)
        lr = ref(x)
        assert lf.shape == lr.shape
        assert (lf - lr).abs().max().item() < 0.05 * lr.abs().max().item() + 1e-3
        logits, hid = fused(x[:, :8], return_prev_hiddens=True)
        outs = [logits[:, -1]]
        for t in range(8, 24):
            logits, hid = fused(x[:, : t + 1], return_prev_hiddens=True, prev_hiddens=hid)
            assert logits.shape == (1, 1, 256)
            outs.append(logits[:, -1])
        dec = torch.stack(outs, 1)
        assert (dec - lr[:, 7:]).abs().max().item() < 0.05 * lr.abs().max().item() + 1e-3


def test_fused_optimizer_matches_unfused_and_trains():
    """Same gradients into the fused (one kernel over the flat buffer) and the per-tensor PyTorch step."""
    fused, _ = make_pair(dim=128, depth=2)
    slow = copy.deepcopy(fused)
    slow.use_fused = False
    of = AdamWScheduleFree(fused.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4)
    os_ = AdamWScheduleFree(slow.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4, fused=False)
    of.train(); os_.train()
    x = zipf_bytes(4, 8 * 65, seed=3).cuda()
    losses = []
    for c in range(8):
        ck = x[:, c * 65:(c + 1) * 65]
        loss = fused(ck, return_loss=True)
        loss.backward()
        for p, q in zip(fused.parameters(), slow.parameters()):
            q.grad = p.grad.clone()
        of.step(); os_.step()
        of.zero_grad(); os_.zero_grad()
        assert all(float(p.grad.abs().max()) == 0 for p in fused.parameters())
        losses.append(loss.item())
    assert of.fused_launches == 8 and os_.fused_launches == 0
    for (n, p), (_, q) in zip(fused.named_parameters(), slow.named_parameters()):
        assert (p - q).abs().max().item() < 1e-5 * max(1.0, q.abs().max().item()), n
    sd = of.state_dict()
    assert set(sd["state"][0]) == {"z", "exp_avg_sq"} and sd["param_groups"][0]["k"] == 8
    assert all(math.isfinite(v) for v in losses)
    assert losses[-1] < losses[0]
    # eval()/train() round trip returns to the same y
    before = [p.detach().clone() for p in fused.parameters()]
    of.eval(); of.train()
    for b, p in zip(before, fused.parameters()):
        assert (b - p).abs().max().item() < 1e-5


def test_overlapped_optimizer_equals_separate_step():
    """Trainer folds the optimizer into backward (per-layer ranges on a side stream); same result as step()."""
    from gruboros_b200.runtime.trainer import Trainer
    a, _ = make_pair(dim=128, depth=3)
    b = copy.deepcopy(a)
    oa = AdamWScheduleFree(a.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4); oa.train()
    ob = AdamWScheduleFree(b.parameters(), lr=1e-3, betas=(0.9, 0.995), weight_decay=1e-4); ob.train()
    ta, tb = Trainer(a, oa, chunk_size=65), Trainer(b, ob, chunk_size=65)
    tb.overlap_optimizer = False
    x = zipf_bytes(3, 4 * 65, seed=21).cuda()
    la = torch.stack(ta.train_sequence(x))
    lb = torch.stack(tb.train_sequence(x))
    torch.cuda.synchronize()
    assert ta.optimizer_steps == tb.optimizer_steps == 4
    assert oa.param_groups[0]["k"] == ob.param_groups[0]["k"] == 4 and oa.fused_launches == 4
    assert (la - lb).abs().max().item() < 2e-3
    fa, fb = a.fused_engine().flat, b.fused_engine().flat
    d = (fa.data - fb.data).abs()
    assert d.max().item() < 1e-2 and d.mean().item() < 2e-5, (d.max().item(), d.mean().item())
    assert float(fa.grad.abs().max()) == 0.0                  # every range cleared its gradients
    assert torch.equal(fa.w16, fa.data.bfloat16())            # bf16 mirror rewritten by the ranged steps
