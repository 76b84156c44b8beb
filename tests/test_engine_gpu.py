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
