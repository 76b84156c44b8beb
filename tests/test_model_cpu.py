"""Module-level model against the unmodified reference modules evaluated in fp64 (the oracle)."""
import math

import pytest
import torch

from gruboros_b200.models.minlm import minLM
from gruboros_b200.models.mingru import minGRU
from tests.refload import load_reference_mingru

REF = load_reference_mingru()
needs_ref = pytest.mark.skipif(REF is None, reason="reference tree not present")


def zipf_bytes(B, T, seed=0, s=1.1):
    g = torch.Generator().manual_seed(seed)
    w = 1.0 / torch.arange(1, 257, dtype=torch.float64) ** s
    return torch.multinomial(w / w.sum(), B * T, replacement=True, generator=g).view(B, T)


def randomize(model, seed=1):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.5 / math.sqrt(p.shape[-1])) + (1.0 if p.dim() == 1 else 0.0))


def test_state_dict_layout_and_counts():
    m = minLM(num_tokens=256, dim=512, depth=6)
    sd = m.state_dict()
    assert len(sd) == 6 * 8 + 3
    assert sum(v.numel() for v in sd.values()) == 19_944_960
    assert sd["layers.0.2.to_hidden_and_gate.weight"].shape == (2 * 768, 512)
    assert sd["layers.5.4.2.bias"].shape == (512,)
    assert list(sd)[:2] == ["token_emb.weight", "layers.0.1.weight"]


def test_init_is_identity_blocks():
    torch.manual_seed(0)
    m = minLM(num_tokens=256, dim=128, depth=3)
    x = zipf_bytes(2, 65)
    loss = m(x, return_loss=True)
    assert abs(loss.item() - math.log(256)) < 0.01
    assert m.layers[0][2].to_out.weight.abs().max() == 0
    assert m.layers[0][4][2].weight.abs().max() == 0 and m.layers[0][4][2].bias.abs().max() == 0
    std = m.token_emb.weight.std().item()
    assert 0.5 < std / (0.02 / math.sqrt(128)) < 1.5


@needs_ref
@pytest.mark.parametrize("T", [1, 2, 33])
@pytest.mark.parametrize("carry", [False, True])
def test_mingru_matches_reference(T, carry):
    ref_g, _ = REF
    torch.manual_seed(0)
    ours, ref = minGRU(32, expansion_factor=1.5).double(), ref_g.minGRU(32, expansion_factor=1.5).double()
    ref.load_state_dict(ours.state_dict())
    x = torch.randn(2, T, 32, dtype=torch.float64)
    h0 = torch.rand(2, 1, 48, dtype=torch.float64) + 0.1 if carry else None
    a, ha = ours(x, h0, return_next_prev_hidden=True)
    b, hb = ref(x, h0, return_next_prev_hidden=True)
    torch.testing.assert_close(a, b, rtol=1e-10, atol=1e-12)
    torch.testing.assert_close(ha, hb, rtol=1e-10, atol=1e-12)


@needs_ref
def test_minlm_matches_reference_forward_backward_and_carry():
    _, ref_l = REF
    cfg = dict(num_tokens=256, dim=64, depth=3, ff_mult=4, expansion=1.5)
    ours, ref = minLM(**cfg).double(), ref_l.minLM(**cfg).double()
    randomize(ours)
    missing = ref.load_state_dict(ours.state_dict())          # identical key set
    assert not missing.missing_keys and not missing.unexpected_keys
    x = zipf_bytes(2, 130)
    hid_o = hid_r = None
    for c in range(2):                                         # two TBPTT chunks with carry
        chunk = x[:, c * 65:(c + 1) * 65]
        lo, hid_o = ours(chunk, return_loss=True, return_prev_hiddens=True, prev_hiddens=hid_o)
        lr, hid_r = ref(chunk, return_loss=True, return_prev_hiddens=True, prev_hiddens=hid_r)
        torch.testing.assert_close(lo, lr, rtol=1e-10, atol=1e-12)
        lo.backward(); lr.backward()
        hid_o = [h.detach() for h in hid_o]; hid_r = [h.detach() for h in hid_r]
    for (n, p), (_, q) in zip(ours.named_parameters(), ref.named_parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-8, atol=1e-12, msg=n)


def test_decode_equals_parallel():
    torch.manual_seed(0)
    m = minLM(num_tokens=256, dim=64, depth=2).double()
    randomize(m)
    x = zipf_bytes(1, 20)
    full = m(x)
    logits, hid = m(x[:, :5], return_prev_hiddens=True)
    outs = [logits[:, -1]]
    for t in range(5, 20):
        logits, hid = m(x[:, : t + 1], return_prev_hiddens=True, prev_hiddens=hid)
        outs.append(logits[:, -1])
    torch.testing.assert_close(torch.stack(outs, 1), full[:, 4:], rtol=1e-9, atol=1e-10)


def test_conv_and_dropout_variants_run():
    m = minLM(num_tokens=256, dim=32, depth=2, enable_conv=True, dropout=0.1)
    loss = m(zipf_bytes(2, 17), return_loss=True)
    loss.backward()
    assert torch.isfinite(loss)
