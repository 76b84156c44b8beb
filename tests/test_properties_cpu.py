"""Property tests (hypothesis) of the recurrence on CPU: the chunk-parallel log-space evaluation, the sequential
definition and chunked evaluation with carry agree for arbitrary shapes, including T = 1 and odd lengths."""
import torch
from hypothesis import given, settings, strategies as st

from gruboros_b200.models.mingru import g, log_g, mingru_scan, minGRU
from gruboros_b200.ops.reference import scan_chunked, scan_ref


@settings(max_examples=25, deadline=None)
@given(B=st.integers(1, 3), T=st.integers(1, 70), C=st.integers(1, 9), carry=st.booleans(), seed=st.integers(0, 10_000))
def test_logspace_scan_equals_sequential_recurrence(B, T, C, carry, seed):
    gen = torch.Generator().manual_seed(seed)
    k = torch.randn(B, T, C, generator=gen, dtype=torch.float64) * 2
    u = torch.randn(B, T, C, generator=gen, dtype=torch.float64) * 2
    h0 = (torch.rand(B, C, generator=gen, dtype=torch.float64) + 0.05) if carry else None
    want, last = scan_ref(k, u, h0)
    got = mingru_scan(u, k, h0.unsqueeze(1) if carry else None)
    torch.testing.assert_close(got, want, rtol=1e-9, atol=1e-12)
    chunked, last_c = scan_chunked(k, u, h0, chunk=7)
    torch.testing.assert_close(chunked, want, rtol=1e-8, atol=1e-11)
    torch.testing.assert_close(last_c, last, rtol=1e-8, atol=1e-11)


@settings(max_examples=15, deadline=None)
@given(T=st.integers(2, 40), split=st.integers(1, 39), seed=st.integers(0, 1000))
def test_chunked_forward_with_carry_equals_full_forward(T, split, seed):
    split = min(split, T - 1)
    torch.manual_seed(seed)
    m = minGRU(8, expansion_factor=1.5).double()
    x = torch.randn(2, T, 8, dtype=torch.float64)
    full, _ = m(x, return_next_prev_hidden=True)
    a, h = m(x[:, :split], return_next_prev_hidden=True)
    b, _ = m(x[:, split:], h, return_next_prev_hidden=True)
    torch.testing.assert_close(torch.cat((a, b), 1), full, rtol=1e-9, atol=1e-11)


@given(x=st.floats(-30, 30))
def test_log_g_is_log_of_g(x):
    t = torch.tensor([x], dtype=torch.float64)
    torch.testing.assert_close(log_g(t).exp(), g(t), rtol=1e-12, atol=1e-300)
