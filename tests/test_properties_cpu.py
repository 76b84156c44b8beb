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


def test_ownership_maps_are_bijections():
    """Round-robin chunk ownership and contiguous shards: (owner, local index) enumerates every rank's compact state
    exactly once, and matches the view the Python side uses to initialise it."""
    from gruboros_b200.parallel.dp import DataParallel as DP
    for world in (2, 3, 4, 8):
        for own in (-4, -6, None):
            chunk = 1 << (-own) if own else 0
            n = world * (chunk or 40) * 3
            desc = own if own else n // world
            seen = {}
            for idx in range(n):
                key = (DP.owner_of(idx, desc, world), DP.local_index(idx, desc, world))
                assert key not in seen and 0 <= key[0] < world and 0 <= key[1] < n // world
                seen[key] = idx
            assert len(seen) == n
            if own:
                flat = torch.arange(n)
                for r in range(world):
                    mine = flat.view(-1, world, chunk)[:, r].reshape(-1)
                    assert [seen[(r, j)] for j in range(n // world)] == mine.tolist()
