"""generate(): prompt in parallel, then step by step with carried state (CPU module path)."""
import io

import torch

from gruboros_b200.models.minlm import minLM
from gruboros_b200.runtime.generation import generate, sample
from tests.test_model_cpu import randomize, zipf_bytes


def test_greedy_generation_equals_recomputing_the_whole_prefix():
    torch.manual_seed(0)
    model = minLM(num_tokens=256, dim=64, depth=2)
    randomize(model, 3)
    prompt = zipf_bytes(1, 9)
    out = io.StringIO()
    got = generate(model, prompt, 7, temperature=0.0, device="cpu", stream=True, out=out)
    assert got.shape == (1, 7) and "GENERATED" in out.getvalue()
    seq = prompt.long()
    with torch.no_grad():
        for i in range(7):
            nxt = model(seq)[:, -1].argmax(-1, keepdim=True)          # no cache: full forward over the prefix
            assert int(nxt) == int(got[0, i])
            seq = torch.cat([seq, nxt], dim=1)


def test_sample_filters():
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0]])
    assert int(sample(logits, temperature=0.0)) == 3
    torch.manual_seed(0)
    picks = {int(sample(logits, temperature=1.0, top_k=2)) for _ in range(50)}
    assert picks <= {2, 3}
    picks = {int(sample(logits, temperature=1.0, top_p=0.5)) for _ in range(50)}
    assert picks == {3}            # the first token alone already exceeds p = 0.5 of the mass (0.64)
