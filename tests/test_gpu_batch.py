"""Small-batch decode: B sequences side by side give, each, the tokens the one-sequence engine gives for its prompt
(the kernels are row-invariant and row b reads sequence b's cache)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from btb_b200.batch import BatchEngine  # noqa: E402

SMALL = E.DenseConfig("small", hidden=256, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=1000)


@pytest.mark.parametrize("B,storage", [(8, "bf16"), (3, "bf16"), (8, "p12"), (1, "bf16")])
def test_batch_tokens_equal_each_sequences_own_greedy_tokens(B, storage):
    mw = E.synth_weights(SMALL, seed=0, on_cpu=True, storage=storage)
    rng = np.random.default_rng(B)
    prompts = [rng.integers(0, SMALL.vocab, size=int(n)).tolist() for n in rng.integers(5, 70, size=B)]
    one = E.CardEngine(mw, cap=512)
    want = [one.generate_greedy(p, 12) for p in prompts]
    be = BatchEngine(mw, B, cap=512)
    got = be.generate_batch(prompts, 12)
    assert got == want
    assert capi.status() == 0
    # the lengths advanced together: prompt + 11 decoded rows each
    assert be.n0b.tolist() == [len(p) + 11 for p in prompts]
