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
from .util import LAYER_STD, lively  # noqa: E402
from btb_b200.batch import BatchEngine  # noqa: E402

SMALL = E.DenseConfig("small", hidden=256, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=1000)


@pytest.mark.parametrize("B,storage", [(8, "bf16"), (3, "bf16"), (8, "p12"), (1, "bf16")])
def test_batch_tokens_equal_each_sequences_own_greedy_tokens(B, storage):
    mw = E.synth_weights(SMALL, seed=0, on_cpu=True, layer_std=LAYER_STD, storage=storage)
    rng = np.random.default_rng(B)
    prompts = [rng.integers(0, SMALL.vocab, size=int(n)).tolist() for n in rng.integers(5, 70, size=B)]
    one = E.CardEngine(mw, cap=512)
    want = [one.generate_greedy(p, 12) for p in prompts]
    for w in want:
        lively(w)
    be = BatchEngine(mw, B, cap=512)
    got = be.generate_batch(prompts, 12)
    assert got == want
    assert capi.status() == 0
    # the lengths advanced together: prompt + 11 decoded rows each
    assert be.n0b.tolist() == [len(p) + 11 for p in prompts]


def test_tensor_core_passes_agree_with_the_chain_passes_to_rounding():
    """with wide_tc a pass of several rows takes the tensor-core matvec: its logits agree with the fp32-chain pass's
    to bf16 rounding carried through the layers, and a one-row step is untouched"""
    mw = E.synth_weights(SMALL, seed=1, on_cpu=True, layer_std=LAYER_STD)
    a, b = E.CardEngine(mw, cap=512), E.CardEngine(mw, cap=512)
    b.wide_tc = True
    ids = torch.arange(9, 41)
    la, lb = a.forward(ids).float(), b.forward(ids).float()
    assert float((la - lb).abs().max()) <= 2.0**-5 * float(la.abs().max())
    assert float((la.argmax(-1) == lb.argmax(-1)).float().mean()) >= 0.9
    one_a, one_b = a.forward(torch.tensor([5])), b.forward(torch.tensor([5]))
    # the step itself runs the same kernels either way; its inputs (the prefilled cache) differ by rounding
    assert float((one_a.float() - one_b.float()).abs().max()) <= 2.0**-5 * float(one_a.float().abs().max())


def test_batch_engine_on_tensor_cores():
    mw = E.synth_weights(SMALL, seed=0, on_cpu=True, layer_std=LAYER_STD)
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, SMALL.vocab, size=int(n)).tolist() for n in rng.integers(5, 70, size=8)]
    be = BatchEngine(mw, 8, cap=512)
    be.wide_tc = True
    got = be.generate_batch(prompts, 12)
    assert capi.status() == 0
    assert got == be.generate_batch(prompts, 12)  # the same tokens every run
    one = E.CardEngine(mw, cap=512)
    want = [one.generate_greedy(p, 12) for p in prompts]
    same = sum(g[:4] == w[:4] for g, w in zip(got, want))
    assert same >= 6  # another summation order: equal except where two logits sit within rounding of each other
