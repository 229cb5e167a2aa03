"""Speculative decode over n-gram trees: the in-place commit of the accepted branch and the loop's contract that its
tokens are the plain greedy loop's (btb/engine/generate.py:682-795, btb/engine/cuda.py:3535-3575)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from .util import LAYER_STD, lively  # noqa: E402
from btb_b200 import moe as MO  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402
from btb_b200.draft import generate_speculative  # noqa: E402


@pytest.mark.parametrize("path", [[0], [0, 1, 2], [0, 2, 5, 7], [0, 3], [0, 1, 4, 8, 30]])
def test_commit_gathers_the_path_in_every_layer(path):
    L, cap, Hk, D, n0 = 3, 96, 2, 64, 17
    g = torch.Generator(device="cuda").manual_seed(len(path))
    K = torch.randn(L, cap, Hk, D, generator=g, device="cuda").bfloat16()
    V = torch.randn(L, cap, Hk, D, generator=g, device="cuda").bfloat16()
    K0, V0 = K.clone(), V.clone()
    n0t = torch.tensor([n0], dtype=torch.int32, device="cuda")
    pt = torch.tensor(path, dtype=torch.int32, device="cuda")
    call("btb_b200_kv_commit", ptr(K), ptr(V), K[0].numel(), L, ptr(n0t), ptr(pt), len(path), Hk * D, Hk * D, 0, cap,
         capi.stream_ptr())  # fmt: skip
    torch.cuda.synchronize()
    for A, A0 in ((K, K0), (V, V0)):
        want = A0.clone()
        for j, p in enumerate(path):
            want[:, n0 + j] = A0[:, n0 + p]
        # rows the path did not land on keep what they held
        assert torch.equal(A[:, : n0 + len(path)], want[:, : n0 + len(path)])
        keep = [s for s in range(n0 + len(path), cap)]
        assert torch.equal(A[:, keep], A0[:, keep])
    assert int(n0t.item()) == n0


def test_commit_refuses_a_path_that_is_not_parents_first():
    K = torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16, device="cuda")
    V = torch.zeros_like(K)
    n0t = torch.zeros(1, dtype=torch.int32, device="cuda")
    pt = torch.tensor([0, 2, 1], dtype=torch.int32, device="cuda")
    capi.status()
    call("btb_b200_kv_commit", ptr(K), ptr(V), K[0].numel(), 1, ptr(n0t), ptr(pt), 3, 64, 64, 0, 64, capi.stream_ptr())
    torch.cuda.synchronize()
    assert capi.status() == capi.ERR_DOMAIN
    with pytest.raises(capi.NativeError):
        call("btb_b200_kv_commit", ptr(K), ptr(V), K[0].numel(), 1, ptr(n0t), ptr(pt), 40, 64, 64, 0, 64, 0)


SMALL = E.DenseConfig("small", hidden=256, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=1000)


def _pattern_prompt(vocab, n=48, period=12, seed=0):
    rng = np.random.default_rng(seed)
    pat = rng.integers(0, vocab, size=period)
    return [int(pat[i % period]) for i in range(n)]


@pytest.mark.parametrize("budget", [1, 4, 8, 31])
def test_speculative_tokens_are_the_greedy_tokens(budget):
    eng = E.CardEngine(E.synth_weights(SMALL, seed=0, on_cpu=True, layer_std=LAYER_STD), cap=1024)
    prompt = _pattern_prompt(SMALL.vocab)
    want = eng.generate_greedy(prompt, 80)
    lively(want)
    got, stats = generate_speculative(eng, prompt, 80, budget=budget)
    assert got == want
    assert stats["passes"] <= 79
    # the cache is left as the greedy loop leaves it: one more plain step gives the same token
    nxt = eng.step(got[-1])
    eng.generate_greedy(prompt, 80)
    assert nxt == eng.step(want[-1])


def test_speculative_accepts_drafts_on_text_that_repeats():
    eng = E.CardEngine(E.synth_weights(SMALL, seed=3, on_cpu=True, layer_std=LAYER_STD), cap=1024)
    prompt = _pattern_prompt(SMALL.vocab, seed=5)
    want = eng.generate_greedy(prompt, 120)
    lively(want)
    # feed the model its own continuation as the prompt's tail: the n-grams now predict what it will say
    got, stats = generate_speculative(eng, prompt + want[:60], 60, budget=8)
    assert got == eng.generate_greedy(prompt + want[:60], 60)
    assert stats["passes"] >= 1


def test_speculative_equals_greedy_in_a_moe_model():
    cfg = MO.MoEConfig("m2", 256, 2, 8, 2, 128, 128, 512, experts=16, top_k=4, router_mode=0, glu_kind=0,
                       expert_fmt="fp8")  # fmt: skip
    eng = MO.MoEEngine(MO.synth_moe_weights(cfg, seed=2, on_cpu=True, layer_std=LAYER_STD), cap=512)
    prompt = _pattern_prompt(cfg.vocab, seed=2)
    want = eng.generate_greedy(prompt, 48)
    lively(want)
    got, _ = generate_speculative(eng, prompt, 48, budget=8)
    assert got == want
