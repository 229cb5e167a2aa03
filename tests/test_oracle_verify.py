"""The oracle's restatement of the verify pass's pick against outcomes the reference's own `Verify.pick_torch` produced
(tests/golden/verify.npz, made by tests/golden/make_golden.py): every packed outcome - accepted slot and token - equal."""

import os

import numpy as np

from oracle import oracle as O

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "verify.npz"))
N_CASES = 6


def test_every_outcome_is_the_reference_s():
    total = rejected = 0
    for ci in range(N_CASES):
        lg, q, P = GOLD[f"v{ci}/logits"], GOLD[f"v{ci}/q"], GOLD[f"v{ci}/params"]
        for i in range(len(GOLD[f"v{ci}/out"])):
            want = GOLD[f"v{ci}/out"][i]
            got = O.sample_verify(lg, q, GOLD[f"v{ci}/kids"][i], GOLD[f"v{ci}/hasq"][i], GOLD[f"v{ci}/keys"][i], P[0],
                                  int(P[1]), P[2])  # fmt: skip
            assert np.array_equal(got, want), (ci, i, got, want)
            total += len(want)
            rejected += int(((want >> 24) == 0).sum())
    assert total > 3000 and rejected > 300  # the residual draw is exercised, not only the first trial


def test_an_outcome_is_a_child_or_a_token_of_the_row():
    ci = 4
    lg, q = GOLD[f"v{ci}/logits"], GOLD[f"v{ci}/q"]
    for i in range(50):
        kids, out = GOLD[f"v{ci}/kids"][i], GOLD[f"v{ci}/out"][i]
        for r in range(lg.shape[0]):
            slot, tok = (int(out[r]) >> 24) - 1, int(out[r]) & 0xFFFFFF
            assert 0 <= tok < lg.shape[1]
            if slot >= 0:
                assert kids[r][slot] == tok and (not GOLD[f"v{ci}/hasq"][i][r] or q[r][tok] > 0)


def test_refusals():
    import pytest

    x = np.zeros((1, 8), np.float32)
    with pytest.raises(O.OracleError):
        O.sample_verify(x, np.zeros((1, 8), np.float32), np.zeros((1, 33), np.int32), [1], [1], 1.0)
