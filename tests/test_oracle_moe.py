"""The oracle's MoE pieces against values made by running the reference's own source (tests/golden/make_golden.py `moe`:
btb/engine/host.py `_Router.forward`, `_Experts._act / gpt_oss_gate / _silu_gate / _down`, and
btb/engine/families/qwen4/router.py `Qwen4Router.forward`), and the oracle's gpt-oss model against the reference's banked
receipts for its tiny gpt-oss fixture (tests/fixtures/receipts_gpt_oss.pt: transformers' f32 forward)."""

import os

import numpy as np
import pytest

from oracle import model as OM
from oracle import oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def gold():
    O.build()
    return np.load(os.path.join(HERE, "golden", "moe.npz"))


@pytest.mark.parametrize("tag,E,k", [("a", 32, 4), ("b", 128, 8), ("c", 8, 2)])
@pytest.mark.parametrize("mode", [0, 1])
def test_router_picks_and_weights(gold, tag, E, k, mode):
    lg = gold[f"route_{tag}_logits"]
    idx, w = O.moe_route(lg, E, k, mode)
    assert np.array_equal(idx, gold[f"route_{tag}_m{mode}_idx"])  # the picks and their order: exact
    # the weights: libm's expf here against torch's; at most one bf16 step, nearly all equal
    d = np.abs(w.astype(np.int32) - gold[f"route_{tag}_m{mode}_w"].astype(np.int32))
    assert d.max() <= 1 and (d == 0).mean() >= 0.95


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("biased", [0, 1])
def test_gated_activation_in_the_row_dtype(gold, kind, biased):
    gu = gold["act_gu"]
    bias = gold["act_bias_gu"][gold["act_rows"]] if biased else None
    got = O.f32_to_bits(O.moe_act(gu, kind, bias, 1.702, 7.0))
    want = gold[f"act_k{kind}_b{biased}"]
    d = np.abs(O.bits_to_f32(got) - O.bits_to_f32(want))
    # exp differs between libm and torch in the last ulp: a bf16 step on a few elements at most
    step = np.abs(O.bits_to_f32(want)) * 2.0**-7 + 1e-30
    assert (d <= step).all() and (got == want).mean() >= 0.98


@pytest.mark.parametrize("biased", [0, 1])
def test_down_rounding_bias_weight_and_ordered_sum(gold, biased):
    got = O.moe_combine(gold["comb_dn"], gold["comb_idx"], gold["comb_w"], gold["act_bias_dn"] if biased else None)
    assert np.array_equal(got, gold[f"comb_b{biased}"])  # no transcendental here: bit for bit


def test_tiny_gpt_oss_receipts():
    """the reference's banked receipts for its tiny gpt-oss checkpoint, reproduced by the oracle's f32 composition of the
    same pieces (router top-k then softmax, MXFP4 experts as stored through the 16-lane GEMV, clamped GLU, sums in
    ascending expert order; attention with sinks, sliding windows and YaRN rotary): prompt logits, the logits after a
    continuation over the kept cache, and the ten greedy tokens, within the reference's own 1e-5"""
    O.build()
    t = np.load(os.path.join(HERE, "golden", "tiny_gpt_oss.npz"))
    m = OM.GptOssF32.from_fixture(t)
    prompt, cont = t["rc/prompt"].tolist(), t["rc/cont"].tolist()
    lg = m.forward(prompt)
    assert np.max(np.abs(lg[-1] - t["rc/prompt_logits"])) <= 1e-5
    nx = m.forward(cont)
    assert np.max(np.abs(nx[-1] - t["rc/next"])) <= 1e-5
    m2 = OM.GptOssF32.from_fixture(t)
    assert m2.greedy(prompt, 10) == t["rc/greedy"].tolist()
