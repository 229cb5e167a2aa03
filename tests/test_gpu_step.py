"""The whole-step kernel against the separate launches: same program, one kernel - every buffer bit-identical."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from .util import LAYER_STD, lively  # noqa: E402

CFG = E.DenseConfig("step-small", hidden=512, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=1280, vocab=2048)


def same(a: torch.Tensor, b: torch.Tensor) -> bool:
    return torch.equal(a.contiguous().view(torch.int16), b.contiguous().view(torch.int16))


@pytest.fixture(scope="module")
def pair():
    mw = E.synth_weights(CFG, seed=5, on_cpu=True, layer_std=LAYER_STD)
    one = E.CardEngine(mw, cap=1024, step_kernel=True)
    many = E.CardEngine(mw, cap=1024, step_kernel=False)
    assert one.step_kernel
    return one, many


def _prefill_both(one, many, prompt):
    for e in (one, many):
        e.reset()
        e.prefill(prompt)


@pytest.mark.parametrize("M,T", [(1, 1), (2, 2), (2, 1)])
def test_pass_is_bit_identical_to_separate_launches(pair, M, T):
    one, many = pair
    prompt = torch.arange(3, 3 + 70) % CFG.vocab
    _prefill_both(one, many, prompt)
    ids = torch.tensor([17, 900][:T])
    ref = many.forward(ids).clone()
    g = one.bufs(M)
    g["ids"][:T].copy_(ids)
    g["depth"][:M].copy_(torch.arange(M, dtype=torch.int32))
    g["par"][:M].copy_(torch.arange(-1, M - 1, dtype=torch.int32))
    one.program(M, 1, pick=False, publish=False).launch(T=T)
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert same(g["logits"][:T], ref)
    assert int(one.n0[0]) == int(many.n0[0]) == 70 + T
    for i in range(CFG.layers):
        assert same(one.K[i][: 70 + T], many.K[i][: 70 + T]) and same(one.V[i][: 70 + T], many.V[i][: 70 + T])


def test_greedy_loop_tokens_and_multi_step_launch(pair):
    one, many = pair
    prompt = torch.arange(100, 140)
    want = many.generate_greedy(prompt, 14)
    lively(want)
    got = one.generate_greedy(prompt, 14)
    assert got == want
    # four steps a launch: the kernel feeds its own pick back through the embedding
    one.reset()
    last = one.prefill(prompt)
    g = one.bufs(1)
    g["ids"][0] = int(last.float().argmax(-1))
    prog = one.program(1, 4, pick=True, publish=True)
    toks = [int(g["ids"][0])]
    for _ in range(3):
        prog.launch()
        torch.cuda.synchronize()
        toks += prog.tok_out.tolist()
        assert int(one.pin_tok[0]) == toks[-1]
    assert toks == want[:13]
    assert capi.status() == 0


def test_packed_weights_through_the_step_kernel():
    cfg = E.DenseConfig("step-p12", hidden=512, layers=2, q_heads=8, kv_heads=2, head_dim=128, inter=1024, vocab=1024)
    a = E.CardEngine(E.synth_weights(cfg, seed=3, on_cpu=True, layer_std=LAYER_STD), cap=512, step_kernel=False)
    b = E.CardEngine(E.synth_weights(cfg, seed=3, on_cpu=True, layer_std=LAYER_STD, storage="p12"), cap=512, step_kernel=True)
    ids = torch.arange(7, 40)
    want = a.generate_greedy(ids, 12)
    lively(want)
    assert want == b.generate_greedy(ids, 12)
    assert capi.status() == 0


def test_a_raised_abort_flag_ends_the_kernel_with_a_status(pair):
    """the bail-out path without a hang: with the abort flag already up every CTA leaves at its first grid barrier,
    the status word says so, and the context stays usable"""
    one, _ = pair
    prog = one.program(1, 1, pick=True, publish=False)
    n_before = int(one.n0[0])
    prog.state.zero_()
    prog.state[1] = 1
    import ctypes as C

    capi.call("btb_b200_step", C.byref(prog.args), prog.M, prog.D, prog.G, capi.stream_ptr())
    torch.cuda.synchronize()
    assert capi.status() == capi.ERR_TIMEOUT
    assert int(one.n0[0]) == n_before  # the step did not complete, nothing advanced
    # and the device still works
    x = torch.ones(8, device="cuda")
    assert float(x.sum()) == 8.0
    assert capi.status() == 0
