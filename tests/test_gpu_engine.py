"""The card engine (embed -> layers -> head -> pick, step graph, greedy loop) against the oracle's card-path
composition on small seeded models, and its own invariants at the benchmark's shapes."""

import json
import os

import numpy as np
import pytest
import torch

from oracle import model as OM
from oracle import oracle as O

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from .util import LAYER_STD, lively, oracle_trace, same_tokens_or_near_tie  # noqa: E402


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def oracle_weights(mw: E.ModelWeights) -> OM.Weights:
    c = mw.cfg
    oc = OM.DenseCfg(c.hidden, c.layers, c.q_heads, c.kv_heads, c.head_dim, c.inter, c.vocab, c.theta, c.eps, c.qk_norm)
    D = c.head_dim
    t = {"model.embed_tokens.weight": bits(mw.embed), "model.norm.weight": bits(mw.norm)}
    for i, L in enumerate(mw.layers):
        qkv, gu = bits(L.qkv), bits(L.gu)
        nq, nk = c.q_heads * D, c.kv_heads * D
        p = f"model.layers.{i}."
        t[p + "self_attn.q_proj.weight"], t[p + "self_attn.k_proj.weight"] = qkv[:nq], qkv[nq : nq + nk]
        t[p + "self_attn.v_proj.weight"] = qkv[nq + nk :]
        t[p + "self_attn.o_proj.weight"] = bits(L.o)
        t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"] = gu[: c.inter], gu[c.inter :]
        t[p + "mlp.down_proj.weight"] = bits(L.down)
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = bits(L.ln1), bits(L.ln2)
        if c.qk_norm:
            t[p + "self_attn.q_norm.weight"], t[p + "self_attn.k_norm.weight"] = bits(L.wq), bits(L.wk)
    return OM.Weights(oc, t)


SMALL = E.DenseConfig("small", hidden=256, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=1000)


@pytest.fixture(scope="module")
def small():
    mw = E.synth_weights(SMALL, seed=0, on_cpu=True, layer_std=LAYER_STD)
    eng = E.CardEngine(mw, cap=1024)
    return mw, eng


def _close_logits(got_bits, want_bits, what):
    got, want = O.bits_to_f32(got_bits), O.bits_to_f32(want_bits)
    tol = 2.0**-6 * max(1.0, float(np.max(np.abs(want))))  # attention's bound carried to the logits
    assert np.max(np.abs(got - want)) <= tol, (what, float(np.max(np.abs(got - want))), tol)


def test_passes_track_the_oracle(small):
    mw, eng = small
    ow = oracle_weights(mw)
    orc = OM.CardPath(ow, cap=eng.cap, tables=(bits(eng.cos), bits(eng.sin)))
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, SMALL.vocab, size=45)
    eng.reset()
    for a in range(0, 45, 32):
        lg = eng.forward(torch.from_numpy(prompt[a : a + 32]))
        want = orc.forward(prompt[a : a + 32].tolist())
        _close_logits(bits(lg), want, f"prefill rows {a}")
    # the cache rows both sides wrote
    torch.cuda.synchronize()
    for i in range(SMALL.layers):
        dk = np.abs(O.bits_to_f32(bits(eng.K[i][:45])) - O.bits_to_f32(orc.K[i][:45]))
        assert dk.max() <= 2.0**-5, (i, dk.max())
    # a tree pass
    par = [-1, 0, 1, 2, 1, 4, 0, 6]
    depth = [0, 1, 2, 3, 2, 3, 1, 2]
    chunk = rng.integers(0, SMALL.vocab, size=8)
    lg = eng.forward(torch.from_numpy(chunk), depth=depth, parents=par, advance=False)
    want = orc.forward(chunk.tolist(), depth=depth, parents=par)
    _close_logits(bits(lg), want, "tree")
    assert capi.status() == 0


def test_greedy_tokens_equal_the_oracle(small):
    mw, eng = small
    ow = oracle_weights(mw)
    orc = OM.CardPath(ow, cap=eng.cap, tables=(bits(eng.cos), bits(eng.sin)))
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, SMALL.vocab, size=40).tolist()
    got = eng.generate_greedy(prompt, 24)
    want, rows = oracle_trace(orc, prompt, 24)
    lively(want, "the oracle's greedy sequence")
    same_tokens_or_near_tie(got, want, rows, min_equal=8)
    assert capi.status() == 0


def test_a_wrong_but_valid_cache_position_fails_the_token_comparison(small):
    """the token tests can fail: the same decode with the cache one row short after the prompt (every later row written a
    slot early, every position off by one - all in range) no longer passes the comparison against the oracle"""
    mw, eng = small
    ow = oracle_weights(mw)
    orc = OM.CardPath(ow, cap=eng.cap, tables=(bits(eng.cos), bits(eng.sin)))
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, SMALL.vocab, size=40).tolist()
    want, rows = oracle_trace(orc, prompt, 24)
    eng.reset()
    last = eng.prefill(torch.tensor(prompt))
    eng.n0.sub_(1)  # the fault
    bad = eng.continue_from(last[0], 24)
    with pytest.raises(AssertionError):
        same_tokens_or_near_tie(bad, want, rows, min_equal=8)
    assert capi.status() == 0


def test_step_graph_equals_eager_steps_and_verify_rows(small):
    """the reference's card-graph invariants (tests/integration/test_card_graph.py:96-203 of btb): the graph loop's
    tokens are the step-by-step tokens, and row t of a chain pass is bit-equal to the step at its position"""
    mw, eng = small
    rng = np.random.default_rng(2)
    prompt = torch.from_numpy(rng.integers(0, SMALL.vocab, size=33))
    toks = eng.generate_greedy(prompt, 12)
    lively(toks)
    # eager steps
    eng.reset()
    last = eng.prefill(prompt)
    eager = [int(last.float().argmax(-1))]
    step_logits = []
    while len(eager) < 12:
        lg = eng.forward(torch.tensor([eager[-1]]))
        step_logits.append(bits(lg)[0].copy())
        eager.append(int(lg.float().argmax(-1)))
    assert toks == eager
    # the same tokens as one chain pass of T rows: each row's logits are its step's, to the bit
    for T in (2, 9, 4, 11):
        eng.reset()
        eng.prefill(prompt)
        lg = eng.forward(torch.tensor(eager[:T]), advance=False)
        for t in range(T):
            assert np.array_equal(bits(lg)[t], step_logits[t]), (T, t)
    # two steps a graph give the same tokens as one
    eng.reset()
    last = eng.prefill(prompt)
    g1 = eng.bufs(1)
    g1["ids"][0] = eager[0]
    graph2 = eng.step_graph(2, publish=True)
    out = [eager[0]]
    for _ in range(5):
        graph2.replay()
        torch.cuda.synchronize()
        out.append(int(eng.pin_tok[0]))
    assert out[1:] == eager[2:12:2]


def test_public_step_call(small):
    mw, eng = small
    prompt = torch.arange(10, 30)
    toks = eng.generate_greedy(prompt, 6)
    lively(toks)
    eng.reset()
    last = eng.prefill(prompt)
    t = int(last.float().argmax(-1))
    got = [t]
    for _ in range(5):
        t = eng.step(t)
        got.append(t)
    assert got == toks


def test_folded_kernels_change_no_bit(small):
    """the norm folded into the GEMV and the SwiGLU fold are the separate kernels' arithmetic: same logits, bit for bit"""
    mw, eng = small
    plain = E.CardEngine(mw, cap=eng.cap, silu_fold=False, fuse_norm=False)
    ids = torch.arange(100, 107)
    for T in (1, 3, 7):
        eng.reset()
        plain.reset()
        a, b = eng.forward(ids[:T]), plain.forward(ids[:T])
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), T
        assert torch.equal(eng.bufs(E.pad_rows(T))["h"][:T].view(torch.int16),
                           plain.bufs(E.pad_rows(T))["h"][:T].view(torch.int16))


def test_p12_model_equals_bf16_model_bits():
    """config 2's requirement: the packed store's logits are the bf16 store's, bit for bit"""
    cfg = E.DenseConfig("small-p12", hidden=256, layers=2, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=512)
    a = E.CardEngine(E.synth_weights(cfg, seed=3, on_cpu=True, layer_std=LAYER_STD), cap=512)
    b = E.CardEngine(E.synth_weights(cfg, seed=3, on_cpu=True, layer_std=LAYER_STD, storage="p12"), cap=512)
    ids = torch.arange(7, 27)
    la, lb = a.forward(ids), b.forward(ids)
    assert torch.equal(la.view(torch.int16), lb.view(torch.int16))
    want = a.generate_greedy(ids, 12)
    lively(want)
    assert want == b.generate_greedy(ids, 12)


def test_tiny_qwen3_fixture_on_the_card(golden_dir):
    """the reference's tiny Qwen3 fixture through the card engine: same top token as its banked (CPU, f32) receipts"""
    tiny = np.load(os.path.join(golden_dir, "tiny_qwen3.npz"))
    cfgj = json.loads(tiny["config"].tobytes())
    cfg = E.DenseConfig("tiny", cfgj["hidden_size"], cfgj["num_hidden_layers"], cfgj["num_attention_heads"],
                        cfgj["num_key_value_heads"], cfgj["head_dim"], cfgj["intermediate_size"], cfgj["vocab_size"],
                        cfgj["rope_parameters"]["rope_theta"], cfgj["rms_norm_eps"])  # fmt: skip

    def w(name):
        a = tiny["w/" + name]
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).cuda()

    mw = E.ModelWeights(cfg, w("model.embed_tokens.weight"), w("model.norm.weight"))
    for i in range(cfg.layers):
        p = f"model.layers.{i}."
        mw.layers.append(E.LayerWeights(
            w(p + "input_layernorm.weight"), w(p + "post_attention_layernorm.weight"),
            torch.cat([w(p + "self_attn.q_proj.weight"), w(p + "self_attn.k_proj.weight"),
                       w(p + "self_attn.v_proj.weight")]).contiguous(),
            w(p + "self_attn.o_proj.weight"),
            torch.cat([w(p + "mlp.gate_proj.weight"), w(p + "mlp.up_proj.weight")]).contiguous(),
            w(p + "mlp.down_proj.weight"), w(p + "self_attn.q_norm.weight"), w(p + "self_attn.k_norm.weight")))  # fmt: skip
    eng = E.CardEngine(mw, cap=512)
    prompt = tiny["rc/prompt"].tolist()
    lg = eng.forward(torch.tensor(prompt))
    ref = tiny["rc/bf16/prompt_logits"]
    got = lg[-1].float().cpu().numpy()
    assert np.max(np.abs(got - ref)) <= 0.05 * np.max(np.abs(ref))
    assert int(np.argmax(ref)) == int(np.argmax(got))
    assert eng.generate_greedy(prompt, 10) == tiny["rc/bf16/greedy"].tolist()


def test_session_feed_mark_rewind_equal_a_fresh_decode():
    """btb's session surface over the card engine: a fed draft's logits are the pass's rows, a rewind drops exactly the
    rows after the mark, and decoding on from a rewound session gives the tokens a fresh prompt gives"""
    from btb_b200.session import State

    mw = E.synth_weights(SMALL, seed=3, layer_std=LAYER_STD)
    eng = E.CardEngine(mw, cap=512)
    prompt = torch.randint(0, SMALL.vocab, (45,), generator=torch.Generator().manual_seed(2)).tolist()
    want = eng.generate_greedy(torch.tensor(prompt), 12)
    lively(want)
    s = eng.session()
    st = s.feed(prompt)
    assert st.logits.shape == (45, SMALL.vocab) and s.state is State.READY
    assert int(st.logits[-1].argmax()) == want[0]
    m = s.mark()
    wrong = [(t + 1) % SMALL.vocab for t in want[:5]]
    s.feed(wrong)  # a draft the target rejects
    s.rewind(m)
    assert len(s) == 45 and int(eng.n0) == 45
    assert s.generate(12) == want and s.state is State.PENDING
    # on from the pending token: the same as one longer decode
    more = s.generate(4)
    assert want + more == eng.generate_greedy(torch.tensor(prompt), 16)
    # crop back into the prompt and feed the rest again: the same logits as the first feed's
    s2 = eng.session()
    first = s2.feed(prompt).logits.clone()
    s2.crop(20)
    again = s2.feed(prompt[20:]).logits
    assert torch.equal(again, first[20:])
