"""The rows layout (a pass's rows as sequences of their own, forks of a shared prefix included): the two kernels against the
oracle and against the reference's own rows kernels, and the engine's rows against one-sequence decodes."""

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from btb_b200 import launcher as L  # noqa: E402
from btb_b200.batch import RowsEngine  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402

from .test_gpu_kernels import _rope_tables, bf, bits, rand_bf  # noqa: E402
from .util import LAYER_STD, lively  # noqa: E402

DEV = "cuda"
s = capi.stream_ptr


def _layout(rng, T, live, cap, forks):
    """a layout of `live` rows (the rest padding): forks share one prefix, else prefixes lie end to end"""
    step, W = int(rng.integers(0, 5)), T
    if forks:
        lens = [int(rng.integers(1, 700))] * live
        offs = [3] * live
    else:
        lens = [int(rng.integers(1, 400)) for _ in range(live)]
        offs = [3 + sum(lens[:b]) for b in range(live)]
    base = 3 + (lens[0] if forks else sum(lens)) + 5
    assert base + (step + 1) * W <= cap
    rw = [base, step, W]
    for b in range(live):
        rw += [b, offs[b], lens[b]]
    rw += [0, 0, -1] * (T - live)
    return np.asarray(rw, np.int32)


@pytest.mark.parametrize("D,Hq,Hk,T,live,forks,win", [(128, 8, 2, 4, 4, True, 0), (128, 8, 2, 8, 5, False, 0),
                                                     (64, 8, 1, 2, 2, True, 128), (128, 32, 8, 16, 9, False, 0),
                                                     (128, 4, 4, 1, 1, True, 0)])  # fmt: skip
def test_rows_kernels_equal_the_oracle_and_the_reference_s(D, Hq, Hk, T, live, forks, win):
    from . import refkernels

    rng = np.random.default_rng(D + T + live)
    cap = 4096
    rw = _layout(rng, T, live, cap, forks)
    qkv = rand_bf(rng, (T, (Hq + 2 * Hk) * D))
    wq, wk = rand_bf(rng, (D,)), rand_bf(rng, (D,))
    cos, sin = _rope_tables(D, cap, rng)
    K0, V0 = rand_bf(rng, (cap, Hk, D)), rand_bf(rng, (cap, Hk, D))
    hs, rs, scale = D, Hk * D, float(D**-0.5)
    Ko, Vo = K0.copy(), V0.copy()
    qo = O.norm_rope_kv_rows(qkv, wq, wk, 1e-6, cos, sin, rw, Ko, Vo, Hq, Hk, D, hs, rs)
    want = O.attn_decode_rows(qo, Ko, Vo, rw, Hq, Hk, D, hs, rs, scale, win)
    S = cap // 512
    rwt = torch.from_numpy(rw).to(DEV)
    keep = [bf(qkv), bf(wq), bf(wk), bf(cos), bf(sin)]
    res = {}
    launchers = {"b200": L.B200Launcher()}
    if refkernels.available():
        launchers["ref"] = refkernels.RefLauncher()
    p = lambda t: t.data_ptr()  # noqa: E731
    for name, lz in launchers.items():
        Kt, Vt, qt = bf(K0), bf(V0), torch.zeros(T, Hq, D, dtype=torch.bfloat16, device=DEV)
        out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=DEV)
        pm = torch.zeros(S * T * Hq, dtype=torch.float32, device=DEV)
        pl = torch.zeros_like(pm)
        pa = torch.zeros(S * T * Hq * D, dtype=torch.float32, device=DEV)
        cnt = torch.zeros(T * Hq, dtype=torch.int32, device=DEV)
        G = Hq // Hk
        for _ in range(2):  # twice: the arrival counters must come back to zero
            L.btb_norm_rope_kv_rows(lz, D, (Hq + 2 * Hk, T, 1), (32, 1, 1), p(keep[0]), p(keep[1]), p(keep[2]), 1e-6,
                                    p(keep[3]), p(keep[4]), p(rwt), p(Kt), p(Vt), p(qt), T, Hq, Hk, hs, rs, 0)  # fmt: skip
            L.btb_attn_flash_rows(lz, D, (T * ((G + 7) // 8), S, Hk), (256, 1, 1), p(qt), p(Kt), p(Vt), p(out), p(rwt), T, Hq,
                                  Hk, hs, rs, scale, p(pm), p(pl), p(pa), p(cnt), win)  # fmt: skip
            torch.cuda.synchronize()
        assert int(cnt.abs().sum()) == 0
        res[name] = (bits(Kt), bits(Vt), bits(qt)[:live], out.float().cpu().numpy()[:live])
    assert capi.status() == 0
    Kg, Vg, qg, og = res["b200"]
    assert np.array_equal(Vg, Vo)  # the value rows are copies: at their steps' cache rows, nothing else touched

    def close(a, b, rel):
        a, b = O.bits_to_f32(a), O.bits_to_f32(b)
        assert np.max(np.abs(a - b)) <= rel * max(1.0, float(np.max(np.abs(b))))

    close(qg, qo[:live], 5e-3)  # rsqrtf on the card against the host's 1/sqrt: a bf16 step at most
    close(Kg, Ko, 5e-3)
    ref = O.bits_to_f32(want)[:live]
    assert np.max(np.abs(og - ref)) <= 2.0**-6 * max(1.0, float(np.max(np.abs(ref))))
    if "ref" in res:
        Kr, Vr, qr, orr = res["ref"]
        assert np.array_equal(Kg, Kr) and np.array_equal(Vg, Vr) and np.array_equal(qg, qr)  # bits
        assert np.max(np.abs(og - orr)) <= 2.0**-6 * max(1.0, float(np.max(np.abs(orr))))


def test_a_rows_row_equals_the_one_sequence_kernels():
    """row t of a rows pass computes the bits the plain kernels compute for that sequence alone (its keys gathered into
    a cache of its own): what makes a fork's or a batch's tokens its own decode's"""
    rng = np.random.default_rng(5)
    D, Hq, Hk, T, cap = 128, 8, 2, 4, 2048
    rw = _layout(rng, T, 3, cap, False)
    rw[1] = 3
    hs, rs, scale = D, Hk * D, float(D**-0.5)
    q = rand_bf(rng, (T, Hq, D))
    K, V = rand_bf(rng, (cap, Hk, D)), rand_bf(rng, (cap, Hk, D))
    S = cap // 512

    def run(name, qq, KK, VV, extra, rows):
        out = torch.zeros(rows, Hq * D, dtype=torch.bfloat16, device=DEV)
        pm = torch.zeros(S * rows * Hq, dtype=torch.float32, device=DEV)
        pa = torch.zeros(S * rows * Hq * D, dtype=torch.float32, device=DEV)
        cnt = torch.zeros(rows * Hk, dtype=torch.int32, device=DEV)
        keep = [bf(qq), bf(KK), bf(VV)]
        if name == "rows":
            call("btb_b200_attn_decode_rows", ptr(keep[0]), ptr(keep[1]), ptr(keep[2]), ptr(out), ptr(extra), rows, Hq, Hk, D,
                 hs, rs, scale, ptr(pm), ptr(pm), ptr(pa), ptr(cnt), 0, 0, cap, s())  # fmt: skip
        else:
            n0t, par = extra
            call("btb_b200_attn_decode", ptr(keep[0]), ptr(keep[1]), ptr(keep[2]), ptr(out), ptr(n0t), ptr(par), rows, Hq, Hk,
                 D, hs, rs, scale, ptr(pm), ptr(pm), ptr(pa), ptr(cnt), 0, 0, 0, cap, s())  # fmt: skip
        return bits(out)

    got = run("rows", q, K, V, torch.from_numpy(rw).to(DEV), T)
    for t in range(3):
        m = O.rows_map(rw, t)
        Kc, Vc = np.zeros_like(K), np.zeros_like(V)
        Kc[: len(m)], Vc[: len(m)] = K[m], V[m]
        n0t = torch.tensor([len(m) - 1], dtype=torch.int32, device=DEV)
        par = torch.tensor([-1], dtype=torch.int32, device=DEV)
        one = run("plain", q[t : t + 1], Kc, Vc, (n0t, par), 1)
        assert np.array_equal(one[0], got[t]), t
    assert not got[3].any()  # padding: nothing computed


def test_rows_refuse_a_layout_outside_the_cache():
    D, Hq, Hk, T, cap = 128, 2, 1, 1, 64
    z = torch.zeros(T, (Hq + 2 * Hk) * D, dtype=torch.bfloat16, device=DEV)
    tab = torch.zeros(cap, D, dtype=torch.bfloat16, device=DEV)
    K = torch.zeros(cap, Hk, D, dtype=torch.bfloat16, device=DEV)
    q = torch.zeros(T, Hq, D, dtype=torch.bfloat16, device=DEV)
    rw = torch.tensor([cap - 1, 1, 1, 0, 0, 10], dtype=torch.int32, device=DEV)  # step 1 lands at cache row cap
    call("btb_b200_norm_rope_kv_rows", ptr(z), 0, 0, 1e-6, ptr(tab), ptr(tab), ptr(rw), ptr(K), ptr(K), ptr(q), T, Hq, Hk, D,
         D, Hk * D, 0, cap, s())  # fmt: skip
    torch.cuda.synchronize()
    assert capi.status() == capi.ERR_DOMAIN
    assert capi.status() == 0
    with pytest.raises(capi.NativeError):
        call("btb_b200_norm_rope_kv_rows", ptr(z), 0, 0, 1e-6, ptr(tab), ptr(tab), 0, ptr(K), ptr(K), ptr(q), T, Hq, Hk, D,
             D, Hk * D, 0, cap, s())  # fmt: skip


SMALL = E.DenseConfig("rows-small", hidden=256, layers=3, q_heads=4, kv_heads=2, head_dim=128, inter=512, vocab=2048)


def test_forks_and_batches_decode_their_own_sequences():
    """B forks of a prompt, each after a first token of its own, and a batch of prompts end to end: every row's greedy
    tokens are the plain engine's for that sequence - the rows' logits its logits to the bit"""
    mw = E.synth_weights(SMALL, seed=4, layer_std=LAYER_STD)
    prompt = torch.randint(0, SMALL.vocab, (70,), generator=torch.Generator().manual_seed(1))
    plain = E.CardEngine(mw, cap=1024)
    eng = RowsEngine(mw, cap=1024)
    last = eng.fork(prompt, 5)
    firsts = torch.topk(last[0].float(), 5).indices.tolist()  # the five best first tokens: five different continuations
    got = eng.generate_rows(firsts, 12)
    seqs = []
    for b, f in enumerate(firsts):
        plain.reset()
        plain.prefill(prompt)
        want = [f]
        for _ in range(11):
            want.append(plain.step(want[-1]))
        assert got[b] == want, (b, got[b], want)
        seqs.append(want)
    assert len({tuple(q) for q in seqs}) == 5
    lively(seqs[0])
    # a batch: prompts of different lengths end to end; one step's logits against the plain engine's, bit for bit
    prompts = [torch.randint(0, SMALL.vocab, (n,), generator=torch.Generator().manual_seed(n)) for n in (40, 9, 130)]
    lasts = eng.batch(prompts)
    toks = [int(x[0].float().argmax()) for x in lasts]
    lg = bits(eng.rows_step(toks))
    for b, pr in enumerate(prompts):
        plain.reset()
        pl = plain.prefill(pr)
        assert np.array_equal(bits(pl), bits(lasts[b]))
        one = plain.forward(torch.tensor([toks[b]]))
        assert np.array_equal(bits(one)[0], lg[b]), b
