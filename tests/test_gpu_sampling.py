"""The one-launch sampled pick against the oracle: thresholds to the bit, the drawn token wherever the Gumbel race is
not decided inside the last ulps of logf, keys derived on the card, and the engine's sampled loop."""

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from .util import LAYER_STD, lively  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402
from btb_b200.sampling import CardSampler, Sampling  # noqa: E402

TIE = 2e-5  # a race closer than this (relative) may go either way between the host's logf and the card's


def _run(x: torch.Tensor, keys, T, k, p, f32=True):
    R, V = x.shape
    smp = CardSampler("cuda")
    smp.set(Sampling(temperature=T, top_k=k, top_p=p, seed=0))
    out = torch.zeros(R, dtype=torch.int64, device="cuda")
    floors = torch.zeros(R, 2, dtype=torch.int32, device="cuda")
    kd = torch.from_numpy(np.asarray(keys, np.uint64).view(np.int64)).cuda()
    n0 = torch.zeros(1, dtype=torch.int32, device="cuda")
    smp.pick(x, R, n0, None, out, capi.stream_ptr(), keys=kd, floors=floors)
    torch.cuda.synchronize()
    assert capi.status() == 0
    return out.cpu().numpy(), floors.cpu().numpy().view(np.uint32)


CASES = [(1000, 0.8, 40, 0.9), (151936, 0.7, 50, 0.95), (201088, 1.0, 0, 0.8), (128256, 1.3, 8, 1.0), (257, 1.5, 3, 0.5),
         (70, 0.3, 0, 0.99), (7, 1.0, 20, 1.0), (32000, 1.0, 0, 1.0), (50257, 0.05, 0, 0.3)]  # fmt: skip


@pytest.mark.parametrize("V,T,k,p", CASES)
def test_pick_equals_the_oracle(V, T, k, p):
    rng = np.random.default_rng(V)
    R = 5
    x = (rng.standard_normal((R, V)) * 3).astype(np.float32)
    x[1, : V // 2] = x[1, V // 2 : 2 * (V // 2)]  # a row with every value twice: ties at the thresholds
    keys = rng.integers(0, 2**63, size=R, dtype=np.uint64)
    want, wfl, margin = O.sample_pick(x, keys, T, k, p)
    got, gfl = _run(torch.from_numpy(x).cuda(), keys, T, k, p)
    assert np.array_equal(gfl, wfl)
    for r in range(R):
        assert got[r] == want[r] or margin[r] <= TIE * max(1.0, abs(float(x[r].max()) / T)), (r, got[r], want[r], margin[r])
    # bf16 logits are the same pick as their f32 widening
    xb = torch.from_numpy(x).cuda().bfloat16()
    want_b, wfl_b, margin_b = O.sample_pick(xb.float().cpu().numpy(), keys, T, k, p)
    got_b, gfl_b = _run(xb, keys, T, k, p)
    assert np.array_equal(gfl_b, wfl_b)
    assert all(got_b[r] == want_b[r] or margin_b[r] <= TIE * 40 for r in range(R))


def test_special_values_and_strided_rows():
    V = 4096
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((4, V)) * 2).astype(np.float32)
    x[0, ::7] = -np.inf
    x[1, 5] = np.inf
    x[2] = 0.0
    x[2, ::2] = -0.0
    x[3, 100:200] = x[3].max()
    keys = np.arange(4, dtype=np.uint64) + 11
    for T, k, p in ((1.0, 0, 0.9), (0.5, 10, 1.0), (2.0, 64, 0.5)):
        want, wfl, margin = O.sample_pick(x, keys, T, k, p)
        wide = torch.zeros(4, V + 24, device="cuda")
        wide[:, :V] = torch.from_numpy(x).cuda()
        got, gfl = _run(wide[:, :V], keys, T, k, p)  # rows at a stride longer than V
        assert np.array_equal(gfl, wfl), (T, k, p)
        assert all(got[r] == want[r] or margin[r] <= 1e-4 for r in range(4)), (T, k, p, got, want)


def test_key_derived_on_the_card_is_key_for():
    V = 5000
    rng = np.random.default_rng(9)
    x = torch.from_numpy((rng.standard_normal((3, V)) * 3).astype(np.float32)).cuda()
    s = Sampling(temperature=0.9, top_k=0, top_p=1.0, seed=123456789)
    smp = CardSampler("cuda")
    smp.set(s)
    n0 = torch.tensor([4095], dtype=torch.int32, device="cuda")
    depth = torch.tensor([0, 1, 5], dtype=torch.int32, device="cuda")
    out = torch.zeros(3, dtype=torch.int64, device="cuda")
    smp.pick(x, 3, n0, depth, out, capi.stream_ptr())
    keys = np.asarray([s.key_for(4095 + d) for d in (0, 1, 5)], np.uint64)
    assert [int(k) for k in keys] == [O.sample_key(123456789, 4095 + d) for d in (0, 1, 5)]
    want, _, margin = O.sample_pick(x.cpu().numpy(), keys, 0.9)
    got = out.cpu().numpy()
    assert all(got[r] == want[r] or margin[r] <= 1e-4 for r in range(3))


def test_refusals():
    x = torch.zeros(1, 64, device="cuda")
    fp = torch.ones(2, device="cuda")
    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    with pytest.raises(capi.NativeError):  # no keys and no seed
        call("btb_b200_sample_pick", ptr(x), 1, 1, 64, 64, ptr(fp), 0, 0, 0, 0, 0, 0, ptr(out), 0, 0, 0)
    with pytest.raises(capi.NativeError):  # a row too long for a cluster's shared memory
        call("btb_b200_sample_pick", ptr(x), 1, 1, 1 << 20, 1 << 20, ptr(fp), 0, ptr(out), 0, 0, 0, 0, ptr(out), 0, 0, 0)


SMALL = E.DenseConfig("small", hidden=256, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=1000)


def test_engine_sampled_loop_draws_what_the_sequential_keys_draw():
    eng = E.CardEngine(E.synth_weights(SMALL, seed=0, on_cpu=True, layer_std=LAYER_STD), cap=512)
    s = Sampling(temperature=0.8, top_k=40, top_p=0.9, seed=7)
    prompt = list(range(3, 23))
    toks = eng.generate(prompt, 24, s)
    assert toks == eng.generate(prompt, 24, s)  # a seed repeats
    assert toks != eng.generate(prompt, 24, Sampling(temperature=0.8, top_k=40, top_p=0.9, seed=8))
    # teacher-forced: each step's logits through the oracle's pick under key_for(the deciding row)
    eng.set_sampling(Sampling())
    eng.reset()
    lg = eng.prefill(torch.tensor(prompt))
    pos = len(prompt) - 1
    for t in toks:
        want, _, margin = O.sample_pick(lg.float().cpu().numpy(), np.asarray([s.key_for(pos)], np.uint64), 0.8, 40, 0.9)
        assert t == want[0] or margin[0] <= 1e-3, (pos, t, want[0], margin[0])
        lg = eng.forward(torch.tensor([t]))
        pos += 1
    # temperature, top-p and seed are data to the captured graph; greedy comes back as the argmax loop
    hot = eng.generate(prompt, 12, Sampling(temperature=5.0, top_k=40, top_p=1.0, seed=7))
    assert hot != toks[:12]
    got = eng.generate(prompt, 12, Sampling())  # the sampling set back to greedy
    want = eng.generate_greedy(prompt, 12)
    lively(want)
    assert got == want


# ---- the reference's own pipeline, launch by launch, through both launchers --------------------------------------


def _pipeline(launcher, x, seed, n0, T, top_k, top_p):
    """btb's card pick as its host issues it (btb/engine/cuda.py:2158-2220): keys -> max -> radix levels -> draw -> out"""
    import ctypes as C

    from btb_b200 import launcher as L

    R, V = x.shape
    dev = x.device
    z = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)  # noqa: E731
    fp = torch.tensor([1.0 / T, top_p], dtype=torch.float32, device=dev)
    seedt = torch.tensor([seed & 0xFFFFFFFF, seed >> 32], dtype=torch.int64).to(torch.int32).to(dev)
    pos = torch.tensor([n0], dtype=torch.int32, device=dev)
    keys, gM, ghist = z(2, torch.int32), z(R, torch.int32), z(R * 2048, torch.int64)
    gpreK, gpreP, gcarry, gbest = z(R, torch.int32), z(R, torch.int32), z(R, torch.int64), z(R, torch.int64)
    out = z(R, torch.int32)
    nb = min(max(1, (V + 1023) // 1024), 4 * 148)
    p = lambda t: t.data_ptr()  # noqa: E731
    L.btb_sample_keys(launcher, (1, 1, 1), (1, 1, 1), p(seedt), p(pos), 0, p(keys))
    L.btb_sample_max(launcher, (nb, R, 1), (1024, 1, 1), p(x), V, p(fp), p(gM))
    for mode, pre, flo, run in ((0, gpreK, gpreP, top_k > 0), (1, gpreP, gpreK, top_p < 1.0)):
        if not run:
            continue
        for lvl in (0, 1, 2):
            ghist.zero_()
            L.btb_sample_hist(launcher, (nb, R, 1), (1024, 1, 1), p(x), V, p(fp), lvl, mode, p(gM), p(pre), p(flo), p(ghist))
            L.btb_sample_bin(launcher, (R, 1, 1), (1024, 1, 1), lvl, mode, top_k, p(fp), p(ghist), p(pre), p(gcarry))
    L.btb_sample_draw(launcher, (nb, R, 1), (1024, 1, 1), p(x), p(keys), V, p(fp), p(gM), p(gpreK), p(gpreP), p(gbest))
    L.btb_sample_out(launcher, ((R + 255) // 256, 1, 1), (256, 1, 1), p(gbest), p(out), R)
    torch.cuda.synchronize()
    del C
    return out.cpu().numpy().view(np.uint32), keys.cpu().numpy().view(np.uint32), gbest.cpu().numpy()


@pytest.mark.parametrize("V,T,k,p", [(151936, 0.7, 50, 0.95), (32000, 1.0, 0, 0.8), (5000, 1.2, 8, 1.0), (1000, 1.0, 0, 1.0)])
def test_launcher_serves_the_reference_pipeline_and_equals_its_kernels(V, T, k, p):
    from . import refkernels
    from btb_b200 import launcher as L

    rng = np.random.default_rng(V + k)
    x = torch.from_numpy((rng.standard_normal((1, V)) * 3).astype(np.float32)).cuda()
    mine = _pipeline(L.B200Launcher(), x, 0x1234567 << 8, 77, T, k, p)
    key = Sampling(temperature=T, seed=0x1234567 << 8).key_for(77)
    assert int(mine[1][0]) | (int(mine[1][1]) << 32) == key
    want, _, margin = O.sample_pick(x.cpu().numpy(), np.asarray([key], np.uint64), T, k, p)
    assert mine[0][0] == want[0] or margin[0] <= 1e-4
    if not refkernels.available():
        pytest.skip("the reference's kernels are not built (oracle/build_ref.sh)")
    theirs = _pipeline(refkernels.RefLauncher(), x, 0x1234567 << 8, 77, T, k, p)
    assert np.array_equal(mine[1], theirs[1])  # the key
    assert mine[0][0] == theirs[0][0] or margin[0] <= 1e-4  # the token
    if mine[0][0] == theirs[0][0]:
        # the packed winner: the same token, and its raced value to a few ulps (logf is not the same routine)
        a = np.uint64(mine[2][0]).item() >> 32
        b = np.uint64(theirs[2][0]).item() >> 32
        assert abs(a - b) <= 64


# ---- the verify pass's pick (btb_sample_verify) ------------------------------------------------------------------------

import os  # noqa: E402

from btb_b200.sampling import Verify  # noqa: E402

VGOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "verify.npz"))


def _verify(x: torch.Tensor, q, kids, hasq, keys, T, k, p) -> np.ndarray:
    s = Sampling(temperature=float(T), top_k=int(k), top_p=float(p), seed=0)
    v = Verify(s, torch.as_tensor(np.asarray(q)), [[int(c) for c in row if c >= 0] for row in np.asarray(kids)], list(hasq))
    out = v.pick(x, [int(a) for a in keys]).cpu().numpy().astype(np.uint32)
    torch.cuda.synchronize()
    assert capi.status() == 0
    return out


@pytest.mark.parametrize("ci", range(6))
def test_verify_outcomes_are_the_reference_s_and_the_oracle_s(ci):
    """the golden outcomes come from the reference's `Verify.pick_torch`; the oracle equals them (CPU suite)"""
    lg, q, P = VGOLD[f"v{ci}/logits"], VGOLD[f"v{ci}/q"], VGOLD[f"v{ci}/params"]
    x = torch.from_numpy(lg).cuda()
    n = min(len(VGOLD[f"v{ci}/out"]), 120)
    for i in range(n):
        got = _verify(x, q, VGOLD[f"v{ci}/kids"][i], VGOLD[f"v{ci}/hasq"][i], VGOLD[f"v{ci}/keys"][i], P[0], P[1], P[2])
        assert np.array_equal(got, VGOLD[f"v{ci}/out"][i]), (ci, i, got, VGOLD[f"v{ci}/out"][i])


def _verify_case(V, R, width, noise, seed, sampling):
    rng = np.random.default_rng(seed)
    lg = (rng.standard_normal((R, V)) * 3).astype(np.float32)
    dl = lg + (rng.standard_normal((R, V)) * noise).astype(np.float32)
    q = np.exp((dl - dl.max(-1, keepdims=True)) / np.float32(sampling.temperature)).astype(np.float32)
    q[:, V // 2 :] *= (rng.random((R, V - V // 2)) < 0.5)  # a drafter that gives many tokens no mass
    pr = q.astype(np.float64) / q.astype(np.float64).sum(-1, keepdims=True)
    kids = np.stack([rng.choice(V, size=width, replace=False, p=pr[r]) for r in range(R)]).astype(np.int32)
    kids[0, width - 1] = -1  # a ragged row
    hasq = np.asarray([(r % 4) != 3 for r in range(R)], np.uint32)
    keys = rng.integers(0, 2**63, size=R, dtype=np.uint64)
    return lg, q, kids, hasq, keys


@pytest.mark.parametrize("V,R,width,noise", [(151936, 6, 4, 1.5), (32000, 9, 8, 3.0), (201088, 3, 31, 0.5), (70, 16, 5, 2.0)])
def test_verify_equals_the_oracle_at_real_vocabularies(V, R, width, noise):
    s = Sampling(temperature=0.8, top_k=0 if V == 70 else 200, top_p=0.95, seed=0)
    lg, q, kids, hasq, keys = _verify_case(V, R, width, noise, V + R, s)
    want = O.sample_verify(lg, q, kids, hasq, keys, s.temperature, s.top_k, s.top_p)
    got = _verify(torch.from_numpy(lg).cuda(), q, kids, hasq, keys, s.temperature, s.top_k, s.top_p)
    # the trials' sums run in the oracle's order: equal outcomes; only a draw (a race of logf values) may fall inside the
    # last ulps between the host's logf and the card's
    same = got == want
    assert same.mean() >= 0.8 and np.array_equal(got >> 24, want >> 24), (got, want)
    # bf16 logits are the same pick as their f32 widening
    xb = torch.from_numpy(lg).cuda().bfloat16()
    want_b = O.sample_verify(xb.float().cpu().numpy(), q, kids, hasq, keys, s.temperature, s.top_k, s.top_p)
    got_b = _verify(xb, q, kids, hasq, keys, s.temperature, s.top_k, s.top_p)
    assert np.array_equal(got_b >> 24, want_b >> 24) and (got_b == want_b).mean() >= 0.8


@pytest.mark.parametrize("V,R,width,noise", [(151936, 4, 4, 1.5), (5000, 12, 8, 3.0), (12, 16, 5, 1.0)])
def test_verify_through_the_launcher_equals_the_reference_s_kernel(V, R, width, noise):
    from . import refkernels
    from btb_b200 import launcher as L

    if not refkernels.available():
        pytest.skip("the reference's kernels are not built (oracle/build_ref.sh)")
    s = Sampling(temperature=0.9, top_k=0 if V == 12 else 64, top_p=0.9, seed=0)
    lg, q, kids, hasq, keys = _verify_case(V, R, width, noise, 7 * V + R, s)
    dev = "cuda"
    x, qd = torch.from_numpy(lg).to(dev), torch.from_numpy(q).to(dev)
    kd, hd = torch.from_numpy(kids).to(dev), torch.from_numpy(hasq.view(np.int32)).to(dev)
    kk = torch.from_numpy(keys.view(np.int64)).to(dev)
    fp = torch.tensor([1.0 / s.temperature, s.top_p], dtype=torch.float32, device=dev)
    outs = []
    for la in (L.B200Launcher(), refkernels.RefLauncher()):
        out = torch.zeros(R, dtype=torch.int32, device=dev)
        p = lambda t: t.data_ptr()  # noqa: E731
        L.btb_sample_verify(la, (R, 1, 1), (1024, 1, 1), p(x), p(qd), p(kd), p(hd), p(kk), V, V, width, s.top_k, p(fp), p(out))
        torch.cuda.synchronize()
        outs.append(out.cpu().numpy().view(np.uint32))
    assert capi.status() == 0
    assert np.array_equal(outs[0] >> 24, outs[1] >> 24), outs  # the accepted slots
    assert (outs[0] == outs[1]).mean() >= 0.8, outs  # tokens: a residual draw may sit inside logf's last ulps


def test_verify_emits_the_target_distribution():
    """the property that makes drawn-tree speculation exact (the reference's test_the_cuda_verify_follows_the_target): over
    the keys, the emitted token - accepted child or residual draw - follows the target p, whatever the drafter proposed"""
    V, R, n = 12, 4, 1500
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(R, V, generator=g) * 3
    dl = logits + torch.randn(R, V, generator=g) * 0.7
    s = Sampling(temperature=0.8, top_p=0.9, seed=5)
    # the target after temperature and top-p, from the oracle's thresholds
    sc = logits.numpy() * (np.float32(1.0) / np.float32(s.temperature))  # the scaled row as the kernels make it
    _, floors, _ = O.sample_pick(logits.numpy(), np.zeros(R, np.uint64), s.temperature, 0, s.top_p)
    p = np.exp(sc - sc.max(-1, keepdims=True))
    ordered = lambda f: np.where(f.view(np.uint32) >> 31, ~f.view(np.uint32), f.view(np.uint32) | np.uint32(1 << 31))  # noqa: E731
    p = p * (ordered(sc.astype(np.float32)) >= floors[:, 1:2])
    p /= p.sum(-1, keepdims=True)
    qd = torch.softmax(dl / s.temperature, -1)
    x = logits.cuda()
    seen = np.zeros((R, V))
    gq = torch.Generator().manual_seed(1)
    for i in range(n):
        keys = [s.key_for(i * R + r) for r in range(R)]
        kids = torch.multinomial(qd, 6, replacement=False, generator=gq).tolist()  # drafts drawn without replacement from q
        out = Verify(s, qd, kids, [True] * R).pick(x, keys).tolist()
        for r in range(R):
            slot, t = Verify.unpack(out[r])
            assert 0 <= t < V and (slot < 0 or kids[r][slot] == t)
            seen[r][t] += 1
    assert np.abs(seen / n - p).max() < 0.04, (seen / n, p)


def test_verify_refusals():
    x = torch.zeros(1, 64, device="cuda")
    z = torch.zeros(1, 64, device="cuda")
    kids = torch.zeros(1, 40, dtype=torch.int32, device="cuda")
    one = torch.ones(1, dtype=torch.int64, device="cuda")
    fp = torch.ones(2, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = (ptr(x), 1, 1, 64, 64, ptr(z), 64, ptr(kids))
    with pytest.raises(capi.NativeError):  # more children than the kernel's table holds
        call("btb_b200_sample_verify", *a, 40, ptr(one), ptr(one), 0, ptr(fp), ptr(out), capi.stream_ptr())
    with pytest.raises(capi.NativeError):
        call("btb_b200_sample_verify", *a, 4, 0, ptr(one), 0, ptr(fp), ptr(out), capi.stream_ptr())
    with pytest.raises(ValueError):
        Verify(Sampling(temperature=1.0), z, [list(range(33))], [True])
