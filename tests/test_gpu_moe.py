"""The MoE block on the card against the oracle: router (both orders), the 16-lane matvecs over bf16 / MXFP4 / FP8 as
stored (bit-equal to the CPU tier's GEMV), the gated activations, the ordered sum, and small MoE models end to end."""

import numpy as np
import pytest
import torch

from oracle import model as OM
from oracle import oracle as O

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import moe as MO  # noqa: E402
from .util import LAYER_STD, lively, oracle_trace, same_tokens_or_near_tie  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402

DEV = "cuda"


def s():
    return capi.stream_ptr()


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.fixture(autouse=True)
def clean_status():
    yield
    torch.cuda.synchronize()
    assert capi.status() == 0


@pytest.mark.parametrize("E,k,mode", [(32, 4, 1), (128, 8, 0), (8, 2, 0), (300, 5, 1), (1024, 8, 0), (2048, 6, 0), (1500, 3, 1)])
@pytest.mark.parametrize("f32", [True, False])
def test_router(E, k, mode, f32):
    rng = np.random.default_rng(E + k)
    T = 5
    lg = rng.standard_normal((T, E)).astype(np.float32) * 2
    lg[0, 3] = lg[0, 7]  # a tie: the lower index first
    if not f32:
        lgb = O.f32_to_bits(lg)
        want_idx, want_w = O.moe_route(lgb, E, k, mode)
        lt = torch.from_numpy(lgb.view(np.int16)).view(torch.bfloat16).to(DEV)
    else:
        want_idx, want_w = O.moe_route(lg, E, k, mode)
        lt = torch.from_numpy(lg).to(DEV)
    idx = torch.zeros(T, k, dtype=torch.int32, device=DEV)
    w = torch.zeros(T, k, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_moe_route", ptr(lt), E, E, k, mode, int(f32), ptr(idx), ptr(w), T, s())
    assert np.array_equal(idx.cpu().numpy(), want_idx)  # the picks are integers: exact
    d = bits(w).astype(np.int32) - want_w.astype(np.int32)
    assert np.max(np.abs(d)) <= 1  # expf on the card against libm: at most one bf16 step


def _mx4(rng, n, R, C_):
    return (rng.integers(0, 256, size=(n, R, C_ // 32, 16), dtype=np.uint8),
            rng.integers(117, 130, size=(n, R, C_ // 32), dtype=np.uint8))


def _fp8(rng, n, R, C_, sr, sc):
    w = rng.integers(0, 256, size=(n, R, C_), dtype=np.uint8)
    w[(w & 0x7F) == 0x7F] = 0x33
    sc_ = O.bits_to_f32(O.f32_to_bits(rng.standard_normal((n, sr, sc)).astype(np.float32) * 0.02))
    return w, sc_


@pytest.mark.parametrize("R,C_", [(64, 128), (300, 2880), (5, 96)])
def test_lane16_gemvs_equal_the_cpu_tier_bits(R, C_):
    rng = np.random.default_rng(R + C_)
    M = 3
    x = rng.standard_normal((M, C_)).astype(np.float32)
    xt = torch.from_numpy(x).to(DEV)
    y = torch.zeros(M, R, dtype=torch.float32, device=DEV)
    wb = O.f32_to_bits(rng.standard_normal((R, C_)).astype(np.float32) * 0.02)
    wt = torch.from_numpy(wb.view(np.int16)).to(DEV)
    call("btb_b200_gemv_lane16_f32", ptr(wt), ptr(xt), ptr(y), M, R, C_, s())
    assert np.array_equal(y.cpu().numpy().view(np.uint32), O.cpu_gemv_bf16(wb, x).view(np.uint32))
    blocks, scales = _mx4(rng, 1, R, C_)
    bt, st = torch.from_numpy(blocks[0]).to(DEV), torch.from_numpy(scales[0]).to(DEV)
    call("btb_b200_gemv_lane16_mx4_f32", ptr(bt), ptr(st), ptr(xt), ptr(y), M, R, C_, s())
    assert np.array_equal(y.cpu().numpy().view(np.uint32), O.cpu_gemv_mxfp4(blocks[0], scales[0], R, C_, x).view(np.uint32))
    if R % 1 == 0 and C_ % 32 == 0:
        sr, sc = (2 if R % 2 == 0 else 1), (C_ // 32)
        w8, s8 = _fp8(rng, 1, R, C_, sr, sc)
        w8t, s8t = torch.from_numpy(w8[0]).to(DEV), torch.from_numpy(s8[0]).to(DEV)
        call("btb_b200_gemv_lane16_fp8_f32", ptr(w8t), ptr(s8t), sr, sc, ptr(xt), ptr(y), M, R, C_, s())
        assert np.array_equal(y.cpu().numpy().view(np.uint32), O.cpu_gemv_fp8(w8[0], s8[0], R, C_, x).view(np.uint32))


def test_mx4_lane16_every_byte_every_scale():
    """all 256 bytes under all 256 scales through the card's widen (x = 1 at one column a row isolates a weight)"""
    blocks = np.broadcast_to(np.arange(256, dtype=np.uint8)[None, :, None], (256, 256, 16)).copy().reshape(256 * 256, 1, 16)
    scales = np.broadcast_to(np.arange(256, dtype=np.uint8)[:, None], (256, 256)).copy().reshape(256 * 256, 1)
    R = 256 * 256
    want = O.widen_mxfp4(blocks.reshape(R, 16), scales.reshape(R), R, 32)
    bt, st = torch.from_numpy(blocks).to(DEV), torch.from_numpy(scales).to(DEV)
    for col in (0, 1, 17):
        x = np.zeros((1, 32), np.float32)
        x[0, col] = 1.0
        xt = torch.from_numpy(x).to(DEV)
        y = torch.zeros(1, R, dtype=torch.float32, device=DEV)
        call("btb_b200_gemv_lane16_mx4_f32", ptr(bt), ptr(st), ptr(xt), ptr(y), 1, R, 32, s())
        got, ref = y.cpu().numpy()[0], want[:, col]
        # rows whose other weights overflow (scale 2^128) turn the zero columns into NaN: compare where the whole row
        # is finite - every byte under every scale up to 2^127 * 6's reach - as bits, and NaN-ness elsewhere
        fin = np.isfinite(want).all(axis=1)
        assert fin.sum() > 250 * 256
        assert np.array_equal(got[fin].view(np.uint32) & 0x7FFFFFFF, ref[fin].view(np.uint32) & 0x7FFFFFFF)


def test_fp8_stream_every_byte_many_scales():
    """all 256 e4m3 bytes under scales of every size and sign through the streaming kernel's widen, on the mixed-precision
    path (x = 1 at one column isolates a weight): the held bf16 the reference's codec makes, to the bit"""
    scales = np.asarray([1.0, -1.0, 0.0123, 3.3e-5, 7e-20, 1.7e-38, 9.1e-41, 448.0, 2.0**100, 3e36, -6.02e-3, 0.33333334],
                        np.float32)  # fmt: skip
    S, C_ = len(scales), 32
    R = 256 * S
    w = np.zeros((R, C_), np.uint8)
    w[:, :] = 0x38  # 1.0 elsewhere: finite
    byte = np.tile(np.arange(256, dtype=np.uint8), S)
    sc = np.repeat(scales, 256).reshape(R, 1)
    for col in (0, 3, 18):
        ww = w.copy()
        ww[:, col] = byte
        full = O.bits_to_f32(O.widen_fp8(ww, sc, R, C_))
        want = full[:, col]
        x = np.zeros((1, C_), np.float32)
        x[0, col] = 1.0
        wt, st_, xt = torch.from_numpy(ww).to(DEV), torch.from_numpy(sc).to(DEV), torch.from_numpy(x).to(DEV)
        y = torch.zeros(1, R, dtype=torch.float32, device=DEV)
        call("btb_b200_moe_gemv", 2, ptr(wt), ptr(st_), 0, 0, R, 1, 0, 1, 1, ptr(xt), 1, ptr(y), R, C_, 0, 1, s())
        got = y.cpu().numpy()[0]
        fin = np.isfinite(full).all(axis=1)
        assert fin.sum() > 240 * S
        assert np.array_equal((got[fin] + np.float32(0)).view(np.uint32), (want[fin] + np.float32(0)).view(np.uint32))
        assert np.isnan(got[np.isnan(want)]).all()


@pytest.mark.parametrize("kind", [0, 1])
def test_act_and_combine(kind):
    rng = np.random.default_rng(kind)
    n, I, H, k, T = 8, 96, 160, 4, 2
    gu = (rng.standard_normal((n, 2 * I)) * 3).astype(np.float32)
    gt, ht = torch.from_numpy(gu).to(DEV), torch.zeros(n, I, dtype=torch.float32, device=DEV)
    call("btb_b200_moe_act", ptr(gt), ptr(ht), 0, 0, n, I, kind, 1.702, 7.0, s())
    want = O.moe_act(gu, kind)
    got = ht.cpu().numpy()
    d = O.f32_to_bits(got).astype(np.int32) - O.f32_to_bits(want).astype(np.int32)
    assert np.max(np.abs(d)) <= (1 if kind == 0 else 2) and np.mean(d != 0) < 5e-3
    dn = rng.standard_normal((T, k, H)).astype(np.float32)
    idx = np.array([[5, 1, 7, 3], [0, 9, 2, 4]], np.int32)
    w = O.f32_to_bits(rng.uniform(0.1, 0.4, size=(T, k)).astype(np.float32))
    y = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    keep = [torch.from_numpy(dn).to(DEV), torch.from_numpy(idx).to(DEV), torch.from_numpy(w.view(np.int16)).to(DEV)]
    call("btb_b200_moe_combine", ptr(keep[0]), ptr(keep[1]), ptr(keep[2]), 0, ptr(y), T, k, H, s())
    assert np.array_equal(bits(y), O.moe_combine(dn, idx, w))  # bf16 adds and multiplies are exact arithmetic


def _oracle_of(mw: MO.MoEWeights, eng) -> OM.MoECardPath:
    c = mw.cfg
    oc = OM.MoECfg(c.hidden, c.layers, c.q_heads, c.kv_heads, c.head_dim, c.inter, c.vocab, c.theta, c.eps, c.qk_norm,
                   c.experts, c.top_k, c.router_mode, c.glu_kind, c.expert_fmt, c.alpha, c.limit)
    layers = []
    for L in mw.layers:
        def stack(st):
            return (st.fmt, st.w.cpu().numpy() if st.fmt != "bf16" else bits(st.w),
                    None if st.scales is None else st.scales.cpu().numpy())
        def dense(W):  # the attention linears as the card holds an FP8 store's: bf16(e4m3 * scale)
            if hasattr(W, "scales"):
                return O.widen_fp8(W.w.cpu().numpy(), W.scales.cpu().numpy(), W.rows, W.cols)
            return bits(W)
        layers.append({"ln1": bits(L.ln1), "ln2": bits(L.ln2), "qkv": dense(L.qkv), "o": dense(L.o), "router": bits(L.router),
                       "wq": None if L.wq is None else bits(L.wq), "wk": None if L.wk is None else bits(L.wk),
                       "gu": stack(L.gu), "dn": stack(L.dn)})
    return OM.MoECardPath(oc, bits(mw.embed), bits(mw.norm), layers, cap=eng.cap, tables=(bits(eng.cos), bits(eng.sin)))


SMALL = {
    "gpt-oss-like": MO.MoEConfig("m1", 256, 2, 8, 2, 64, 128, 512, theta=150000.0, eps=1e-5, qk_norm=False, experts=8,
                                 top_k=2, router_mode=1, glu_kind=1, expert_fmt="mx4"),
    "qwen-moe-like": MO.MoEConfig("m2", 256, 2, 8, 2, 128, 128, 512, experts=16, top_k=4, router_mode=0, glu_kind=0,
                                  expert_fmt="fp8"),
    "qwen-moe-fp8-dense": MO.MoEConfig("m3", 256, 2, 8, 2, 128, 128, 512, experts=16, top_k=4, router_mode=0, glu_kind=0,
                                       expert_fmt="fp8", dense_fmt="fp8"),
}


@pytest.mark.parametrize("name", list(SMALL))
def test_moe_model_tracks_the_oracle(name):
    cfg = SMALL[name]
    mw = MO.synth_moe_weights(cfg, seed=1, on_cpu=True, layer_std=LAYER_STD)
    eng = MO.MoEEngine(mw, cap=512)
    orc = _oracle_of(mw, eng)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab, size=20)
    lg = eng.forward(torch.from_numpy(prompt))
    want = orc.forward(prompt.tolist())
    got_f, want_f = O.bits_to_f32(bits(lg)), O.bits_to_f32(want)
    assert np.max(np.abs(got_f - want_f)) <= 2.0**-6 * max(1.0, float(np.max(np.abs(want_f))))
    # one more row: the step after the prompt
    lg1 = eng.forward(torch.tensor([7]))
    w1 = orc.forward([7])
    assert np.max(np.abs(O.bits_to_f32(bits(lg1)) - O.bits_to_f32(w1))) <= 2.0**-6 * max(1.0, float(np.max(np.abs(O.bits_to_f32(w1)))))
    want, rows = oracle_trace(_oracle_of(mw, eng), prompt.tolist(), 16)
    lively(want, "the oracle's greedy sequence")
    same_tokens_or_near_tie(eng.generate_greedy(prompt.tolist(), 16), want, rows)


def test_verify_rows_equal_steps_in_a_moe_model():
    cfg = SMALL["qwen-moe-like"]
    eng = MO.MoEEngine(MO.synth_moe_weights(cfg, seed=2, on_cpu=True, layer_std=LAYER_STD), cap=512)
    prompt = torch.arange(5, 30)
    toks = eng.generate_greedy(prompt, 6)
    lively(toks)
    eng.reset()
    eng.prefill(prompt)
    steps = []
    for t in toks[:5]:
        steps.append(bits(eng.forward(torch.tensor([t])))[0].copy())
    eng.reset()
    eng.prefill(prompt)
    lg = bits(eng.forward(torch.tensor(toks[:5]), advance=False))
    for t in range(5):
        assert np.array_equal(lg[t], steps[t]), t


# ---- the picked experts' matvecs through the streaming kernel ------------------------------------------------------


@pytest.mark.parametrize("R,C_,n,k", [(1536, 2048, 8, 8), (2048, 768, 8, 1), (5760, 2880, 4, 4), (2880, 2880, 4, 1),
                                      (300, 2880, 5, 1), (13, 96, 3, 3), (64, 128, 40, 8), (8, 32, 1, 1)])  # fmt: skip
@pytest.mark.parametrize("fmt", ["bf16", "mx4", "fp8"])
@pytest.mark.parametrize("xbf", [False, True])
def test_expert_gemv_stream_equals_the_cpu_tier_bits(R, C_, n, k, fmt, xbf):
    """task i multiplies expert idx[i] with x row i // x_div: every output the oracle's 16-lane sum to the bit - for any
    f32 x, and for an x of bf16 values (what the engine's experts are given), which the kernel multiplies on the
    mixed-precision fma"""
    rng = np.random.default_rng(R + C_ + n)
    E = 6
    idx = rng.integers(0, E, size=n).astype(np.int32)
    x = rng.standard_normal(((n + k - 1) // k, C_)).astype(np.float32)
    if xbf:
        x = O.bfround(x * np.float32(3.0))
        x[0, : min(8, C_)] = np.asarray([0.0, -0.0, 1e-38, -3e38, 2.0**-130, 1.0, -1.0, 65280.0], np.float32)[: min(8, C_)]
        x = O.bfround(x)
    xt, it = torch.from_numpy(x).to(DEV), torch.from_numpy(idx).to(DEV)
    y = torch.full((n, R), 7.0, dtype=torch.float32, device=DEV)
    if fmt == "bf16":
        wb = O.f32_to_bits(rng.standard_normal((E, R, C_)).astype(np.float32) * 0.02)
        wt = torch.from_numpy(wb.view(np.int16)).to(DEV)
        args = (0, ptr(wt), 0, R * C_ * 2, 0, 1, 1)
        want = [O.cpu_gemv_bf16(wb[idx[i]], x[i // k : i // k + 1])[0] for i in range(n)]
    elif fmt == "mx4":
        blocks, scales = _mx4(rng, E, R, C_)
        bt, st = torch.from_numpy(blocks).to(DEV), torch.from_numpy(scales).to(DEV)
        args = (1, ptr(bt), ptr(st), R * C_ // 2, R * C_ // 32, 1, 1)
        want = [O.cpu_gemv_mxfp4(blocks[idx[i]], scales[idx[i]], R, C_, x[i // k : i // k + 1])[0] for i in range(n)]
    else:
        sr = next(d for d in (12, 8, 4, 2, 1) if R % d == 0)
        sc = C_ // 128 if C_ % 128 == 0 else C_ // 32
        w8, s8 = _fp8(rng, E, R, C_, sr, sc)
        wt, st = torch.from_numpy(w8).to(DEV), torch.from_numpy(s8).to(DEV)
        args = (2, ptr(wt), ptr(st), R * C_, sr * sc * 4, sr, sc)
        want = [O.cpu_gemv_fp8(w8[idx[i]], s8[idx[i]], R, C_, x[i // k : i // k + 1])[0] for i in range(n)]
    f, w, sc_, ws, ss, sr_, scn = args
    call("btb_b200_moe_gemv", f, w, sc_, ws, ss, sr_, scn, ptr(it), n, E, ptr(xt), k, ptr(y), R, C_, 0, 1, s())
    got = y.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), np.stack(want).view(np.uint32))
    # the plain 16-lane kernel gives the same bits
    capi.set_tuning(moe_stream=0)
    try:
        y2 = torch.zeros_like(y)
        call("btb_b200_moe_gemv", f, w, sc_, ws, ss, sr_, scn, ptr(it), n, E, ptr(xt), k, ptr(y2), R, C_, 0, 1, s())
        assert torch.equal(y2.view(torch.int32), y.view(torch.int32))
    finally:
        capi.set_tuning(moe_stream=1)
    # expert parallel: a rank's own experts, zeros for the others'; the ranks' sum is the whole
    parts = []
    for rank in range(2):
        yp = torch.full((n, R), 3.0, dtype=torch.float32, device=DEV)
        Wl = w  # expert e of rank r is global expert 2 e + r: the test hands each rank a strided view
        call("btb_b200_moe_gemv", f, Wl + rank * ws, (sc_ + rank * ss) if sc_ else 0, 2 * ws, 2 * ss, sr_, scn, ptr(it), n, E,
             ptr(xt), k, ptr(yp), R, C_, rank, 2, s())  # fmt: skip
        parts.append(yp)
    tot = parts[0] + parts[1]
    assert torch.equal(tot.view(torch.int32), y.view(torch.int32))
    assert all(bool((parts[int(idx[i]) % 2 ^ 1][i] == 0).all()) for i in range(n))


@pytest.mark.parametrize("I,C_,n,k", [(768, 2048, 8, 8), (2880, 2880, 4, 4), (20, 96, 3, 1), (100, 64, 5, 5)])
@pytest.mark.parametrize("fmt", ["bf16", "mx4", "fp8"])
@pytest.mark.parametrize("kind", [0, 1])
def test_expert_gate_up_with_the_activation_in_its_epilogue(I, C_, n, k, fmt, kind):
    """btb_b200_moe_gemv_glu: the activated rows are btb_b200_moe_gemv's outputs through btb_b200_moe_act, bit for bit"""
    rng = np.random.default_rng(I + C_ + n + kind)
    E, R = 5, 2 * I
    idx = rng.integers(0, E, size=n).astype(np.int32)
    x = O.bfround(rng.standard_normal(((n + k - 1) // k, C_)).astype(np.float32) * 2)
    xt, it = torch.from_numpy(x).to(DEV), torch.from_numpy(idx).to(DEV)
    if fmt == "bf16":
        wb = O.f32_to_bits(rng.standard_normal((E, R, C_)).astype(np.float32) * 0.05)
        keep = [torch.from_numpy(wb.view(np.int16)).to(DEV)]
        args = (0, ptr(keep[0]), 0, R * C_ * 2, 0, 1, 1)
    elif fmt == "mx4":
        blocks, scales = _mx4(rng, E, R, C_)
        keep = [torch.from_numpy(blocks).to(DEV), torch.from_numpy(scales).to(DEV)]
        args = (1, ptr(keep[0]), ptr(keep[1]), R * C_ // 2, R * C_ // 32, 1, 1)
    else:
        sr = next(d for d in (12, 8, 4, 2, 1) if R % d == 0)
        sc = C_ // 128 if C_ % 128 == 0 else C_ // 32
        w8, s8 = _fp8(rng, E, R, C_, sr, sc)
        keep = [torch.from_numpy(w8).to(DEV), torch.from_numpy(s8).to(DEV)]
        args = (2, ptr(keep[0]), ptr(keep[1]), R * C_, sr * sc * 4, sr, sc)
    f, w, sc_, ws, ss, sr_, scn = args
    y = torch.zeros(n, R, dtype=torch.float32, device=DEV)
    h1 = torch.zeros(n, I, dtype=torch.float32, device=DEV)
    call("btb_b200_moe_gemv", f, w, sc_, ws, ss, sr_, scn, ptr(it), n, E, ptr(xt), k, ptr(y), R, C_, 0, 1, s())
    call("btb_b200_moe_act", ptr(y), ptr(h1), 0, 0, n, I, kind, 1.702, 7.0, s())
    h2 = torch.full((n, I), 5.0, dtype=torch.float32, device=DEV)
    call("btb_b200_moe_gemv_glu", f, w, sc_, ws, ss, sr_, scn, ptr(it), n, E, ptr(xt), k, ptr(h2), R, C_, kind, 1.702, 7.0, 0, 1,
         s())  # fmt: skip
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert torch.equal(h1.view(torch.int32), h2.view(torch.int32))
    assert float(h1.abs().max()) > 0
    # expert parallel: a rank activates its own picks' rows, zeros for the others'
    h3 = torch.full((n, I), 5.0, dtype=torch.float32, device=DEV)
    call("btb_b200_moe_gemv_glu", f, w, sc_ if sc_ else 0, 2 * ws, 2 * ss, sr_, scn, ptr(it), n, E, ptr(xt), k, ptr(h3), R, C_, kind,
         1.702, 7.0, 0, 2, s())  # fmt: skip
    torch.cuda.synchronize()
    for i in range(n):
        if int(idx[i]) % 2 == 0:
            assert torch.equal(h3[i].view(torch.int32), h1[i].view(torch.int32)), i
        else:
            assert not h3[i].any()


@pytest.mark.parametrize("name", list(SMALL))
def test_folded_moe_pass_equals_the_unfolded_pass(name):
    """the activation inside the down matvecs' launch and the picks' sum inside the next norm's change no bit"""
    cfg = SMALL[name]
    mw = MO.synth_moe_weights(cfg, seed=3, on_cpu=True, layer_std=LAYER_STD)
    a, b = MO.MoEEngine(mw, cap=512), MO.MoEEngine(mw, cap=512)
    a.fold, b.fold = True, False
    prompt = torch.arange(7, 40)
    la, lb = a.forward(prompt[:20]), b.forward(prompt[:20])
    assert torch.equal(la.view(torch.int16), lb.view(torch.int16))
    la, lb = a.forward(prompt[20:21]), b.forward(prompt[20:21])
    assert torch.equal(la.view(torch.int16), lb.view(torch.int16))
    assert torch.equal(a.K.view(torch.int16), b.K.view(torch.int16))
    want = b.generate_greedy(prompt, 12)
    lively(want)
    assert a.generate_greedy(prompt, 12) == want


@pytest.mark.parametrize("E,H,k,mode", [(128, 2048, 8, 0), (32, 2880, 4, 1), (8, 256, 2, 0), (300, 512, 5, 1), (1024, 264, 8, 0),
                                        (7, 64, 3, 1)])  # fmt: skip
def test_router_cluster_launch_equals_matvec_then_route(E, H, k, mode):
    """btb_b200_moe_router: the logits are the 16-lane matvec's bits, the picks and weights btb_b200_moe_route's"""
    rng = np.random.default_rng(E + H)
    T = 3
    wb = O.f32_to_bits(rng.standard_normal((E, H)).astype(np.float32) * 0.05)
    x = rng.standard_normal((T, H)).astype(np.float32)
    wt = torch.from_numpy(wb.view(np.int16)).to(DEV)
    xt = torch.from_numpy(x).to(DEV)
    rl_a = torch.zeros(T, E, dtype=torch.float32, device=DEV)
    idx_a, w_a = torch.zeros(T, k, dtype=torch.int32, device=DEV), torch.zeros(T, k, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_lane16_f32", ptr(wt), ptr(xt), ptr(rl_a), T, E, H, s())
    call("btb_b200_moe_route", ptr(rl_a), E, E, k, mode, 1, ptr(idx_a), ptr(w_a), T, s())
    rl_b = torch.zeros_like(rl_a)
    idx_b, w_b = torch.zeros_like(idx_a), torch.zeros_like(w_a)
    call("btb_b200_moe_router", ptr(wt), ptr(xt), ptr(rl_b), E, H, k, mode, ptr(idx_b), ptr(w_b), T, s())
    torch.cuda.synchronize()
    assert np.array_equal(rl_b.cpu().numpy().view(np.uint32), O.cpu_gemv_bf16(wb, x).view(np.uint32))
    assert torch.equal(rl_a.view(torch.int32), rl_b.view(torch.int32))
    assert torch.equal(idx_a, idx_b) and torch.equal(w_a.view(torch.int16), w_b.view(torch.int16))
    idx_c, w_c = torch.zeros_like(idx_a), torch.zeros_like(w_a)
    call("btb_b200_moe_router", ptr(wt), ptr(xt), 0, E, H, k, mode, ptr(idx_c), ptr(w_c), T, s())  # without the logits
    assert torch.equal(idx_a, idx_c) and torch.equal(w_a.view(torch.int16), w_c.view(torch.int16))
    # the block's add + RMSNorm + widen in the router launch's prologue: the bits of the norm's own launch, then the router's
    hb = torch.from_numpy(O.f32_to_bits(rng.standard_normal((T, H)).astype(np.float32)).view(np.int16)).to(DEV)
    yb = torch.from_numpy(O.f32_to_bits(rng.standard_normal((T, H)).astype(np.float32) * 0.3).view(np.int16)).to(DEV)
    nw = torch.from_numpy(O.f32_to_bits(1 + 0.1 * rng.standard_normal(H).astype(np.float32)).view(np.int16)).to(DEV)
    h1, x1, xf1 = hb.clone(), torch.zeros_like(hb), torch.zeros(T, H, dtype=torch.float32, device=DEV)
    call("btb_b200_add_rmsnorm_wide", ptr(h1), ptr(yb), ptr(nw), 1e-6, ptr(x1), ptr(xf1), T, H, 0, s())
    idx_d, w_d, rl_d = torch.zeros_like(idx_a), torch.zeros_like(w_a), torch.zeros_like(rl_a)
    call("btb_b200_moe_router", ptr(wt), ptr(xf1), ptr(rl_d), E, H, k, mode, ptr(idx_d), ptr(w_d), T, s())
    h2, x2, xf2 = torch.zeros_like(hb), torch.zeros_like(hb), torch.zeros_like(xf1)
    idx_e, w_e, rl_e = torch.zeros_like(idx_a), torch.zeros_like(w_a), torch.zeros_like(rl_a)
    call("btb_b200_moe_router_norm", ptr(wt), ptr(hb), ptr(yb), ptr(nw), 1e-6, 0, ptr(h2), ptr(x2), ptr(xf2), ptr(rl_e), E, H,
         k, mode, ptr(idx_e), ptr(w_e), T, s())  # fmt: skip
    torch.cuda.synchronize()
    assert torch.equal(h1, h2) and torch.equal(x1, x2) and torch.equal(xf1.view(torch.int32), xf2.view(torch.int32))
    assert torch.equal(rl_d.view(torch.int32), rl_e.view(torch.int32))
    assert torch.equal(idx_d, idx_e) and torch.equal(w_d.view(torch.int16), w_e.view(torch.int16))
    # the grid form (any router size): the same bits again, its counter left at zero, twice in a row
    cnt = torch.zeros(T, dtype=torch.int32, device=DEV)
    for _ in range(2):
        h3, x3, xf3 = torch.zeros_like(hb), torch.zeros_like(hb), torch.zeros_like(xf1)
        idx_f, w_f, rl_f = torch.zeros_like(idx_a), torch.zeros_like(w_a), torch.zeros_like(rl_a)
        call("btb_b200_moe_router_grid", ptr(wt), ptr(hb), ptr(yb), ptr(nw), 1e-6, 0, ptr(h3), ptr(x3), ptr(xf3), ptr(rl_f),
             ptr(cnt), E, H, k, mode, ptr(idx_f), ptr(w_f), T, s())  # fmt: skip
        torch.cuda.synchronize()
        assert torch.equal(h1, h3) and torch.equal(x1, x3) and torch.equal(xf1.view(torch.int32), xf3.view(torch.int32))
        assert torch.equal(rl_d.view(torch.int32), rl_f.view(torch.int32))
        assert torch.equal(idx_d, idx_f) and torch.equal(w_d.view(torch.int16), w_f.view(torch.int16))
        assert int(cnt.abs().sum()) == 0
    # ... and without the norm: x read as given
    idx_g, w_g, rl_g = torch.zeros_like(idx_a), torch.zeros_like(w_a), torch.zeros_like(rl_a)
    call("btb_b200_moe_router_grid", ptr(wt), 0, 0, 0, 1e-6, 0, 0, 0, ptr(xt), ptr(rl_g), ptr(cnt), E, H, k, mode, ptr(idx_g),
         ptr(w_g), T, s())  # fmt: skip
    torch.cuda.synchronize()
    assert torch.equal(rl_a.view(torch.int32), rl_g.view(torch.int32)) and torch.equal(idx_a, idx_g)
    with pytest.raises(capi.NativeError):  # the new residual may not land in the buffer other CTAs still read
        call("btb_b200_moe_router_norm", ptr(wt), ptr(hb), ptr(yb), ptr(nw), 1e-6, 0, ptr(hb), 0, ptr(xf2), 0, E, H, k, mode,
             ptr(idx_e), ptr(w_e), T, s())  # fmt: skip
