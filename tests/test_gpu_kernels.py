"""GPU parity tests, through the C-ABI: each kernel against the CPU oracle on seeded inputs and, where the reference's
own card kernels are built (oracle/_ref), against those kernels on the same device, compared as bits."""

import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi, launcher as L  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402

from . import refkernels  # noqa: E402

DEV = "cuda"


def bf(a: np.ndarray) -> torch.Tensor:
    """uint16 bit patterns -> a bf16 tensor on the card"""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).to(DEV)


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def rand_bf(rng, shape, scale=1.0) -> np.ndarray:
    return O.f32_to_bits(rng.standard_normal(shape).astype(np.float32) * np.float32(scale))


def s() -> int:
    return capi.stream_ptr()


@pytest.fixture(scope="module")
def b200():
    return L.B200Launcher()


@pytest.fixture(scope="module")
def ref():
    if not refkernels.available():
        pytest.skip("the reference's kernels are not built (oracle/build_ref.sh)")
    return refkernels.RefLauncher()


@pytest.fixture(autouse=True)
def clean_status():
    yield
    torch.cuda.synchronize()
    assert capi.status() == 0, "a kernel recorded a device-side refusal"


# ---- GEMV --------------------------------------------------------------------------------------------------------

GEMV_SHAPES = [(1, 8), (3, 264), (5, 2880), (149, 512), (300, 2560), (37, 9728), (2, 256), (1184, 1024)]


@pytest.mark.parametrize("R,Cc", GEMV_SHAPES)
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
def test_gemv_bf16_equals_oracle_bits(R, Cc, M):
    rng = np.random.default_rng(R * 131 + Cc + M)
    w, x = rand_bf(rng, (R, Cc), 0.02), rand_bf(rng, (M, Cc))
    wt, xt = bf(w), bf(x)
    y = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_bf16", ptr(wt), ptr(xt), ptr(y), M, R, Cc, s())
    assert np.array_equal(bits(y), O.gemv_card_bf16(w, x))


def test_gemv_rows_are_invariant_to_width():
    rng = np.random.default_rng(5)
    R, Cc = 777, 2560
    w, x = rand_bf(rng, (R, Cc), 0.02), rand_bf(rng, (32, Cc))
    wt, xt = bf(w), bf(x)
    y32 = torch.zeros(32, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_bf16", ptr(wt), ptr(xt), ptr(y32), 32, R, Cc, s())
    for M in (1, 2, 4, 8, 16):
        y = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
        call("btb_b200_gemv_bf16", ptr(wt), ptr(xt), ptr(y), M, R, Cc, s())
        assert torch.equal(y.view(torch.int16), y32[:M].view(torch.int16)), M


@pytest.mark.parametrize("tune", [dict(ring_bytes=32768, seg_bytes=1024), dict(ring_bytes=160 * 1024, seg_bytes=8192),
                                  dict(ctas_per_sm=2, ring_bytes=65536), dict(evict_first=0), dict(x_smem_max=0)])  # fmt: skip
def test_gemv_bits_do_not_depend_on_the_ring_geometry(tune):
    rng = np.random.default_rng(11)
    R, Cc, M = 523, 4096, 4
    w, x = rand_bf(rng, (R, Cc), 0.02), rand_bf(rng, (M, Cc))
    wt, xt = bf(w), bf(x)
    want = O.gemv_card_bf16(w, x)
    dflt = dict(ring_bytes=96 * 1024, seg_bytes=4096, x_smem_max=160 * 1024, ctas_per_sm=1, evict_first=1)
    try:
        capi.set_tuning(**tune)
        y = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
        call("btb_b200_gemv_bf16", ptr(wt), ptr(xt), ptr(y), M, R, Cc, s())
        assert np.array_equal(bits(y), want)
    finally:
        capi.set_tuning(**dflt)


def test_gemv_refuses_bad_arguments():
    w = torch.zeros(4, 16, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(capi.NativeError) as e:
        call("btb_b200_gemv_bf16", 0, ptr(w), ptr(w), 1, 4, 16, s())
    assert e.value.rc == capi.ERR_NULL
    for M, R, Cc in ((3, 4, 16), (1, 0, 16), (1, 4, 12)):
        with pytest.raises(capi.NativeError) as e:
            call("btb_b200_gemv_bf16", ptr(w), ptr(w), ptr(w), M, R, Cc, s())
        assert e.value.rc == capi.ERR_DOMAIN
    with pytest.raises(capi.NativeError):  # misaligned weights
        call("btb_b200_gemv_bf16", ptr(w) + 2, ptr(w), ptr(w), 1, 2, 8, s())


@pytest.mark.parametrize("M", [1, 2, 8])
@pytest.mark.parametrize("R,Cc", [(64, 128), (300, 9728), (5, 2880)])
def test_gemv_silu_fold_equals_two_kernels(M, R, Cc):
    rng = np.random.default_rng(R + M)
    w, gu = rand_bf(rng, (R, Cc), 0.02), rand_bf(rng, (M, 2 * Cc), 1.5)
    wt, gt = bf(w), bf(gu)
    y = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    if M * Cc * 2 > 160 * 1024:  # the activated x does not fit its shared-memory budget: refused, by contract
        with pytest.raises(capi.NativeError) as e:
            call("btb_b200_gemv_silu_bf16", ptr(wt), ptr(gt), ptr(y), M, R, Cc, s())
        assert e.value.rc == capi.ERR_DOMAIN
        return
    call("btb_b200_gemv_silu_bf16", ptr(wt), ptr(gt), ptr(y), M, R, Cc, s())
    m = torch.zeros(M, Cc, dtype=torch.bfloat16, device=DEV)
    y2 = torch.zeros_like(y)
    call("btb_b200_silu_mul", ptr(gt), ptr(m), M, Cc, s())
    call("btb_b200_gemv_bf16", ptr(wt), ptr(m), ptr(y2), M, R, Cc, s())
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    # against the oracle: the card's expf is within 2 ulp of libm's, so after the two bf16 roundings a few activations
    # may sit one bf16 step away; the product sum then moves by far less than the output's own rounding step
    want = O.bits_to_f32(O.gemv_card_silu_bf16(w, gu))
    got = O.bits_to_f32(bits(y))
    assert np.max(np.abs(got - want)) <= 2.0**-7 * max(1.0, float(np.max(np.abs(want))))
    mo = O.silu_mul(gu)
    diff = bits(m).astype(np.int32) - mo.astype(np.int32)
    assert np.max(np.abs(diff)) <= 1 and np.mean(diff != 0) < 1e-3


@pytest.mark.parametrize("M,T", [(1, 1), (4, 3), (8, 8)])
@pytest.mark.parametrize("R,H", [(300, 2560), (64, 264), (1000, 4096)])
@pytest.mark.parametrize("add", [True, False])
def test_gemv_with_norm_prologue_equals_two_kernels(M, T, R, H, add):
    rng = np.random.default_rng(R + H + M)
    w, h0, yv, nw = rand_bf(rng, (R, H), 0.02), rand_bf(rng, (M, H)), rand_bf(rng, (M, H), 0.1), rand_bf(rng, (H,))
    wt, nt = bf(w), bf(nw)
    yt = bf(yv) if add else None
    # two kernels
    h1, x1, y1 = bf(h0), torch.zeros(M, H, dtype=torch.bfloat16, device=DEV), torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_add_rmsnorm", ptr(h1), ptr(yt), ptr(nt), 1e-6, ptr(x1), T, H, 0, s())
    call("btb_b200_gemv_bf16", ptr(wt), ptr(x1), ptr(y1), M, R, H, s())
    # one
    hin, hout, y2 = bf(h0), torch.zeros(M, H, dtype=torch.bfloat16, device=DEV), torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_norm", ptr(wt), 0, 0, 0, 0, 0, ptr(hin), ptr(yt), ptr(nt), 1e-6, 0, ptr(hout) if add else 0,
         ptr(y2), T, M, R, H, s())  # fmt: skip
    assert torch.equal(y1[:T].view(torch.int16), y2[:T].view(torch.int16))
    assert int(y2[T:].float().abs().sum()) == 0  # padding rows multiply zeros
    assert np.array_equal(bits(hin), h0)  # the input residual is left alone
    if add:
        assert torch.equal(h1[:T].view(torch.int16), hout[:T].view(torch.int16))


# ---- pack12 ------------------------------------------------------------------------------------------------------


def test_card_pack12_encoder_writes_the_reference_encoders_bytes(golden_dir):
    """the library's on-card encoder against the parts the reference's own encoder wrote for the same tensors (golden
    fixtures), and against the oracle's restatement on larger seeded tensors whose escapes span many tiles"""
    import os

    from btb_b200 import pack12

    g = np.load(os.path.join(golden_dir, "codecs.npz"))
    cases = [(f"golden {c}", g[f"p12_{c}_src"], [g[f"p12_{c}_{n}"] for n in ("lo", "hi4", "tbl", "esc_idx", "esc_val")])
             for c in "abcd"]  # fmt: skip
    rng = np.random.default_rng(12)
    for R, Cc, dense in ((300, 2560, False), (129, 4097, True), (1, 1, False), (64, 9728, True)):
        f = rng.standard_normal((R, Cc)).astype(np.float32) * 0.02
        if dense:
            f *= np.logspace(-9, 3, Cc, dtype=np.float32)[None, :]
        src = O.f32_to_bits(f)
        cases.append((f"seeded {R}x{Cc}", src, list(O.pack_p12(src))))
    for what, src, want in cases:
        t = torch.from_numpy(src.view(np.int16)).view(torch.bfloat16).to(DEV)
        lo, hi4, table, ei, ev = pack12.pack_bf16(t)
        got = [lo.cpu().numpy(), hi4.cpu().numpy(), np.frombuffer(table, np.uint8), ei.cpu().numpy(), ev.cpu().numpy()]
        for mine, theirs, name in zip(got, want, ("lo", "hi4", "table", "esc_idx", "esc_val")):
            assert np.array_equal(mine, theirs), (what, name)
        assert np.array_equal(O.widen_p12(*got, src.size), src.reshape(-1)), what


def _p12_case(rng, R, Cc, scale_cols=False):
    from btb_b200 import pack12

    f = rng.standard_normal((R, Cc)).astype(np.float32) * 0.02
    if scale_cols:  # many distinct high bytes: escapes everywhere
        f *= np.logspace(-9, 3, Cc, dtype=np.float32)[None, :]
    wb = O.f32_to_bits(f)
    t = torch.from_numpy(wb.view(np.int16)).view(torch.bfloat16)
    lo, hi4, table, ei, ev = pack12.pack_bf16(t)  # the card's encoder; numpy copies for the oracle's arguments
    return wb, (lo.cpu().numpy(), hi4.cpu().numpy(), np.frombuffer(table, np.uint8).copy(), ei.cpu().numpy(), ev.cpu().numpy())


@pytest.mark.parametrize("R,Cc,dense", [(40, 256, False), (300, 2560, False), (64, 9728, False), (33, 512, True),
                                        (7, 4096, True)])  # fmt: skip
@pytest.mark.parametrize("M", [1, 4, 16])
def test_gemv_p12_equals_bf16_gemv_bits(R, Cc, dense, M):
    from btb_b200.engine import P12Matrix

    rng = np.random.default_rng(R + Cc)
    wb, parts = _p12_case(rng, R, Cc, dense)
    if dense:
        assert parts[3].size > R  # the case does exercise escapes
    x = rand_bf(rng, (M, Cc))
    P = P12Matrix(parts, R, Cc, DEV)
    xt = bf(x)
    y = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_p12", ptr(P.lo), ptr(P.hi4), P.table, ptr(P.esc_idx), ptr(P.esc_val), ptr(P.esc_row), ptr(xt),
         ptr(y), M, R, Cc, s())  # fmt: skip
    assert np.array_equal(bits(y), O.gemv_card_bf16(wb, x))
    assert np.array_equal(bits(y), O.gemv_card_p12(*parts, x, R, Cc))
    if M <= 8 and M * Cc * 2 <= 64 * 1024:
        # the folds over packed weights equal the folds over the bf16 matrix
        wt = bf(wb)
        gu, nw = bf(rand_bf(rng, (M, 2 * Cc), 1.5)), bf(rand_bf(rng, (Cc,)))
        ya, yb = torch.zeros_like(y), torch.zeros_like(y)
        call("btb_b200_gemv_silu_bf16", ptr(wt), ptr(gu), ptr(ya), M, R, Cc, s())
        call("btb_b200_gemv_silu_p12", ptr(P.lo), ptr(P.hi4), P.table, ptr(P.esc_idx), ptr(P.esc_val), ptr(P.esc_row),
             ptr(gu), ptr(yb), M, R, Cc, s())  # fmt: skip
        assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))
        call("btb_b200_gemv_norm", ptr(wt), 0, 0, 0, 0, 0, ptr(xt), 0, ptr(nw), 1e-6, 0, 0, ptr(ya), M, M, R, Cc, s())
        call("btb_b200_gemv_norm", ptr(P.lo), ptr(P.hi4), P.table, ptr(P.esc_idx), ptr(P.esc_val), ptr(P.esc_row),
             ptr(xt), 0, ptr(nw), 1e-6, 0, 0, ptr(yb), M, M, R, Cc, s())  # fmt: skip
        assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))


@pytest.mark.parametrize("R,Cc,sr,sc", [(256, 256, 2, 2), (384, 2048, 3, 16), (128, 768, 1, 6), (40, 64, 5, 1)])
@pytest.mark.parametrize("M", [1, 8, 16])
def test_gemv_fp8_equals_bf16_gemv_over_held_weights(R, Cc, sr, sc, M):
    rng = np.random.default_rng(R + Cc + M)
    w8 = rng.integers(0, 256, size=(R, Cc), dtype=np.uint8)
    w8[(w8 & 0x7F) == 0x7F] = 0x2A
    scales = O.bits_to_f32(O.f32_to_bits(rng.standard_normal((sr, sc)).astype(np.float32) * 0.02))
    x = rand_bf(rng, (M, Cc))
    held = O.widen_fp8(w8, scales, R, Cc)
    want = O.gemv_card_bf16(held, x)
    assert np.array_equal(want, O.gemv_card_fp8(w8, scales, x, R, Cc))
    wt, st, xt = torch.from_numpy(w8).to(DEV), torch.from_numpy(scales).to(DEV), bf(x)
    y = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_fp8", ptr(wt), ptr(st), sr, sc, ptr(xt), ptr(y), M, R, Cc, s())
    assert np.array_equal(bits(y), want)


@pytest.mark.parametrize("R,H,sr,sc", [(384, 2048, 3, 16), (5120, 2048, 40, 16), (128, 768, 1, 6)])
@pytest.mark.parametrize("M,T,add", [(1, 1, True), (1, 1, False), (8, 5, True)])
def test_gemv_fp8_with_norm_prologue_equals_two_kernels(R, H, sr, sc, M, T, add):
    rng = np.random.default_rng(R + H + M)
    w8 = rng.integers(0, 256, size=(R, H), dtype=np.uint8)
    w8[(w8 & 0x7F) == 0x7F] = 0x2A
    scales = O.bits_to_f32(O.f32_to_bits(rng.standard_normal((sr, sc)).astype(np.float32) * 0.02))
    h0, yv, nw = rand_bf(rng, (M, H)), rand_bf(rng, (M, H), 0.1), rand_bf(rng, (H,))
    wt, st, nt = torch.from_numpy(w8).to(DEV), torch.from_numpy(scales).to(DEV), bf(nw)
    yt = bf(yv) if add else None
    h1, x1, y1 = bf(h0), torch.zeros(M, H, dtype=torch.bfloat16, device=DEV), torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_add_rmsnorm", ptr(h1), ptr(yt), ptr(nt), 1e-6, ptr(x1), T, H, 0, s())
    call("btb_b200_gemv_fp8", ptr(wt), ptr(st), sr, sc, ptr(x1), ptr(y1), M, R, H, s())
    hin, hout, y2 = bf(h0), torch.zeros(M, H, dtype=torch.bfloat16, device=DEV), torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_norm_fp8", ptr(wt), ptr(st), sr, sc, ptr(hin), ptr(yt), ptr(nt), 1e-6, 0, ptr(hout) if add else 0,
         ptr(y2), T, M, R, H, s())  # fmt: skip
    assert torch.equal(y1[:T].view(torch.int16), y2[:T].view(torch.int16))
    assert np.array_equal(bits(hin), h0)
    if add:
        assert torch.equal(h1[:T].view(torch.int16), hout[:T].view(torch.int16))


# ---- the small kernels -------------------------------------------------------------------------------------------


def _close_bf16(got: np.ndarray, want: np.ndarray, frac: float = 2e-3) -> None:
    """bf16 results of a kernel that uses the card's approximate rsqrt / expf against the oracle's exact ones: never
    more than one bf16 step apart, and only on a small fraction of the elements"""
    d = got.astype(np.int32) - want.astype(np.int32)
    assert np.max(np.abs(d)) <= 1, np.max(np.abs(d))
    assert np.mean(d != 0) <= frac, np.mean(d != 0)


@pytest.mark.parametrize("T,H", [(1, 2560), (5, 64), (32, 2880), (2, 8192)])
def test_add_rmsnorm(T, H):
    rng = np.random.default_rng(T + H)
    h, y, w = rand_bf(rng, (T, H)), rand_bf(rng, (T, H), 0.1), rand_bf(rng, (H,), 1.0)
    for yy in (y, None):
        ht, wt, xt = bf(h), bf(w), torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
        yt = None if yy is None else bf(yy)
        call("btb_b200_add_rmsnorm", ptr(ht), ptr(yt), ptr(wt), 1e-6, ptr(xt), T, H, 0, s())
        h2, x2 = O.add_rmsnorm(h, yy, w, 1e-6)
        assert np.array_equal(bits(ht), h2)  # the residual add is exact arithmetic
        _close_bf16(bits(xt), x2)


def _rope_tables(D, cap, rng):
    ang = rng.uniform(0, 6.28, size=(cap, D)).astype(np.float32)
    return O.f32_to_bits(np.cos(ang)), O.f32_to_bits(np.sin(ang))


@pytest.mark.parametrize("D,Hq,Hk,T,norm,paged", [(128, 4, 2, 1, True, False), (128, 8, 2, 9, True, True),
                                                 (64, 8, 1, 5, False, False), (128, 32, 8, 32, True, False)])  # fmt: skip
def test_norm_rope_kv(D, Hq, Hk, T, norm, paged):
    rng = np.random.default_rng(D + T)
    cap, n0 = 128, 37
    qkv = rand_bf(rng, (T, (Hq + 2 * Hk) * D))
    wq = rand_bf(rng, (D,)) if norm else None
    wk = rand_bf(rng, (D,)) if norm else None
    cos, sin = _rope_tables(D, cap, rng)
    depth = rng.integers(0, 6, size=T).astype(np.int32)
    tbl = rng.permutation(cap).astype(np.int32) if paged else None
    K0, V0 = rand_bf(rng, (cap, Hk, D)), rand_bf(rng, (cap, Hk, D))
    Ko, Vo = K0.copy(), V0.copy()
    qo = O.norm_rope_kv(qkv, wq, wk, 1e-6, cos, sin, n0, depth, Ko, Vo, Hq, Hk, D, D, Hk * D, tbl=tbl)
    Kt, Vt, qt = bf(K0), bf(V0), torch.zeros(T, Hq, D, dtype=torch.bfloat16, device=DEV)
    n0t = torch.tensor([n0], dtype=torch.int32, device=DEV)
    dt = torch.from_numpy(depth).to(DEV)
    tt = None if tbl is None else torch.from_numpy(tbl).to(DEV)
    keep = [bf(qkv), None if wq is None else bf(wq), None if wk is None else bf(wk), bf(cos), bf(sin)]
    call("btb_b200_norm_rope_kv", ptr(keep[0]), ptr(keep[1]), ptr(keep[2]), 1e-6, ptr(keep[3]), ptr(keep[4]), ptr(n0t),
         ptr(dt), ptr(Kt), ptr(Vt), ptr(qt), T, Hq, Hk, D, D, Hk * D, 0, ptr(tt), cap, s())  # fmt: skip
    assert np.array_equal(bits(Vt), Vo)  # a copy
    if norm:
        _close_bf16(bits(qt), qo, 5e-3)
        _close_bf16(bits(Kt), Ko, 5e-3)
    else:
        assert np.array_equal(bits(qt), qo) and np.array_equal(bits(Kt), Ko)  # rope alone is exact arithmetic


def test_norm_rope_kv_refuses_a_row_past_the_cache():
    D, Hq, Hk, T, cap = 128, 2, 1, 2, 16
    z = torch.zeros(T, (Hq + 2 * Hk) * D, dtype=torch.bfloat16, device=DEV)
    tab = torch.zeros(cap, D, dtype=torch.bfloat16, device=DEV)
    K = torch.zeros(cap, Hk, D, dtype=torch.bfloat16, device=DEV)
    q = torch.zeros(T, Hq, D, dtype=torch.bfloat16, device=DEV)
    n0 = torch.tensor([cap - 1], dtype=torch.int32, device=DEV)  # row 1 would land at slot cap
    dp = torch.zeros(T, dtype=torch.int32, device=DEV)
    call("btb_b200_norm_rope_kv", ptr(z), 0, 0, 1e-6, ptr(tab), ptr(tab), ptr(n0), ptr(dp), ptr(K), ptr(K), ptr(q), T,
         Hq, Hk, D, D, Hk * D, 0, 0, cap, s())  # fmt: skip
    torch.cuda.synchronize()
    assert capi.status() == capi.ERR_DOMAIN  # recorded, nothing written out of range, the context lives on
    assert capi.status() == 0


def _attn_case(rng, D, Hq, Hk, n0, T, par, cap, paged=False, win=0, sinks=False):
    hs, rs = D, Hk * D
    q = rand_bf(rng, (T, Hq, D))
    K, V = rand_bf(rng, (cap, Hk, D)), rand_bf(rng, (cap, Hk, D))
    tbl = rng.permutation(cap).astype(np.int32) if paged else None
    sk = rng.standard_normal(Hq).astype(np.float32) if sinks else None
    scale = float(D**-0.5)
    want = O.attn_decode(q, K, V, n0, par, Hq, Hk, D, hs, rs, scale, win, tbl, sk)
    S = (cap + 511) // 512
    qt, Kt, Vt = bf(q), bf(K), bf(V)
    out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=DEV)
    pm = torch.zeros(S * T * Hq, dtype=torch.float32, device=DEV)
    pl = torch.zeros_like(pm)
    pa = torch.zeros(S * T * Hq * D, dtype=torch.float32, device=DEV)
    cnt = torch.zeros(T * Hk, dtype=torch.int32, device=DEV)
    n0t = torch.tensor([n0], dtype=torch.int32, device=DEV)
    pt = torch.from_numpy(np.asarray(par, np.int32)).to(DEV)
    tt = None if tbl is None else torch.from_numpy(tbl).to(DEV)
    st = None if sk is None else torch.from_numpy(sk).to(DEV)
    for _ in range(2):  # twice: the arrival counters must come back to zero
        out.zero_()
        call("btb_b200_attn_decode", ptr(qt), ptr(Kt), ptr(Vt), ptr(out), ptr(n0t), ptr(pt), T, Hq, Hk, D, hs, rs, scale,
             ptr(pm), ptr(pl), ptr(pa), ptr(cnt), win, ptr(tt), ptr(st), cap, s())  # fmt: skip
        got = O.bits_to_f32(bits(out))
        ref = O.bits_to_f32(want)
        # the reference's own bound for its attention against an f32 softmax (tests/kernels/test_card_kernels.py:776-778)
        assert np.max(np.abs(got - ref)) <= 2.0**-6 * max(1.0, float(np.max(np.abs(ref))))
    assert int(cnt.abs().sum()) == 0
    return out


CHAIN = lambda T: list(range(-1, T - 1))  # noqa: E731


@pytest.mark.parametrize("D,Hq,Hk,n0,T,cap", [(128, 4, 1, 0, 1, 512), (128, 8, 2, 100, 1, 512), (128, 32, 8, 255, 1, 1024),
                                              (128, 8, 1, 700, 1, 2048), (64, 16, 2, 1500, 3, 2048),
                                              (128, 8, 2, 511, 4, 1024), (128, 16, 2, 63, 32, 512)])  # fmt: skip
def test_attention_chain(D, Hq, Hk, n0, T, cap):
    _attn_case(np.random.default_rng(n0 + T), D, Hq, Hk, n0, T, CHAIN(T), cap)


def test_attention_tree_paged_window_sinks():
    par = [-1, 0, 1, 2, 1, 4, 0, 6]
    rng = np.random.default_rng(3)
    _attn_case(rng, 128, 8, 2, 530, 8, par, 1024)
    _attn_case(rng, 128, 8, 2, 530, 8, par, 1024, paged=True)
    _attn_case(rng, 64, 8, 1, 900, 2, CHAIN(2), 1024, win=128)
    _attn_case(rng, 64, 64, 8, 300, 1, CHAIN(1), 512, sinks=True)
    _attn_case(rng, 64, 16, 2, 1100, 4, CHAIN(4), 2048, paged=True, win=700, sinks=True)


def test_attention_tree_row_equals_its_chain():
    """a tree's node computes what the same node computes at the end of a chain of its ancestors"""
    rng = np.random.default_rng(9)
    D, Hq, Hk, n0, cap = 128, 8, 2, 77, 512
    par = [-1, 0, 1, 2, 1, 4, 0, 6]
    hs, rs = D, Hk * D
    q = rand_bf(rng, (8, Hq, D))
    K, V = rand_bf(rng, (cap, Hk, D)), rand_bf(rng, (cap, Hk, D))

    def run(qrows, par_, Kc, Vc):
        T = len(par_)
        S = 1
        out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=DEV)
        pm = torch.zeros(S * T * Hq, dtype=torch.float32, device=DEV)
        pa = torch.zeros(S * T * Hq * D, dtype=torch.float32, device=DEV)
        cnt = torch.zeros(T * Hk, dtype=torch.int32, device=DEV)
        n0t = torch.tensor([n0], dtype=torch.int32, device=DEV)
        keep = [bf(qrows), bf(Kc), bf(Vc), torch.tensor(par_, dtype=torch.int32, device=DEV)]
        call("btb_b200_attn_decode", ptr(keep[0]), ptr(keep[1]), ptr(keep[2]), ptr(out), ptr(n0t), ptr(keep[3]), T, Hq,
             Hk, D, hs, rs, float(D**-0.5), ptr(pm), ptr(pm), ptr(pa), ptr(cnt), 0, 0, 0, cap, s())  # fmt: skip
        return bits(out)

    tree = run(q, par, K, V)
    for node, path in ((5, [0, 1, 4, 5]), (7, [0, 6, 7]), (3, [0, 1, 2, 3])):
        Kc, Vc = K.copy(), V.copy()
        for j, p in enumerate(path):  # the path's rows gathered to the front, as a commit does
            Kc[n0 + j], Vc[n0 + j] = K[n0 + p], V[n0 + p]
        chain = run(q[path], CHAIN(len(path)), Kc, Vc)
        assert np.array_equal(chain[-1], tree[node])


@pytest.mark.parametrize("T,V", [(1, 151936), (3, 1000), (2, 2057), (32, 4096)])
def test_argmax_lowest_index_on_ties(T, V):
    rng = np.random.default_rng(V)
    lg = rand_bf(rng, (T, V))
    top = O.f32_to_bits(np.array([50.0], np.float32))[0]
    for t in range(T):  # plant exact ties at the maximum
        for i in rng.integers(0, V, size=3):
            lg[t, i] = top
    lt = bf(lg)
    scratch = torch.zeros(int(capi.lib().btb_b200_argmax_scratch_bytes(T)) // 8 + 1, dtype=torch.int64, device=DEV)
    out = torch.zeros(T, dtype=torch.int64, device=DEV)
    for _ in range(2):  # the scratch must come back clean
        call("btb_b200_argmax_bf16", ptr(lt), T, V, ptr(scratch), ptr(out), s())
        assert np.array_equal(out.cpu().numpy(), O.argmax_bf16(lg))
        assert np.array_equal(out.cpu().numpy(), lt.float().argmax(-1).cpu().numpy())
    assert int(scratch.abs().sum()) == 0


def test_embed_and_publish():
    rng = np.random.default_rng(1)
    V, H = 300, 64
    tab = rand_bf(rng, (V, H))
    ids = torch.tensor([5, 299, 0], dtype=torch.int64, device=DEV)
    tt, h = bf(tab), torch.zeros(3, H, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_embed", ptr(tt), ptr(ids), ptr(h), 3, H, V, s())
    assert np.array_equal(bits(h), tab[[5, 299, 0]])
    n0 = torch.tensor([41], dtype=torch.int32, device=DEV)
    tok, pn, ts = (torch.zeros(1, dtype=d).pin_memory() for d in (torch.int64, torch.int32, torch.int64))
    call("btb_b200_publish", ptr(n0), ptr(ids), ptr(tok), ptr(pn), ptr(ts), 1, s())
    torch.cuda.synchronize()
    assert int(n0[0]) == 42 and int(pn[0]) == 42 and int(tok[0]) == 5 and int(ts[0]) > 0


# ---- against the reference's own kernels, bit for bit -----------------------------------------------------------


def _P(t):
    return 0 if t is None else t.data_ptr()


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16, 32])
def test_ref_gemv_bits(ref, b200, M):
    rng = np.random.default_rng(M)
    for R, Cc in ((300, 2560), (64, 9728), (37, 264)):
        w, x = bf(rand_bf(rng, (R, Cc), 0.02)), bf(rand_bf(rng, (M, Cc)))
        ya = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
        yb = torch.zeros_like(ya)
        for lz, y in ((ref, ya), (b200, yb)):
            L.btb_gemv_bf16(lz, M, ((R + 3) // 4, 1, 1), (128, 1, 1), _P(w), _P(x), _P(y), R, Cc)
        assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))
        if M <= 8 and M * Cc * 2 <= 64 * 1024:  # the fold's shared-memory budget for the activated x
            gu = bf(rand_bf(rng, (M, 2 * Cc), 1.5))
            for lz, y in ((ref, ya), (b200, yb)):
                L.btb_gemv_silu_bf16(lz, M, ((R + 3) // 4, 1, 1), (128, 1, 1), _P(w), _P(gu), _P(y), R, Cc)
            assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))


def test_ref_small_kernels_bits(ref, b200):
    rng = np.random.default_rng(0)
    T, H, I = 7, 2560, 9728
    h0, y, w = rand_bf(rng, (T, H)), bf(rand_bf(rng, (T, H), 0.1)), bf(rand_bf(rng, (H,)))
    outs = []
    for lz in (ref, b200):
        h, x = bf(h0), torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
        L.btb_add_rmsnorm(lz, (T, 1, 1), (256, 1, 1), _P(h), _P(y), _P(w), 1e-6, _P(x), H, 0)
        outs.append((bits(h), bits(x)))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    gu = bf(rand_bf(rng, (T, 2 * I), 1.5))
    ms = []
    for lz in (ref, b200):
        m = torch.zeros(T, I, dtype=torch.bfloat16, device=DEV)
        L.btb_silu_mul(lz, (min(4096, (T * I + 255) // 256), 1, 1), (256, 1, 1), _P(gu), _P(m), T, I)
        ms.append(bits(m))
    assert np.array_equal(ms[0], ms[1])
    # norm + rope + cache write, plain and through a row map
    D, Hq, Hk, cap, n0 = 128, 8, 2, 256, 50
    qkv = bf(rand_bf(rng, (T, (Hq + 2 * Hk) * D)))
    wq, wk = bf(rand_bf(rng, (D,))), bf(rand_bf(rng, (D,)))
    cos, sin = (bf(a) for a in _rope_tables(D, cap, rng))
    n0t = torch.tensor([n0], dtype=torch.int32, device=DEV)
    dep = torch.tensor([0, 1, 2, 3, 2, 3, 1], dtype=torch.int32, device=DEV)
    tbl = torch.from_numpy(rng.permutation(cap).astype(np.int32)).to(DEV)
    K0 = rand_bf(rng, (cap, Hk, D))
    for paged in (False, True):
        res = []
        for lz in (ref, b200):
            K, V, q = bf(K0), bf(K0), torch.zeros(T, Hq, D, dtype=torch.bfloat16, device=DEV)
            a = (D, (Hq + 2 * Hk, T, 1), (32, 1, 1), _P(qkv), _P(wq), _P(wk), 1e-6, _P(cos), _P(sin), _P(n0t), _P(dep),
                 _P(K), _P(V), _P(q), T, Hq, Hk, D, Hk * D, 0)  # fmt: skip
            if paged:
                L.btb_norm_rope_kv_tbl(lz, *a, _P(tbl))
            else:
                L.btb_norm_rope_kv(lz, *a)
            res.append((bits(K), bits(V), bits(q)))
        for a_, b_ in zip(res[0], res[1]):
            assert np.array_equal(a_, b_)


def test_ref_attention_close(ref, b200):
    """the reference's tensor-core attention and this library's SIMT attention: same folds, dot products in another
    order - held to the reference's own 2^-6 bound"""
    rng = np.random.default_rng(4)
    D, Hq, Hk, cap = 128, 8, 2, 2048
    S = cap // 512
    for n0, par in ((100, [-1]), (1300, [-1, 0, 1, 2]), (530, [-1, 0, 1, 2, 1, 4, 0, 6])):
        T = len(par)
        G = Hq // Hk
        q, K, V = bf(rand_bf(rng, (T, Hq, D))), bf(rand_bf(rng, (cap, Hk, D))), bf(rand_bf(rng, (cap, Hk, D)))
        n0t = torch.tensor([n0], dtype=torch.int32, device=DEV)
        pt = torch.tensor(par, dtype=torch.int32, device=DEV)
        outs = []
        for lz in (ref, b200):
            out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=DEV)
            pm = torch.zeros(S * T * Hq, dtype=torch.float32, device=DEV)
            pl = torch.zeros_like(pm)
            pa = torch.zeros(S * T * Hq * D, dtype=torch.float32, device=DEV)
            cnt = torch.zeros(T * Hq, dtype=torch.int32, device=DEV)
            L.btb_attn_flash(lz, D, ((T * G + 7) // 8, S, Hk), (256, 1, 1), _P(q), _P(K), _P(V), _P(out), _P(n0t), _P(pt),
                             T, Hq, Hk, D, Hk * D, float(D**-0.5), _P(pm), _P(pl), _P(pa), _P(cnt), 0, 0)  # fmt: skip
            outs.append(out.float().cpu().numpy())
        assert np.max(np.abs(outs[0] - outs[1])) <= 2.0**-6 * max(1.0, float(np.max(np.abs(outs[0]))))


def test_launcher_refuses_unknown_kernels(b200):
    with pytest.raises(KeyError):
        b200.launch("btb_delta_nodes", (1, 1, 1), (32, 1, 1), [])
    assert b200.serves("btb_gemv_bf16_m8") and not b200.serves("btb_gemv_q4k_bf16_m1")
    assert isinstance(C.c_void_p(0), C._SimpleCData) and os.path.exists(capi.LIB_PATH)


# ---- SwiGLU in the gate/up GEMV's epilogue -----------------------------------------------------------------------


@pytest.mark.parametrize("M,T", [(1, 1), (2, 2), (4, 3), (8, 8)])
@pytest.mark.parametrize("I,H", [(9728, 2560), (512, 256), (300, 264), (37, 1024)])
def test_gemv_norm_swiglu_equals_gemv_norm_then_silu_mul(M, T, I, H):
    rng = np.random.default_rng(I + H + M)
    w = bf(rand_bf(rng, (2 * I, H), 0.05))
    h, yadd, nw = bf(rand_bf(rng, (M, H))), bf(rand_bf(rng, (M, H))), bf(rand_bf(rng, (H,)))
    h2a, h2b = torch.zeros_like(h), torch.zeros_like(h)
    gu = torch.zeros(M, 2 * I, dtype=torch.bfloat16, device=DEV)
    want = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    got = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_norm", ptr(w), 0, 0, 0, 0, 0, ptr(h), ptr(yadd), ptr(nw), 1e-6, 0, ptr(h2a), ptr(gu), T, M, 2 * I,
         H, s())  # fmt: skip
    call("btb_b200_silu_mul", ptr(gu), ptr(want), M, I, s())
    call("btb_b200_gemv_norm_swiglu", ptr(w), 0, 0, 0, 0, 0, ptr(h), ptr(yadd), ptr(nw), 1e-6, 0, ptr(h2b), ptr(got), T,
         M, 2 * I, H, s())  # fmt: skip
    assert np.array_equal(bits(got)[:T], bits(want)[:T])
    assert np.array_equal(bits(h2a)[:T], bits(h2b)[:T])


def test_gemv_norm_swiglu_over_pack12_weights():
    from btb_b200.engine import P12Matrix

    rng = np.random.default_rng(5)
    I, H, M = 384, 512, 2
    wbits, parts = _p12_case(rng, 2 * I, H, True)
    w = bf(wbits)
    P = P12Matrix(parts, 2 * I, H, DEV)
    h, yadd, nw = bf(rand_bf(rng, (M, H))), bf(rand_bf(rng, (M, H))), bf(rand_bf(rng, (H,)))
    h2a, h2b = torch.zeros_like(h), torch.zeros_like(h)
    want = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    got = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemv_norm_swiglu", ptr(w), 0, 0, 0, 0, 0, ptr(h), ptr(yadd), ptr(nw), 1e-6, 0, ptr(h2a), ptr(want), M, M,
         2 * I, H, s())  # fmt: skip
    call("btb_b200_gemv_norm_swiglu", ptr(P.lo), ptr(P.hi4), P.table, ptr(P.esc_idx), ptr(P.esc_val), ptr(P.esc_row),
         ptr(h), ptr(yadd), ptr(nw), 1e-6, 0, ptr(h2b), ptr(got), M, M, 2 * I, H, s())  # fmt: skip
    assert np.array_equal(bits(got), bits(want))
