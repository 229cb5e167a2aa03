"""Parity at the benchmark configurations' REAL shapes (the small-model tests cover the logic; these cover the widths).

Dense configs (Qwen3-4B, Llama-3.1-70B shapes): one layer's kernel sequence and the head GEMV are launched through the
reference's own kernels compiled for this card (oracle/_ref, driven by `RefLauncher`) and through `B200Launcher` with
the same typed calls on the same seeded tensors; every kernel's output is compared as BITS, the attention within the
reference's own 2^-6 bound (two summation orders). Each of this library's kernels is fed the reference's inputs, so a
difference is that kernel's own. MoE configs (gpt-oss-20b, Qwen3-30B-A3B shapes): one full-shape MoE block against the
CPU oracle stage by stage, and the router and 16-lane matvecs against the reference's kernels as well.
"""

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


def bf(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16).to(DEV)


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def randn_bf(gen, shape, scale=1.0):
    return (torch.randn(*shape, generator=gen, device=DEV) * scale).to(torch.bfloat16)


def _P(t):
    return 0 if t is None else t.data_ptr()


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


def same_bits(a, b, what):
    assert torch.equal(a.view(torch.int16), b.view(torch.int16)), what


DENSE = {
    # hidden, q heads, kv heads, head dim, intermediate, vocab, q/k norm, eps
    "qwen3-4b": (2560, 32, 8, 128, 9728, 151936, True, 1e-6),
    "llama-3.1-70b": (8192, 64, 8, 128, 28672, 128256, False, 1e-5),
}


@pytest.mark.parametrize("name,M", [("qwen3-4b", 1), ("qwen3-4b", 8), ("llama-3.1-70b", 1)])
def test_dense_layer_and_head_equal_the_reference_kernels(ref, b200, name, M):
    H, Hq, Hk, D, I, V, qk, eps = DENSE[name]
    gen = torch.Generator(device=DEV).manual_seed(sum(name.encode()) + M)
    QR = (Hq + 2 * Hk) * D
    w_qkv, w_o = randn_bf(gen, (QR, H), 0.02), randn_bf(gen, (H, Hq * D), 0.02)
    w_gu, w_dn = randn_bf(gen, (2 * I, H), 0.02), randn_bf(gen, (H, I), 0.02)
    ln1, ln2 = randn_bf(gen, (H,), 1.0), randn_bf(gen, (H,), 1.0)
    wq = randn_bf(gen, (D,), 1.0) if qk else None
    wk = randn_bf(gen, (D,), 1.0) if qk else None
    n0, cap = 700, 1024
    S = cap // 512
    K0, V0 = randn_bf(gen, (cap, Hk, D)), randn_bf(gen, (cap, Hk, D))
    ang = torch.rand(cap, D, generator=gen, device=DEV) * 6.28
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    n0t = torch.tensor([n0], dtype=torch.int32, device=DEV)
    depth = torch.arange(M, dtype=torch.int32, device=DEV)
    par = torch.arange(-1, M - 1, dtype=torch.int32, device=DEV)
    h0, y0 = randn_bf(gen, (M, H)), randn_bf(gen, (M, H), 0.3)
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=DEV)  # noqa: E731
    gemv_grid = lambda R: ((R + 3) // 4, 1, 1)  # noqa: E731  the reference's launch: a warp a row, four a block

    def norm(lz, h_in, y_in, w):
        h, x = h_in.clone(), z(M, H)
        L.btb_add_rmsnorm(lz, (M, 1, 1), (256, 1, 1), _P(h), _P(y_in), _P(w), eps, _P(x), H, 0)
        return h, x

    def gemv(lz, w, x, R, C_):
        y = z(M, R)
        L.btb_gemv_bf16(lz, M, gemv_grid(R), (128, 1, 1), _P(w), _P(x), _P(y), R, C_)
        return y

    def rope(lz, qkv):
        K, V_, q = K0.clone(), V0.clone(), z(M, Hq, D)
        L.btb_norm_rope_kv(lz, D, (Hq + 2 * Hk, M, 1), (32, 1, 1), _P(qkv), _P(wq), _P(wk), eps, _P(cos), _P(sin), _P(n0t),
                           _P(depth), _P(K), _P(V_), _P(q), M, Hq, Hk, D, Hk * D, 0)  # fmt: skip
        return K, V_, q

    def attn(lz, q, K, V_):
        out = z(M, Hq * D)
        pm = torch.zeros(S * M * Hq, dtype=torch.float32, device=DEV)
        pl, pa = torch.zeros_like(pm), torch.zeros(S * M * Hq * D, dtype=torch.float32, device=DEV)
        cnt = torch.zeros(M * Hq, dtype=torch.int32, device=DEV)
        G = Hq // Hk
        L.btb_attn_flash(lz, D, ((M * G + 7) // 8, S, Hk), (256, 1, 1), _P(q), _P(K), _P(V_), _P(out), _P(n0t), _P(par), M,
                         Hq, Hk, D, Hk * D, float(D**-0.5), _P(pm), _P(pl), _P(pa), _P(cnt), 0, 0)  # fmt: skip
        return out

    def down(lz, gu):
        y = z(M, H)
        L.btb_gemv_silu_bf16(lz, M, gemv_grid(H), (128, 1, 1), _P(w_dn), _P(gu), _P(y), H, I)
        return y

    # the reference's chain makes every stage's input; this library's kernel runs on the same input
    h1, x1 = norm(ref, h0, y0, ln1)
    for a, b, what in zip(norm(b200, h0, y0, ln1), (h1, x1), ("residual", "normed")):
        same_bits(a, b, what)
    qkv = gemv(ref, w_qkv, x1, QR, H)
    same_bits(gemv(b200, w_qkv, x1, QR, H), qkv, "qkv")
    Kr, Vr, qr = rope(ref, qkv)
    for a, b, what in zip(rope(b200, qkv), (Kr, Vr, qr), ("K rows", "V rows", "q")):
        same_bits(a, b, what)
    att = attn(ref, qr, Kr, Vr)
    mine = attn(b200, qr, Kr, Vr)
    tol = 2.0**-6 * max(1.0, float(att.float().abs().max()))
    assert float((att.float() - mine.float()).abs().max()) <= tol
    yo = gemv(ref, w_o, att, H, Hq * D)
    same_bits(gemv(b200, w_o, att, H, Hq * D), yo, "o projection")
    h2, x2 = norm(ref, h1, yo, ln2)
    for a, b, what in zip(norm(b200, h1, yo, ln2), (h2, x2), ("residual 2", "normed 2")):
        same_bits(a, b, what)
    gu = gemv(ref, w_gu, x2, 2 * I, H)
    same_bits(gemv(b200, w_gu, x2, 2 * I, H), gu, "gate/up")
    if M * I * 2 <= 160 * 1024:  # the fold stages the activated row in shared memory
        yd = down(ref, gu)
        same_bits(down(b200, gu), yd, "down with the SwiGLU fold")
    # the fused forms the step really launches: norm inside the GEMV, SwiGLU in the gate/up GEMV's epilogue
    if M * H * 2 <= 64 * 1024:
        hf, qf = z(M, H), z(M, QR)
        call("btb_b200_gemv_norm", ptr(w_qkv), 0, 0, 0, 0, 0, ptr(h0), ptr(y0), ptr(ln1), eps, 0, ptr(hf), ptr(qf), M, M,
             QR, H, capi.stream_ptr())  # fmt: skip
        same_bits(hf, h1, "fused norm: residual")
        same_bits(qf, qkv, "fused norm: qkv")
        mf, hf2 = z(M, I), z(M, H)
        call("btb_b200_gemv_norm_swiglu", ptr(w_gu), 0, 0, 0, 0, 0, ptr(h1), ptr(yo), ptr(ln2), eps, 0, ptr(hf2), ptr(mf),
             M, M, 2 * I, H, capi.stream_ptr())  # fmt: skip
        mr = z(M, I)
        L.btb_silu_mul(ref, (min(4096, (M * I + 255) // 256), 1, 1), (256, 1, 1), _P(gu), _P(mr), M, I)
        same_bits(mf, mr, "SwiGLU epilogue")
        yd2 = gemv(ref, w_dn, mr, H, I)
        same_bits(gemv(b200, w_dn, mr, H, I), yd2, "down")
    del w_gu, w_dn, w_qkv, w_o
    # the head: the tied embedding table as a GEMV over the final norm's row
    w_head = randn_bf(gen, (V, H), 0.02)
    lg = gemv(ref, w_head, x2, V, H)
    same_bits(gemv(b200, w_head, x2, V, H), lg, "head")
    # and the pick: the lowest index among equal maxima (torch.argmax over the bf16 row, btb/engine/cuda.py:2237)
    lg[0, 77], lg[0, 90000] = 30000.0, 30000.0
    pick = torch.zeros(M, dtype=torch.int64, device=DEV)
    scratch = torch.zeros((int(capi.lib().btb_b200_argmax_scratch_bytes(M)) + 7) // 8, dtype=torch.int64, device=DEV)
    call("btb_b200_argmax_bf16", ptr(lg), M, V, ptr(scratch), ptr(pick), capi.stream_ptr())
    assert int(pick[0]) == 77
    assert pick[1:].tolist() == lg[1:].float().argmax(-1).tolist()


MOE = {
    # hidden, experts, top-k, intermediate, router mode, glu kind, expert format
    "gpt-oss-20b": (2880, 32, 4, 2880, 1, 1, "mx4"),
    "qwen3-30b-a3b": (2048, 128, 8, 768, 0, 0, "fp8"),
}


@pytest.mark.parametrize("name", list(MOE))
@pytest.mark.parametrize("T", [1, 3])
def test_moe_block_at_full_shape_equals_the_oracle(name, T):
    """router matvec -> picks -> the picked experts' gate/up -> gated activation -> down -> ordered sum, each stage on
    the oracle's input for it: matvec and sum bit for bit, picks exact, expf-carrying stages within a bf16 step"""
    H, E, k, I, mode, kind, fmt = MOE[name]
    rng = np.random.default_rng(len(name) + T)
    sp = capi.stream_ptr()
    x = O.bits_to_f32(O.f32_to_bits(rng.standard_normal((T, H)).astype(np.float32)))  # a normed bf16 row, widened
    xt = torch.from_numpy(x).to(DEV)
    rw = O.f32_to_bits(rng.standard_normal((E, H)).astype(np.float32) * 0.05)
    rwt = bf(rw)
    logits = O.cpu_gemv_bf16(rw, x)
    want_idx, want_w = O.moe_route(logits, E, k, mode)
    idx = torch.zeros(T, k, dtype=torch.int32, device=DEV)
    w = torch.zeros(T, k, dtype=torch.bfloat16, device=DEV)
    rl = torch.zeros(T, E, dtype=torch.float32, device=DEV)
    call("btb_b200_moe_gemv", 0, ptr(rwt), 0, 0, 0, 1, 1, 0, T, 1, ptr(xt), 1, ptr(rl), E, H, 0, 1, sp)
    assert np.array_equal(rl.cpu().numpy().view(np.uint32), logits.view(np.uint32))
    call("btb_b200_moe_route", ptr(rl), E, E, k, mode, 1, ptr(idx), ptr(w), T, sp)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.max(np.abs(bits(w).astype(np.int32) - want_w.astype(np.int32))) <= 1
    if E * H <= 131072 and H % 8 == 0:  # the one-launch router
        idx2, w2 = torch.zeros_like(idx), torch.zeros_like(w)
        call("btb_b200_moe_router", ptr(rwt), ptr(xt), 0, E, H, k, mode, ptr(idx2), ptr(w2), T, sp)
        assert torch.equal(idx2, idx) and torch.equal(w2.view(torch.int16), w.view(torch.int16))
    # the experts as stored; only the picked ones are drawn in full
    picked = sorted(set(want_idx.reshape(-1).tolist()))
    slot = {e: i for i, e in enumerate(picked)}
    n = len(picked)
    if fmt == "mx4":
        gu_w = rng.integers(0, 256, size=(n, 2 * I, H // 32, 16), dtype=np.uint8)
        gu_s = rng.integers(119, 128, size=(n, 2 * I, H // 32), dtype=np.uint8)
        dn_w = rng.integers(0, 256, size=(n, H, I // 32, 16), dtype=np.uint8)
        dn_s = rng.integers(119, 128, size=(n, H, I // 32), dtype=np.uint8)
        gemv = lambda W, S_, e, R, C_, xx: O.cpu_gemv_mxfp4(W[e], S_[e], R, C_, xx)  # noqa: E731
        args = lambda W, S_, R, C_: (1, ptr(W), ptr(S_), R * C_ // 2, R * C_ // 32, 1, 1)  # noqa: E731
    else:
        def draw(R, C_):
            wq = rng.integers(0, 256, size=(n, R, C_), dtype=np.uint8)
            wq[(wq & 0x7F) == 0x7F] = 0x30
            sc = O.bits_to_f32(O.f32_to_bits(rng.standard_normal((n, R // 128, C_ // 128)).astype(np.float32) * 0.02))
            return wq, sc
        (gu_w, gu_s), (dn_w, dn_s) = draw(2 * I, H), draw(H, I)
        gemv = lambda W, S_, e, R, C_, xx: O.cpu_gemv_fp8(W[e], S_[e], R, C_, xx)  # noqa: E731
        args = lambda W, S_, R, C_: (2, ptr(W), ptr(S_), R * C_, (R // 128) * (C_ // 128) * 4, R // 128, C_ // 128)  # noqa: E731
    # the card holds the picked experts as a stack of n; the index list names them by their place in it
    local = torch.tensor([[slot[int(e)] for e in row] for row in want_idx], dtype=torch.int32, device=DEV)
    tw = [torch.from_numpy(a).to(DEV) for a in (gu_w, gu_s, dn_w, dn_s)]
    egu = torch.zeros(T * k, 2 * I, dtype=torch.float32, device=DEV)
    f, wp, scp, ws, ss, sr, sc = args(tw[0], tw[1], 2 * I, H)
    call("btb_b200_moe_gemv", f, wp, scp, ws, ss, sr, sc, ptr(local), T * k, n, ptr(xt), k, ptr(egu), 2 * I, H, 0, 1, sp)
    want_gu = np.stack([gemv(gu_w, gu_s, slot[int(want_idx[t, j])], 2 * I, H, x[t : t + 1])[0] for t in range(T) for j in range(k)])
    assert np.array_equal(egu.cpu().numpy().view(np.uint32), want_gu.view(np.uint32))
    eh = torch.zeros(T * k, I, dtype=torch.float32, device=DEV)
    call("btb_b200_moe_act", ptr(egu), ptr(eh), 0, 0, T * k, I, kind, 1.702, 7.0, sp)
    want_h = O.moe_act(want_gu, kind)
    d = O.f32_to_bits(eh.cpu().numpy()).astype(np.int32) - O.f32_to_bits(want_h).astype(np.int32)
    assert np.max(np.abs(d)) <= 2 and np.mean(d != 0) < 5e-3
    # the down matvecs on the oracle's activated rows, then the sum
    eht = torch.from_numpy(want_h).to(DEV)
    edn = torch.zeros(T * k, H, dtype=torch.float32, device=DEV)
    f, wp, scp, ws, ss, sr, sc = args(tw[2], tw[3], H, I)
    call("btb_b200_moe_gemv", f, wp, scp, ws, ss, sr, sc, ptr(local), T * k, n, ptr(eht), 1, ptr(edn), H, I, 0, 1, sp)
    want_dn = np.stack([gemv(dn_w, dn_s, slot[int(want_idx[t, j])], H, I, want_h[t * k + j][None])[0] for t in range(T) for j in range(k)])
    assert np.array_equal(edn.cpu().numpy().view(np.uint32), want_dn.view(np.uint32))
    y = torch.zeros(T, H, dtype=torch.bfloat16, device=DEV)
    wt = bf(want_w)
    it = torch.from_numpy(want_idx).to(DEV)
    call("btb_b200_moe_combine", ptr(edn), ptr(it), ptr(wt), 0, ptr(y), T, k, H, sp)
    assert np.array_equal(bits(y), O.moe_combine(want_dn.reshape(T, k, H), want_idx, want_w))


def test_moe_kernels_equal_the_reference_kernels(ref, b200):
    """btb_moe_route and btb_gemv_lane16{,_mx4}_f32_m* by the reference's names and parameter lists through both
    launchers: the picks exact, the weights and the matvecs bit for bit (the same device computes expf for both)"""
    rng = np.random.default_rng(11)
    for E, k, T in ((128, 8, 5), (32, 4, 1), (300, 5, 3)):
        lg = O.f32_to_bits(rng.standard_normal((T, E + 1)).astype(np.float32) * 2)  # ls = E + 1: a gate column rides along
        lg[0, 3] = lg[0, 7]
        lt = bf(lg)
        res = []
        for lz in (ref, b200):
            idx = torch.zeros(T, k, dtype=torch.int32, device=DEV)
            w = torch.zeros(T, k, dtype=torch.bfloat16, device=DEV)
            L.btb_moe_route(lz, (T, 1, 1), (256, 1, 1), _P(lt), E + 1, E, k, _P(idx), _P(w), 0, 0, 0, 0, 0, shared=E * 4)
            res.append((idx.cpu(), bits(w)))
        assert torch.equal(res[0][0], res[1][0])
        assert np.array_equal(res[0][1], res[1][1])
    for R, C_, M in ((5760, 2880, 1), (2880, 2880, 4), (128, 2048, 2), (37, 264, 1)):
        x = torch.from_numpy(rng.standard_normal((M, C_)).astype(np.float32)).to(DEV)
        wb = bf(O.f32_to_bits(rng.standard_normal((R, C_)).astype(np.float32) * 0.02))
        ys = []
        for lz in (ref, b200):
            y = torch.zeros(M, R, dtype=torch.float32, device=DEV)
            L.btb_gemv_lane16_f32(lz, M, ((R + 7) // 8, 1, 1), (128, 1, 1), _P(wb), _P(x), _P(y), R, C_)
            ys.append(y)
        assert torch.equal(ys[0].view(torch.int32), ys[1].view(torch.int32)), (R, C_, M)
        if C_ % 32:
            continue
        blocks = torch.from_numpy(rng.integers(0, 256, size=(R, C_ // 32, 16), dtype=np.uint8)).to(DEV)
        scales = torch.from_numpy(rng.integers(117, 130, size=(R, C_ // 32), dtype=np.uint8)).to(DEV)
        ys = []
        for lz in (ref, b200):
            y = torch.zeros(M, R, dtype=torch.float32, device=DEV)
            L.btb_gemv_lane16_mx4_f32(lz, M, ((R + 7) // 8, 1, 1), (128, 1, 1), _P(blocks), _P(scales), _P(x), _P(y), R, C_)
            ys.append(y)
        assert torch.equal(ys[0].view(torch.int32), ys[1].view(torch.int32)), (R, C_, M, "mx4")
