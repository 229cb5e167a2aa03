"""The CPU oracle against the reference's own outputs (tests/golden, made by make_golden.py from the reference's
Python codecs and banked receipts). CPU only."""

import json
import os

import numpy as np
import pytest

from oracle import model as OM
from oracle import oracle as O


@pytest.fixture(scope="module")
def codecs(golden_dir):
    return np.load(os.path.join(golden_dir, "codecs.npz"))


@pytest.fixture(scope="module")
def tiny(golden_dir):
    return np.load(os.path.join(golden_dir, "tiny_qwen3.npz"))


@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_p12_widen_equals_reference_unpack(codecs, case):
    g = lambda k: codecs[f"p12_{case}_{k}"]  # noqa: E731
    src = g("src")
    out = O.widen_p12(g("lo"), g("hi4"), g("tbl"), g("esc_idx"), g("esc_val"), src.size)
    assert np.array_equal(out, g("unpacked").reshape(-1))
    assert np.array_equal(out, src.reshape(-1))


def test_p12_rejects_unsorted_escapes(codecs):
    g = lambda k: codecs[f"p12_b_{k}"]  # noqa: E731
    ei = g("esc_idx").copy()
    assert ei.size >= 2
    ei[0], ei[1] = ei[1], ei[0]
    with pytest.raises(O.OracleError):
        O.widen_p12(g("lo"), g("hi4"), g("tbl"), ei, g("esc_val"), g("src").size)


def test_mxfp4_every_byte_every_scale(codecs):
    pair = codecs["mx4_pair"]  # [scale, byte, 2] uint32 bits of the reference's dequantize
    blocks = np.broadcast_to(np.arange(256, dtype=np.uint8)[None, :, None], (256, 256, 16)).copy()
    scales = np.broadcast_to(np.arange(256, dtype=np.uint8)[:, None], (256, 256)).copy()
    out = O.widen_mxfp4(blocks.reshape(256 * 256, 16), scales.reshape(-1), 256 * 256, 32).view(np.uint32)
    out = out.reshape(256, 256, 32)
    ref = np.tile(pair, (1, 1, 16))
    # NaN payloads (0 * inf under scale 255) compare as NaN-ness; everything else to the bit
    nan = (ref & 0x7FFFFFFF) > 0x7F800000
    assert np.array_equal(nan, (out & 0x7FFFFFFF) > 0x7F800000)
    assert np.array_equal(out[~nan], ref[~nan])


def test_mxfp4_matrix_layout(codecs):
    mb, ms = codecs["mx4_m_blocks"], codecs["mx4_m_scales"]
    out = O.widen_mxfp4(mb, ms, 6, 128).view(np.uint32)
    assert np.array_equal(out, codecs["mx4_m_deq"])


def test_fp8_every_byte_under_scales(codecs):
    sc = codecs["fp8_scales"]
    n = sc.size
    w = np.broadcast_to(np.arange(256, dtype=np.uint8)[None, :], (n, 256)).copy()
    out = O.widen_fp8(w, sc.reshape(n, 1), n, 256)
    ref = codecs["fp8_held"]
    nan = (ref & 0x7FFF) > 0x7F80
    assert np.array_equal(nan, (out & 0x7FFF) > 0x7F80)
    assert np.array_equal(out[~nan], ref[~nan])


def test_fp8_block_grid(codecs):
    out = O.widen_fp8(codecs["fp8_m_w"], codecs["fp8_m_scales"], 8, 12)
    assert np.array_equal(out, codecs["fp8_m_held"])


def _split_p12(blob: np.ndarray, meta: np.ndarray):
    """the reference's on-disk pack12 entry (btb/pack12.py:100-133) into its parts"""
    import struct

    table = meta[:16].copy()
    n_esc, rank = struct.unpack("<II", meta[16:24].tobytes())
    shape = struct.unpack(f"<{rank}q", meta[24 : 24 + 8 * rank].tobytes())
    n = int(np.prod(shape))
    lo = blob[:n]
    hi4 = blob[n : n + (n + 1) // 2]
    off = n + (n + 1) // 2
    off += (-off) % 4
    esc_idx = blob[off : off + 4 * n_esc].view(np.int32)
    esc_val = blob[off + 4 * n_esc : off + 5 * n_esc]
    return lo, hi4, table, esc_idx, esc_val, shape


def test_p12_store_of_tiny_model_widens_to_its_bf16(tiny):
    names = [k[4:-7] for k in tiny.files if k.startswith("p12/") and k.endswith(".pack12")]
    assert len(names) > 40
    for name in names:
        lo, hi4, table, ei, ev, shape = _split_p12(tiny[f"p12/{name}.pack12"], tiny[f"p12/{name}.pack12.meta"])
        out = O.widen_p12(lo, hi4, table, ei, ev, int(np.prod(shape)))
        assert np.array_equal(out.reshape(shape), tiny[f"w/{name}"]), name


def test_fp8_store_of_tiny_model_is_reference_quantize(tiny):
    # the FP8 store's held values: bf16(e4m3 * scale); the grid is the store's own
    keys = [k for k in tiny.files if k.startswith("f8/") and k.endswith("_scale_inv")]
    assert keys
    for sk in keys:
        wk = sk[: -len("_scale_inv")]
        w, s = tiny[wk], tiny[sk]
        held = O.widen_fp8(w, s.astype(np.float32), *w.shape)
        ref = O.bits_to_f32(tiny["w/" + wk[3:]])
        got = O.bits_to_f32(held)
        # quantisation error of e4m3 (3 mantissa bits) against the bf16 original
        assert np.max(np.abs(got - ref)) <= np.max(np.abs(ref)) * 2.0**-3


def _tiny_weights(tiny) -> OM.Weights:
    cfg = json.loads(tiny["config"].tobytes())
    c = OM.DenseCfg(
        hidden=cfg["hidden_size"], layers=cfg["num_hidden_layers"], q_heads=cfg["num_attention_heads"],
        kv_heads=cfg["num_key_value_heads"], head_dim=cfg["head_dim"], inter=cfg["intermediate_size"],
        vocab=cfg["vocab_size"], theta=cfg["rope_parameters"]["rope_theta"], eps=cfg["rms_norm_eps"],
    )  # fmt: skip
    return OM.Weights(c, {k[2:]: tiny[k] for k in tiny.files if k.startswith("w/")})


def test_cpu_tier_reproduces_banked_receipts(tiny):
    """the oracle's CPU-tier step (16-lane GEMV, f32 block) against the reference's receipts: prompt logits, the
    8-node tree's logits, K/V rows, the logits after the commit, and the greedy tokens"""
    w = _tiny_weights(tiny)
    tol = 1e-5  # the reference's own tolerance for an arm that sums in another order (test_receipts.py:205-208)
    m = OM.CpuTier(w)
    prompt = tiny["rc/prompt"].tolist()
    lg = m.forward(prompt)
    assert np.max(np.abs(lg[-1] - tiny["rc/bf16/prompt_logits"])) <= tol
    base = m.n
    depth = tiny["rc/depth"].tolist()
    chunk = m.forward(tiny["rc/chunk"].tolist(), positions=[base + d for d in depth], parents=tiny["rc/parents"].tolist())
    assert np.max(np.abs(chunk - tiny["rc/bf16/chunk_logits"])) <= tol
    path = tiny["rc/path"].tolist()
    m.keep_path(base, path)
    for i in range(w.cfg.layers):
        assert np.max(np.abs(m.K[i][:, : m.n] - tiny[f"rc/bf16/k{i}"][0][:, : m.n])) <= tol
        assert np.max(np.abs(m.V[i][:, : m.n] - tiny[f"rc/bf16/v{i}"][0][:, : m.n])) <= tol
    nxt = m.forward([int(tiny["rc/chunk"][path[-1]])])  # the step over the last accepted token (tests/helpers.py:276)
    assert np.max(np.abs(nxt[0] - tiny["rc/bf16/next"])) <= tol
    # greedy from the prompt
    g = OM.CpuTier(w)
    lg = g.forward(prompt)
    toks = [int(np.argmax(lg[-1]))]
    while len(toks) < 10:
        toks.append(int(np.argmax(g.forward([toks[-1]])[0])))
    assert toks == tiny["rc/bf16/greedy"].tolist()
    # the packed store's receipts are the bf16 store's, to the bit
    for k in ("prompt_logits", "chunk_logits", "next"):
        assert np.array_equal(tiny[f"rc/p12/{k}"], tiny[f"rc/bf16/{k}"])


def test_cpu_gemv_paths_agree_to_the_bit():
    rng = np.random.default_rng(0)
    for R, C_ in [(5, 40), (9, 528), (64, 1040), (3, 17)]:
        w = O.f32_to_bits(rng.standard_normal((R, C_)).astype(np.float32) * 0.02)
        x = rng.standard_normal((3, C_)).astype(np.float32)
        a = O.cpu_gemv_bf16(w, x, threads=1)
        b = O.cpu_gemv_bf16(w, x, threads=4)
        one = np.concatenate([O.cpu_gemv_bf16(w, x[i : i + 1]) for i in range(3)])
        O.force_scalar(True)
        try:
            s = O.cpu_gemv_bf16(w, x)
        finally:
            O.force_scalar(False)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        assert np.array_equal(a.view(np.uint32), one.view(np.uint32))
        assert np.array_equal(a.view(np.uint32), s.view(np.uint32))
        ref = O.bits_to_f32(w).astype(np.float64) @ x.astype(np.float64).T
        assert np.max(np.abs(a.T - ref)) <= 1e-5 * np.max(np.abs(ref)) + 1e-6


def test_cpu_packed_gemvs_equal_gemv_over_their_widen(codecs):
    rng = np.random.default_rng(1)
    # pack12: the packed matrix multiplies to the bf16 matrix's bits (native/tests/gemv.rs: p12 == bf16)
    src = codecs["p12_a_src"]
    R, C_ = src.shape
    x = rng.standard_normal((2, C_)).astype(np.float32)
    g = lambda k: codecs[f"p12_a_{k}"]  # noqa: E731
    yp = O.cpu_gemv_p12(g("lo"), g("hi4"), g("tbl"), g("esc_idx"), g("esc_val"), R, C_, x)
    assert np.array_equal(yp.view(np.uint32), O.cpu_gemv_bf16(src, x).view(np.uint32))
    srcb = codecs["p12_b_src"]
    R, C_ = srcb.shape
    x = rng.standard_normal((2, C_)).astype(np.float32)
    g = lambda k: codecs[f"p12_b_{k}"]  # noqa: E731
    yp = O.cpu_gemv_p12(g("lo"), g("hi4"), g("tbl"), g("esc_idx"), g("esc_val"), R, C_, x)
    assert np.array_equal(yp.view(np.uint32), O.cpu_gemv_bf16(srcb, x).view(np.uint32))
    # fp8: held values are bf16, so the bf16 GEMV over them is the same sum
    w8 = rng.integers(0, 256, size=(16, 256), dtype=np.uint8)
    w8[(w8 & 0x7F) == 0x7F] = 0x11
    sc = O.bits_to_f32(O.f32_to_bits(rng.standard_normal((2, 2)).astype(np.float32) * 0.02))
    x = rng.standard_normal((1, 256)).astype(np.float32)
    y8 = O.cpu_gemv_fp8(w8, sc, 16, 256, x)
    assert np.array_equal(y8.view(np.uint32), O.cpu_gemv_bf16(O.widen_fp8(w8, sc, 16, 256), x).view(np.uint32))


def test_card_gemv_is_row_invariant_and_close_to_f64():
    rng = np.random.default_rng(2)
    R, C_ = 33, 2560
    w = O.f32_to_bits(rng.standard_normal((R, C_)).astype(np.float32) * 0.02)
    x = O.f32_to_bits(rng.standard_normal((8, C_)).astype(np.float32))
    y8 = O.gemv_card_bf16(w, x)
    y1 = np.concatenate([O.gemv_card_bf16(w, x[i : i + 1]) for i in range(8)])
    assert np.array_equal(y8, y1)
    ref = O.bits_to_f32(x).astype(np.float64) @ O.bits_to_f32(w).astype(np.float64).T
    assert np.max(np.abs(O.bits_to_f32(y8) - ref)) <= 2.0**-7 * np.max(np.abs(ref))


def test_card_path_tiny_model_tracks_cpu_tier(tiny):
    """bf16 activations against f32 activations on the tiny fixture: same top token, logits within bf16's reach"""
    w = _tiny_weights(tiny)
    card = OM.CardPath(w)
    lg = card.forward(tiny["rc/prompt"].tolist())
    ref = tiny["rc/bf16/prompt_logits"]
    got = O.bits_to_f32(lg[-1])
    assert np.max(np.abs(got - ref)) <= 0.05 * np.max(np.abs(ref))
    assert int(np.argmax(ref)) == int(O.argmax_bf16(lg[-1:])[0])
