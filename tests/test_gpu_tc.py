"""The tensor-core matvec (tcgen05, accumulator in tensor memory) for passes of up to 32 rows: right to bf16 rounding
against an exact reference, a row's bits independent of the pass width, the same bits every launch."""

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402

DEV = "cuda"


_WS = {}


def _workspace(nbytes):
    """ONE workspace for every shape, as an engine keeps, filled with NaN before each call: a slice of partial sums that
    the launch reads without having written it (an empty K range) poisons the output instead of reading zeros"""
    n = max(nbytes // 4, 4)
    if "t" not in _WS or _WS["t"].numel() < n:
        _WS["t"] = torch.empty(n, dtype=torch.float32, device=DEV)
    _WS["t"].fill_(float("nan"))
    _WS["t"][:256] = 0  # (the head holds the tiles' counters: zero between launches)
    return _WS["t"]


def _run(w, x, M=None):
    M = x.shape[0] if M is None else M
    R, C_ = w.shape
    y = torch.zeros(M, R, dtype=torch.bfloat16, device=DEV)
    nbytes = int(capi.lib().btb_b200_gemv_tc_workspace_bytes(R, C_))
    ws = _workspace(nbytes)
    call("btb_b200_gemv_tc_bf16", ptr(w), ptr(x), ptr(y), M, R, C_, ptr(ws), capi.stream_ptr())
    torch.cuda.synchronize()
    assert capi.status() == 0
    return y


# (2560, 4096), (4096, 4096), (2880, 4096) and (1000, 2880) are shapes whose wanted count of K ranges does not divide
# the K blocks: the ranges are recounted so that none is empty
SHAPES = [(128, 64), (256, 512), (300, 2560), (2560, 4096), (2560, 9728), (6144, 2560), (19456, 2560), (5, 72), (129, 8),
          (1000, 2880), (4096, 4096), (2880, 4096)]  # fmt: skip


@pytest.mark.parametrize("R,C_", SHAPES)
@pytest.mark.parametrize("M", [1, 3, 8, 32])
def test_tc_gemv_is_right_to_bf16_rounding(R, C_, M):
    g = torch.Generator(device=DEV).manual_seed(R + C_ + M)
    w = (torch.randn(R, C_, generator=g, device=DEV) * 0.05).bfloat16()
    x = torch.randn(M, C_, generator=g, device=DEV).bfloat16()
    y = _run(w, x)
    ref = x.double() @ w.double().t()
    # the products are exact in f32 and the sums are f32 over at most C terms: the error is the final rounding to bf16
    # (2^-9 relative) plus the f32 accumulation's (C * 2^-24 of the row's absolute sum)
    bound = ref.abs() * 2.0**-8 + (x.double().abs() @ w.double().abs().t()) * (C_ * 2.0**-24) + 1e-30
    assert bool(((y.double() - ref).abs() <= bound).all())


@pytest.mark.parametrize("R,C_", [(300, 2560), (2560, 4096), (19456, 2560)])
def test_a_rows_bits_do_not_depend_on_the_pass_width(R, C_):
    g = torch.Generator(device=DEV).manual_seed(R)
    w = (torch.randn(R, C_, generator=g, device=DEV) * 0.05).bfloat16()
    x = torch.randn(32, C_, generator=g, device=DEV).bfloat16()
    wide = _run(w, x)
    again = _run(w, x)
    assert torch.equal(wide.view(torch.int16), again.view(torch.int16))  # the same bits every launch
    for m in (0, 7, 31):
        one = _run(w, x[m : m + 1].contiguous())
        assert torch.equal(one.view(torch.int16)[0], wide.view(torch.int16)[m])
    eight = _run(w, x[:8].contiguous())
    assert torch.equal(eight.view(torch.int16), wide.view(torch.int16)[:8])


def test_tc_gemv_agrees_with_the_chain_gemv_to_rounding():
    g = torch.Generator(device=DEV).manual_seed(1)
    R, C_, M = 2560, 2560, 8
    w = (torch.randn(R, C_, generator=g, device=DEV) * 0.02).bfloat16()
    x = torch.randn(M, C_, generator=g, device=DEV).bfloat16()
    y = _run(w, x)
    y2 = torch.zeros_like(y)
    call("btb_b200_gemv_bf16", ptr(w), ptr(x), ptr(y2), M, R, C_, capi.stream_ptr())
    d = (y.float() - y2.float()).abs()
    assert float(d.max()) <= 2.0**-7 * float(y2.float().abs().max())
    assert float((d > 0).float().mean()) < 0.5  # most outputs round to the same bf16


def test_tc_gemv_refuses_bad_arguments():
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    for M, R, C_ in ((0, 128, 64), (33, 128, 64), (1, 0, 64), (1, 128, 60)):
        with pytest.raises(capi.NativeError) as e:
            call("btb_b200_gemv_tc_bf16", ptr(w), ptr(w), ptr(w), M, R, C_, 0, 0)
        assert e.value.rc == capi.ERR_DOMAIN
    with pytest.raises(capi.NativeError):
        call("btb_b200_gemv_tc_bf16", 0, ptr(w), ptr(w), 1, 128, 64, 0, 0)
    big = torch.zeros(2560, 4096, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(capi.NativeError):  # a matrix of few tiles needs the partial sums' workspace
        call("btb_b200_gemv_tc_bf16", ptr(big), ptr(big), ptr(big), 1, 2560, 4096, 0, 0)


def test_launcher_serves_the_reference_mma_matvec():
    """btb_gemv_mma_bf16 by the reference's name and parameter list: the library's tensor-core kernel and - where the
    reference's kernels are built - the reference's own mma.sync kernel agree to rounding (two summation orders)"""
    from btb_b200 import launcher as L

    from . import refkernels

    R, C_, M = 2560, 4096, 5
    g = torch.Generator(device=DEV).manual_seed(3)
    w = (torch.randn(R, C_, generator=g, device=DEV) * 0.05).bfloat16()
    x = torch.zeros(32, C_, dtype=torch.bfloat16, device=DEV)
    x[:M] = torch.randn(M, C_, generator=g, device=DEV).bfloat16()
    y = torch.zeros(32, R, dtype=torch.bfloat16, device=DEV)
    L.btb_gemv_mma_bf16(L.B200Launcher(), ((R + 63) // 64, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(), y.data_ptr(), R, C_, M)
    torch.cuda.synchronize()
    ref = x[:M].double() @ w.double().t()
    assert float((y[:M].double() - ref).abs().max()) <= 2.0**-7 * float(ref.abs().max())
    assert float(y[M:].float().abs().max()) == 0.0  # rows past M are not written
    if not refkernels.available():
        return
    y2 = torch.zeros(32, R, dtype=torch.bfloat16, device=DEV)
    L.btb_gemv_mma_bf16(refkernels.RefLauncher(), ((R + 63) // 64, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(),
                        y2.data_ptr(), R, C_, M)  # fmt: skip
    torch.cuda.synchronize()
    assert float((y[:M].float() - y2[:M].float()).abs().max()) <= 2.0**-7 * float(ref.abs().max())


# ---- the prefill GEMM: the same kernel over tiles of up to 256 x rows ------------------------------------------------


def _gemm(w, x):
    T, (R, C_) = x.shape[0], w.shape
    y = torch.full((T, R), 7.0, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_gemm_tc_bf16", ptr(w), ptr(x), ptr(y), T, R, C_, capi.stream_ptr())
    torch.cuda.synchronize()
    assert capi.status() == 0
    return y


@pytest.mark.parametrize("R,C_", [(300, 2560), (2560, 4096), (6144, 2560), (129, 72), (2560, 9728)])
@pytest.mark.parametrize("T", [1, 40, 128, 200, 300, 700])
def test_prefill_gemm_rows_are_the_matvecs_rows(R, C_, T):
    """row t of a chunk of any size carries the bits the tensor-core matvec gives that row in a pass of its own: one
    accumulation over all of k in k order per output, whatever tile the row falls in"""
    g = torch.Generator(device=DEV).manual_seed(R + C_ + T)
    w = (torch.randn(R, C_, generator=g, device=DEV) * 0.05).bfloat16()
    x = torch.randn(T, C_, generator=g, device=DEV).bfloat16()
    y = _gemm(w, x)
    ref = x.double() @ w.double().t()
    bound = ref.abs() * 2.0**-8 + (x.double().abs() @ w.double().abs().t()) * (C_ * 2.0**-24) + 1e-30
    assert bool(((y.double() - ref).abs() <= bound).all())
    for a in sorted({0, max(0, T - 32), (T // 2) & ~31}):
        rows = x[a : a + 32].contiguous()
        assert torch.equal(_run(w, rows).view(torch.int16), y[a : a + rows.shape[0]].view(torch.int16)), a


def test_prefill_on_the_tensor_cores_leaves_the_chain_passes_cache():
    """`CardEngine.prefill_gemm` (GEMMs over chunks of 100 rows, the attention 32 rows at a time) writes the cache rows
    that 32-row tensor-core passes write, bit for bit, and its last row's logits agree with theirs to rounding"""
    from btb_b200 import engine as E

    cfg = E.DenseConfig("pf", hidden=256, layers=3, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=1000)
    mw = E.synth_weights(cfg, seed=2, on_cpu=True, layer_std=0.1)
    a, b = E.CardEngine(mw, cap=1024), E.CardEngine(mw, cap=1024)
    a.wide_tc = True
    prompt = torch.randint(0, cfg.vocab, (333,), generator=torch.Generator().manual_seed(5))
    la = a.prefill(prompt)
    lb = b.prefill_gemm(prompt, chunk=100)
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert int(a.n0[0]) == int(b.n0[0]) == 333
    assert torch.equal(a.K[:, :333].view(torch.int16), b.K[:, :333].view(torch.int16))
    assert torch.equal(a.V[:, :333].view(torch.int16), b.V[:, :333].view(torch.int16))
    assert float((la.float() - lb.float()).abs().max()) <= 2.0**-5 * float(la.float().abs().max())
    # decode goes on from either cache alike
    ta, tb = a.step(int(la.float().argmax())), b.step(int(la.float().argmax()))
    assert ta == tb


# ---- the gate/up form and the reference's other names ------------------------------------------------------------------


@pytest.mark.parametrize("I,C_", [(9728, 2560), (512, 256), (300, 264), (96, 4096), (768, 2048)])
@pytest.mark.parametrize("M", [1, 5, 32])
def test_glu_form_is_the_matvec_then_silu_mul(I, C_, M):
    """btb_b200_gemv_tc_glu_bf16 = btb_b200_gemv_tc_bf16 over the merged gate/up block + btb_b200_silu_mul, bit for bit
    (matrices of many tiles in one launch, of few tiles through K ranges and the ordered sum)"""
    g = torch.Generator(device=DEV).manual_seed(I + C_ + M)
    w = (torch.randn(2 * I, C_, generator=g, device=DEV) * 0.05).bfloat16()
    x = torch.randn(M, C_, generator=g, device=DEV).bfloat16()
    gu = _run(w, x)
    want = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    call("btb_b200_silu_mul", ptr(gu), ptr(want), M, I, capi.stream_ptr())
    got = torch.full((M, I), 3.0, dtype=torch.bfloat16, device=DEV)
    ws = _workspace(int(capi.lib().btb_b200_gemv_tc_glu_workspace_bytes(I, C_)))
    call("btb_b200_gemv_tc_glu_bf16", ptr(w), ptr(x), ptr(got), M, I, C_, ptr(ws), capi.stream_ptr())
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_launcher_serves_the_reference_mma8_and_glu_names():
    """btb_gemv_mma8_bf16 and btb_gemv_mma_glu_silu by the reference's names and parameter lists; beside the
    reference's own kernels (where built) they agree to rounding - two summation orders, as for the plain matvec"""
    from btb_b200 import launcher as L

    from . import refkernels

    R, C_, M, I = 1024, 2048, 3, 512
    g = torch.Generator(device=DEV).manual_seed(9)
    w = (torch.randn(R, C_, generator=g, device=DEV) * 0.05).bfloat16()
    x = torch.zeros(32, C_, dtype=torch.bfloat16, device=DEV)
    x[:M] = torch.randn(M, C_, generator=g, device=DEV).bfloat16()
    b200 = L.B200Launcher()
    y8, y16 = torch.zeros(32, R, dtype=torch.bfloat16, device=DEV), torch.zeros(32, R, dtype=torch.bfloat16, device=DEV)
    L.btb_gemv_mma8_bf16(b200, ((R + 31) // 32, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(), y8.data_ptr(), R, C_, M)
    L.btb_gemv_mma_bf16(b200, ((R + 63) // 64, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(), y16.data_ptr(), R, C_, M)
    assert torch.equal(y8.view(torch.int16), y16.view(torch.int16))  # the block's size moves no bit, here as there
    m = torch.zeros(32, I, dtype=torch.bfloat16, device=DEV)
    L.btb_gemv_mma_glu_silu(b200, ((I + 63) // 64, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(), m.data_ptr(), I, C_, M)
    torch.cuda.synchronize()
    gu = x[:M].double() @ w.double().t()
    ref = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    assert float((m[:M].double() - ref).abs().max()) <= 2.0**-6 * float(ref.abs().max())
    if not refkernels.available():
        return
    theirs = refkernels.RefLauncher()
    m2 = torch.zeros(32, I, dtype=torch.bfloat16, device=DEV)
    L.btb_gemv_mma_glu_silu(theirs, ((I + 63) // 64, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(), m2.data_ptr(), I, C_, M)
    y2 = torch.zeros(32, R, dtype=torch.bfloat16, device=DEV)
    L.btb_gemv_mma8_bf16(theirs, ((R + 31) // 32, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(), y2.data_ptr(), R, C_, M)
    torch.cuda.synchronize()
    assert float((m[:M].float() - m2[:M].float()).abs().max()) <= 2.0**-6 * float(ref.abs().max())
    assert float((y8[:M].float() - y2[:M].float()).abs().max()) <= 2.0**-7 * float(y2[:M].float().abs().max())


# ---- the tensor-core matvec over pack12 weights read as stored ------------------------------------------------------------


@pytest.mark.parametrize("R,Cc,dense", [(300, 2560, False), (2560, 9728, False), (19456, 2560, False), (200, 256, True),
                                        (129, 64, True), (6144, 2560, True)])  # fmt: skip
@pytest.mark.parametrize("M", [1, 8, 32])
def test_tc_matvec_over_pack12_equals_the_bf16_kernel_over_the_widened_matrix(R, Cc, dense, M):
    """the packed tile is widened on its way into the MMA's operand: the same bits in the same places as the bf16 tile
    TMA would have brought, so the same sums - escapes, partial tiles and K ranges included"""
    from btb_b200.engine import P12Matrix

    from .test_gpu_kernels import _p12_case, bf, bits, rand_bf

    rng = np.random.default_rng(R + Cc + M)
    wb, parts = _p12_case(rng, R, Cc, dense)
    if dense:
        assert parts[3].size > 0
    x = rand_bf(rng, (M, Cc))
    P = P12Matrix(parts, R, Cc, "cuda")
    wt, xt = bf(wb), bf(x)
    need = int(capi.lib().btb_b200_gemv_tc_workspace_bytes(R, Cc))
    ws = torch.full((max(need // 4, 4),), float("nan"), dtype=torch.float32, device="cuda")
    ws[:256] = 0  # (the head holds the tiles' counters: zero between launches)
    ya = torch.zeros(M, R, dtype=torch.bfloat16, device="cuda")
    yb = torch.full((M, R), 3.0, dtype=torch.bfloat16, device="cuda")
    call("btb_b200_gemv_tc_bf16", ptr(wt), ptr(xt), ptr(ya), M, R, Cc, ptr(ws), capi.stream_ptr())
    ws[256:].fill_(float("nan"))
    assert int(ws[:256].view(torch.int32).abs().sum()) == 0  # the counters are back at zero after a launch
    call("btb_b200_gemv_tc_p12", ptr(P.lo), ptr(P.hi4), P.table, ptr(P.esc_idx), ptr(P.esc_val), ptr(P.esc_row), ptr(xt), ptr(yb),
         M, R, Cc, ptr(ws), capi.stream_ptr())  # fmt: skip
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert torch.equal(ya.view(torch.int16), yb.view(torch.int16))
    # and it tracks the fp32-chain kernel to rounding, as the bf16 form does
    want = O.bits_to_f32(O.gemv_card_bf16(wb, x))
    got = yb.float().cpu().numpy()
    assert np.max(np.abs(got - want)) <= 2.0**-6 * max(1.0, float(np.max(np.abs(want))))


@pytest.mark.parametrize("R,Cc", [(2560, 9728), (6144, 2560), (2560, 4096), (300, 2560)])
@pytest.mark.parametrize("M", [1, 8, 32])
def test_adding_the_k_ranges_in_the_launch_gives_the_second_launchs_bits(R, Cc, M):
    """the `tc_fold` tunable: the CTA that arrives last on a tile's counter adds the ranges' partial sums in range order -
    the bits of the ordered second launch, for the bf16 and the pack12 kernel, and the counters stand at zero again
    afterwards (the same workspace serves the next launch as it is)"""
    from btb_b200.engine import P12Matrix

    from .test_gpu_kernels import _p12_case, bf, rand_bf

    rng = np.random.default_rng(7 * R + Cc + M)
    wb, parts = _p12_case(rng, R, Cc, False)
    x = rand_bf(rng, (M, Cc))
    P = P12Matrix(parts, R, Cc, "cuda")
    wt, xt = bf(wb), bf(x)
    need = int(capi.lib().btb_b200_gemv_tc_workspace_bytes(R, Cc))
    assert need > 1024  # these shapes are cut over K
    ws = torch.full((need // 4,), float("nan"), dtype=torch.float32, device="cuda")
    ws[:256] = 0

    def both(fold):
        capi.set_tuning(tc_fold=fold)
        try:
            ya = torch.full((M, R), 3.0, dtype=torch.bfloat16, device="cuda")
            yb = torch.full((M, R), 5.0, dtype=torch.bfloat16, device="cuda")
            for _ in range(2):  # twice over the same workspace: the counters were left at zero
                ws[256:].fill_(float("nan"))
                call("btb_b200_gemv_tc_bf16", ptr(wt), ptr(xt), ptr(ya), M, R, Cc, ptr(ws), capi.stream_ptr())
                call("btb_b200_gemv_tc_p12", ptr(P.lo), ptr(P.hi4), P.table, ptr(P.esc_idx), ptr(P.esc_val), ptr(P.esc_row),
                     ptr(xt), ptr(yb), M, R, Cc, ptr(ws), capi.stream_ptr())  # fmt: skip
            torch.cuda.synchronize()
            assert capi.status() == 0
            assert int(ws[:256].view(torch.int32).abs().sum()) == 0
            return ya, yb
        finally:
            capi.set_tuning(tc_fold=0)

    a0, b0 = both(0)
    a1, b1 = both(1)
    assert torch.equal(a0.view(torch.int16), a1.view(torch.int16))
    assert torch.equal(b0.view(torch.int16), b1.view(torch.int16))
    assert torch.equal(a1.view(torch.int16), b1.view(torch.int16))


def test_tc_p12_refusals():
    z = torch.zeros(64, 96, dtype=torch.uint8, device="cuda")
    x = torch.zeros(1, 96, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda")
    tab = bytes(16)
    with pytest.raises(capi.NativeError):  # C not a multiple of 64
        call("btb_b200_gemv_tc_p12", ptr(z), ptr(z), tab, 0, 0, 0, ptr(x), ptr(y), 1, 64, 96, 0, capi.stream_ptr())
    with pytest.raises(capi.NativeError):
        call("btb_b200_gemv_tc_p12", 0, ptr(z), tab, 0, 0, 0, ptr(x), ptr(y), 1, 64, 128, 0, capi.stream_ptr())
