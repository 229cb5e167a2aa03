"""The C-ABI without a GPU: the library loads, exports every symbol the header declares, the Python binding types
every one of them, and argument checks that need no device answer with the header's codes."""

import ctypes as C
import os
import re

import pytest

from btb_b200 import build as B
from btb_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "btb_b200.h")


def declared() -> dict[str, int]:
    """function name -> parameter count, read off the header"""
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    out = {}
    for m in re.finditer(r"\b(?:int|size_t|void\s*\*|void)\s*(btb_b200_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        params = m.group(2).strip()
        out[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    return out


@pytest.fixture(scope="module")
def lib():
    B.build()
    return capi.lib()


def test_header_binding_and_library_agree(lib):
    decl = declared()
    assert len(decl) >= 15
    assert set(decl) == set(capi.SIGNATURES), set(decl) ^ set(capi.SIGNATURES)
    for name, n in decl.items():
        assert hasattr(lib, name), f"{name} is declared but not exported"
        assert len(capi.SIGNATURES[name][1]) == n, name


def test_every_declaration_cites_the_reference():
    text = open(HEADER).read()
    for name in declared():
        if name in ("btb_b200_version", "btb_b200_sm_count", "btb_b200_set_tuning", "btb_b200_status"):
            continue
        at = text.index(name + "(")
        comment = text[text.rfind("/*", 0, at) : at]
        assert (re.search(r"\.(cu|cuh|rs|py):\d+", comment) or "btb_b200_" in comment
                or "no counterpart in the reference" in comment), name


def test_host_side_argument_checks(lib):
    assert lib.btb_b200_version() >= 1
    # null pointers and bad shapes are refused before anything touches a device
    assert lib.btb_b200_gemv_bf16(None, None, None, 1, 4, 16, None) == capi.ERR_NULL
    buf = C.create_string_buffer(64)
    p = C.addressof(buf)
    p16 = (p + 15) & ~15
    assert lib.btb_b200_gemv_bf16(p16, p16, p16, 3, 4, 16, None) == capi.ERR_DOMAIN  # M not a pass width
    assert lib.btb_b200_gemv_bf16(p16, p16, p16, 1, 4, 12, None) == capi.ERR_DOMAIN  # C not a multiple of 8
    assert lib.btb_b200_gemv_bf16(p16 + 2, p16, p16, 1, 4, 16, None) == capi.ERR_DOMAIN  # misaligned weights
    assert lib.btb_b200_gemv_p12(p16, p16, p16, None, None, None, p16, p16, 1, 4, 40, None) == capi.ERR_DOMAIN
    assert lib.btb_b200_add_rmsnorm(None, None, None, 1e-6, None, 1, 8, 0, None) == capi.ERR_NULL
    assert lib.btb_b200_attn_decode(*([p16] * 6), 1, 6, 4, 128, 128, 512, 0.1, p16, p16, p16, p16, 0, None, None, 512,
                                    None) == capi.ERR_DOMAIN  # 6 query heads over 4 kv heads
    assert lib.btb_b200_set_tuning(b"no_such_knob", 1) == capi.ERR_DOMAIN
    assert lib.btb_b200_set_tuning(None, 1) == capi.ERR_NULL


def test_binding_raises_the_reference_error_types(lib):
    with pytest.raises(capi.NativeError) as e:
        capi.call("btb_b200_gemv_bf16", 0, 0, 0, 1, 4, 16, 0)
    assert e.value.rc == capi.ERR_NULL and "btb_b200_gemv_bf16" in str(e.value)
    import torch

    with pytest.raises(capi.NativeDtypeError):
        capi.need(torch.zeros(2, dtype=torch.float32), torch.bfloat16, "weights")


def test_engine_fails_loudly_without_a_device():
    import torch

    from btb_b200 import engine as E

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    cfg = E.DenseConfig("t", 64, 1, 2, 1, 128, 64, 128)
    with pytest.raises((RuntimeError, AssertionError)):
        E.CardEngine(E.synth_weights(cfg, on_cpu=True, device="cpu"), cap=512, device="cpu")


def test_oracle_pack12_encoder_equals_the_reference_encoders_bytes(golden_dir):
    """the oracle's restatement of the encoder against the parts the reference's own encoder wrote (the card's encoder is
    checked against both in the GPU tests)"""
    import numpy as np

    from oracle import oracle as O

    g = np.load(os.path.join(golden_dir, "codecs.npz"))
    for case in "abcd":
        src = g[f"p12_{case}_src"]
        parts = O.pack_p12(src)
        for mine, name in zip(parts, ("lo", "hi4", "tbl", "esc_idx", "esc_val")):
            assert np.array_equal(mine, g[f"p12_{case}_{name}"]), (case, name)
        assert np.array_equal(O.widen_p12(*parts, src.size), src.reshape(-1))
