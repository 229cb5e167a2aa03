"""The step's fused row (norm + RoPE + cache write + attention in one launch) leaves the bits the two separate kernels
leave: the cache rows, the query buffer and the attention output, over head shapes, cache lengths on both sides of
the tile and group boundaries, a window, a row map and sinks."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402

DEV = "cuda"


def _case(Hq, Hk, D, n0, cap, win=0, tbl=False, sinks=False, qk_norm=True, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, device=DEV)  # noqa: E731
    S = (cap + 511) // 512
    base = {
        "qkv": rnd(1, (Hq + 2 * Hk) * D).bfloat16(),
        "wq": (1 + 0.1 * rnd(D)).bfloat16() if qk_norm else None,
        "wk": (1 + 0.1 * rnd(D)).bfloat16() if qk_norm else None,
        "cos": torch.cos(rnd(cap, D)).bfloat16(), "sin": torch.sin(rnd(cap, D)).bfloat16(),
        "K": rnd(cap, Hk, D).bfloat16(), "V": rnd(cap, Hk, D).bfloat16(),
        "n0": torch.tensor([n0], dtype=torch.int32, device=DEV),
        "depth": torch.zeros(1, dtype=torch.int32, device=DEV),
        "par": torch.full((1,), -1, dtype=torch.int32, device=DEV),
        "tbl": torch.randperm(cap, generator=g, device=DEV).to(torch.int32) if tbl else None,
        "sinks": rnd(Hq) if sinks else None,
    }  # fmt: skip

    def fresh():
        d = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in base.items()}
        d.update(q=torch.zeros(1, Hq, D, dtype=torch.bfloat16, device=DEV),
                 att=torch.zeros(1, Hq * D, dtype=torch.bfloat16, device=DEV),
                 pm=torch.zeros(S * Hq, device=DEV), pl=torch.zeros(S * Hq, device=DEV),
                 pa=torch.zeros(S * Hq * D, device=DEV), cnt=torch.zeros(Hq, dtype=torch.int32, device=DEV))  # fmt: skip
        return d

    s = capi.stream_ptr()
    a, b = fresh(), fresh()
    hs, rs, scale = D, Hk * D, float(D**-0.5)
    call("btb_b200_norm_rope_kv", ptr(a["qkv"]), ptr(a["wq"]), ptr(a["wk"]), 1e-6, ptr(a["cos"]), ptr(a["sin"]),
         ptr(a["n0"]), ptr(a["depth"]), ptr(a["K"]), ptr(a["V"]), ptr(a["q"]), 1, Hq, Hk, D, hs, rs, 0, ptr(a["tbl"]), cap, s)  # fmt: skip
    call("btb_b200_attn_decode", ptr(a["q"]), ptr(a["K"]), ptr(a["V"]), ptr(a["att"]), ptr(a["n0"]), ptr(a["par"]), 1, Hq,
         Hk, D, hs, rs, scale, ptr(a["pm"]), ptr(a["pl"]), ptr(a["pa"]), ptr(a["cnt"]), win, ptr(a["tbl"]), ptr(a["sinks"]),
         cap, s)  # fmt: skip
    call("btb_b200_attn_step", ptr(b["qkv"]), ptr(b["wq"]), ptr(b["wk"]), 1e-6, ptr(b["cos"]), ptr(b["sin"]), ptr(b["n0"]),
         ptr(b["depth"]), ptr(b["K"]), ptr(b["V"]), ptr(b["q"]), ptr(b["att"]), Hq, Hk, D, hs, rs, 0, scale, ptr(b["pm"]),
         ptr(b["pl"]), ptr(b["pa"]), ptr(b["cnt"]), win, ptr(b["tbl"]), ptr(b["sinks"]), cap, s)  # fmt: skip
    torch.cuda.synchronize()
    assert capi.status() == 0
    for name in ("K", "V", "q", "att"):
        assert torch.equal(a[name].view(torch.int16), b[name].view(torch.int16)), name
    assert int(b["cnt"].abs().sum()) == 0  # the arrival counters are back at zero for the next launch
    assert float(a["att"].float().abs().max()) > 0


@pytest.mark.parametrize("Hq,Hk,D", [(32, 8, 128), (64, 8, 64), (8, 8, 128), (16, 8, 64), (32, 4, 128)])
@pytest.mark.parametrize("n0", [0, 1, 31, 32, 63, 64, 160, 511, 512, 513, 1023, 1024, 1500])
def test_fused_row_equals_the_two_kernels(Hq, Hk, D, n0):
    _case(Hq, Hk, D, n0, cap=2048, seed=n0 + Hq)


@pytest.mark.parametrize("Hq,Hk,D", [(32, 8, 128), (64, 8, 64), (8, 8, 128)])
@pytest.mark.parametrize("n0", [4095, 4096, 4097, 6000])
def test_fused_row_past_the_head_split(Hq, Hk, D, n0):
    """at 4096 cached rows the kernel goes from a block a query head to a block a kv head"""
    _case(Hq, Hk, D, n0, cap=6144, seed=n0 + Hq)


@pytest.mark.parametrize("n0", [5, 200, 700, 1100])
def test_fused_row_with_window_row_map_sinks_and_no_qk_norm(n0):
    _case(64, 8, 64, n0, cap=1536, win=128, sinks=True, qk_norm=False, seed=n0)
    _case(32, 8, 128, n0, cap=1536, tbl=True, seed=n0 + 1)
    _case(32, 8, 128, n0, cap=1536, win=600, tbl=True, sinks=True, seed=n0 + 2)


def test_fused_row_refuses_a_full_cache():
    Hq, Hk, D, cap = 8, 2, 128, 512
    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt, device=DEV)  # noqa: E731
    n0 = torch.tensor([cap], dtype=torch.int32, device=DEV)
    S = 1
    capi.status()
    call("btb_b200_attn_step", ptr(z(1, (Hq + 2 * Hk) * D)), 0, 0, 1e-6, ptr(z(cap, D)), ptr(z(cap, D)), ptr(n0),
         ptr(z(1, dt=torch.int32)), ptr(z(cap, Hk, D)), ptr(z(cap, Hk, D)), ptr(z(1, Hq, D)), ptr(z(1, Hq * D)), Hq, Hk, D,
         D, Hk * D, 0, 0.1, ptr(z(S * Hq, dt=torch.float32)), ptr(z(S * Hq, dt=torch.float32)),
         ptr(z(S * Hq * D, dt=torch.float32)), ptr(z(Hq, dt=torch.int32)), 0, 0, 0, cap, capi.stream_ptr())  # fmt: skip
    torch.cuda.synchronize()
    assert capi.status() == capi.ERR_DOMAIN


@pytest.mark.parametrize("Hq,Hk,D,H", [(32, 8, 128, 2560), (64, 8, 64, 2880), (8, 8, 128, 512)])
@pytest.mark.parametrize("n0", [0, 63, 160, 512, 1500, 4096, 5000])
def test_attention_and_projection_in_one_launch(Hq, Hk, D, H, n0):
    """btb_b200_attn_o_step leaves what btb_b200_attn_step then btb_b200_gemv_bf16 leave: cache, q, att and y"""
    cap = 6144
    gen = torch.Generator(device=DEV).manual_seed(n0 + Hq)
    rnd = lambda *s: torch.randn(*s, generator=gen, device=DEV)  # noqa: E731
    S = cap // 512
    qkv = rnd(1, (Hq + 2 * Hk) * D).bfloat16()
    wq, wk = (1 + 0.1 * rnd(D)).bfloat16(), (1 + 0.1 * rnd(D)).bfloat16()
    cos, sin = torch.cos(rnd(cap, D)).bfloat16(), torch.sin(rnd(cap, D)).bfloat16()
    K0, V0 = rnd(cap, Hk, D).bfloat16(), rnd(cap, Hk, D).bfloat16()
    wo = (rnd(H, Hq * D) * 0.05).bfloat16()
    n0t = torch.tensor([n0], dtype=torch.int32, device=DEV)
    depth = torch.zeros(1, dtype=torch.int32, device=DEV)
    bar = torch.zeros(2, dtype=torch.int32, device=DEV)

    def bufs():
        return dict(K=K0.clone(), V=V0.clone(), q=torch.zeros(1, Hq, D, dtype=torch.bfloat16, device=DEV),
                    att=torch.zeros(1, Hq * D, dtype=torch.bfloat16, device=DEV), y=torch.zeros(1, H, dtype=torch.bfloat16, device=DEV),
                    pm=torch.zeros(S * Hq, device=DEV), pl=torch.zeros(S * Hq, device=DEV), pa=torch.zeros(S * Hq * D, device=DEV),
                    cnt=torch.zeros(Hq, dtype=torch.int32, device=DEV))  # fmt: skip

    a, b = bufs(), bufs()
    s = capi.stream_ptr()
    scale = float(D**-0.5)
    call("btb_b200_attn_step", ptr(qkv), ptr(wq), ptr(wk), 1e-6, ptr(cos), ptr(sin), ptr(n0t), ptr(depth), ptr(a["K"]),
         ptr(a["V"]), ptr(a["q"]), ptr(a["att"]), Hq, Hk, D, D, Hk * D, 0, scale, ptr(a["pm"]), ptr(a["pl"]), ptr(a["pa"]),
         ptr(a["cnt"]), 0, 0, 0, cap, s)  # fmt: skip
    call("btb_b200_gemv_bf16", ptr(wo), ptr(a["att"]), ptr(a["y"]), 1, H, Hq * D, s)
    for _ in range(3):  # the barrier's generation carries over from launch to launch
        call("btb_b200_attn_o_step", ptr(qkv), ptr(wq), ptr(wk), 1e-6, ptr(cos), ptr(sin), ptr(n0t), ptr(depth),
             ptr(b["K"]), ptr(b["V"]), ptr(b["q"]), ptr(b["att"]), Hq, Hk, D, D, Hk * D, 0, scale, ptr(b["pm"]),
             ptr(b["pl"]), ptr(b["pa"]), ptr(b["cnt"]), 0, 0, cap, ptr(wo), ptr(b["y"]), H, ptr(bar), s)  # fmt: skip
    torch.cuda.synchronize()
    assert capi.status() == 0
    for name in ("K", "V", "q", "att", "y"):
        assert torch.equal(a[name].view(torch.int16), b[name].view(torch.int16)), name
    assert bar.tolist() == [0, 3]
