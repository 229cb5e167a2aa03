"""The tensor-parallel engine and its peer-store exchange on the card: one rank equals the plain engine; N ranks taking
turns on ONE GPU (tests/lockstep.py) equal it too - slices, offsets, arrival counts and the merged pick all at work;
a wait nobody answers gives up with ERR_TIMEOUT instead of hanging; and, when the box has them, two real GPUs equal one."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import capi  # noqa: E402
from btb_b200 import engine as E  # noqa: E402
from btb_b200 import parallel as P  # noqa: E402
from btb_b200.capi import call, ptr  # noqa: E402

from . import lockstep  # noqa: E402
from .util import LAYER_STD, lively  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def test_one_rank_tensor_parallel_engine_equals_the_plain_engine():
    cfg = E.DenseConfig("tp1", hidden=256, layers=2, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=640)
    prompt = torch.arange(5, 50)
    plain = E.CardEngine(E.synth_weights(cfg, seed=9, on_cpu=True, layer_std=LAYER_STD), cap=512, step_kernel=False)
    want = plain.generate_greedy(prompt, 12)
    lively(want)
    tp = P.TPEngine(cfg, P.shard_dense(E.synth_weights(cfg, seed=9, on_cpu=True, layer_std=LAYER_STD), 0, 1), 0, 1, cap=512)
    assert tp.generate_greedy(prompt, 12) == want  # prefill passes, then the captured step graph with its exchanges
    # the pass's logits too, bit for bit
    plain.reset()
    tp.reset()
    a, b = plain.forward(prompt[:20]), tp.forward(prompt[:20])
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert capi.status() == 0


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_taking_turns_on_one_gpu_equal_the_plain_engine(world):
    cfg = E.DenseConfig("tpN", hidden=256 * world, layers=3, q_heads=4 * world, kv_heads=world, head_dim=128,
                        inter=256 * world, vocab=160 * world)  # fmt: skip
    draw = lambda: E.synth_weights(cfg, seed=4, on_cpu=True, layer_std=LAYER_STD)  # noqa: E731
    plain = E.CardEngine(draw(), cap=512, step_kernel=False)
    prompt = torch.arange(3, 48) % cfg.vocab
    want = plain.generate_greedy(prompt, 16)
    lively(want)
    engs = lockstep.make(cfg, draw, world)
    got = lockstep.greedy(engs, prompt, 16)
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert all(g == want for g in got), (got, want)
    # a wide pass (the separate norm kernels, waits as launches of their own) and a narrow one: every rank's slice of
    # the logits is the plain engine's columns, bit for bit
    for T in (20, 3, 1):
        plain.reset()
        for e in engs:
            e.reset()
        full = plain.forward(prompt[:T])
        parts = lockstep.forward(engs, prompt[:T])
        assert torch.equal(torch.cat(parts, dim=1).view(torch.int16), full.view(torch.int16)), T
    # each rank's copy of an exchanged vector holds every rank's slice: the copies are equal
    for k in ("att_t", "yo_t", "m_t", "yd_t"):
        for e in engs[1:]:
            assert torch.equal(e.tp_bufs(1)[k].view(torch.int16), engs[0].tp_bufs(1)[k].view(torch.int16)), k
    assert capi.status() == 0


@pytest.mark.parametrize("world,fmt,layers", [(2, "fp8", 2), (4, "mx4", 3)])
def test_expert_parallel_ranks_taking_turns_equal_one_gpu(world, fmt, layers):
    """experts cut over ranks (expert e on rank e % world), the products exchanged as marked words: every rank's logits
    are the one-GPU engine's, bit for bit; three layers make the buffers' rotation (2, then the odd last one) show"""
    from btb_b200 import moe as MO

    cfg = MO.MoEConfig("ep", 256, layers, 8, 2, 128, 128, 512, experts=8, top_k=4, router_mode=0 if fmt == "fp8" else 1,
                       glu_kind=0 if fmt == "fp8" else 1, expert_fmt=fmt)  # fmt: skip
    one = MO.MoEEngine(MO.synth_moe_weights(cfg, seed=6, on_cpu=True, layer_std=LAYER_STD), cap=512)
    prompt = torch.arange(3, 48)
    want = one.generate_greedy(prompt, 14)
    lively(want)
    engs = lockstep.make_moe(cfg, world, 6, LAYER_STD)
    got = lockstep.moe_greedy(engs, prompt, 14)
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert all(g == want for g in got), (got, want)
    for T in (20, 1):
        one.reset()
        for e in engs:
            e.reset()
        full = one.forward(prompt[:T])
        for lg in lockstep.moe_forward(engs, prompt[:T]):
            assert torch.equal(lg.view(torch.int16), full.view(torch.int16)), T
    assert capi.status() == 0


def test_a_vector_nobody_sends_gives_up():
    """a consumer whose producers never write (a peer that died between steps) returns after about a second with
    ERR_TIMEOUT in the status word; the context stays usable"""
    words = torch.zeros(1, 64, dtype=torch.int32, device="cuda")
    dst = torch.zeros(1, 64, dtype=torch.bfloat16, device="cuda")
    pas = torch.zeros(1, dtype=torch.int32, device="cuda")
    r = capi.Recv(ptr(pas), 4, 3)  # awaits words marked 0 * 4 + 3
    call("btb_b200_xchg_unpack", ptr(words), ptr(dst), 1, 64, r, capi.stream_ptr())
    torch.cuda.synchronize()
    assert capi.status() == capi.ERR_TIMEOUT
    # the words in (one rank sending to itself): the same take returns at once with the elements
    src = torch.arange(64, dtype=torch.float32, device="cuda").to(torch.bfloat16).reshape(1, 64)
    s = capi.Send()
    s.out[0], s.n, s.stride, s.offset, s.pass_, s.per_pass, s.base = ptr(words), 1, 64, 0, ptr(pas), 4, 3
    call("btb_b200_xchg_send", ptr(src), 1, 64, s, capi.stream_ptr())
    call("btb_b200_xchg_unpack", ptr(words), ptr(dst), 1, 64, r, capi.stream_ptr())
    torch.cuda.synchronize()
    assert capi.status() == 0 and torch.equal(dst, src)
    assert int(words[0, 5]) == (3 << 16) | int(src.view(torch.int16)[0, 5])
    with pytest.raises(capi.NativeError):  # a slice that does not fit its vector is refused on the host
        s.offset = 32
        call("btb_b200_xchg_send", ptr(src), 1, 64, s, capi.stream_ptr())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_one_gpu():
    n = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "mp_gpu_check.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0 and "multi-gpu ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
