"""Tensor-parallel and expert-parallel engines on the card: one rank equals the plain engine; two or more ranks (when
the box has them) equal one GPU's tokens."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from btb_b200 import engine as E  # noqa: E402
from .util import LAYER_STD, lively  # noqa: E402
from btb_b200 import parallel as P  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def test_one_rank_tensor_parallel_engine_equals_the_plain_engine():
    cfg = E.DenseConfig("tp1", hidden=256, layers=2, q_heads=8, kv_heads=2, head_dim=128, inter=512, vocab=640)
    prompt = torch.arange(5, 50)
    plain = E.CardEngine(E.synth_weights(cfg, seed=9, on_cpu=True, layer_std=LAYER_STD), cap=512, step_kernel=False)
    want = plain.generate_greedy(prompt, 12)
    lively(want)
    tp = P.TPEngine(cfg, P.shard_dense(E.synth_weights(cfg, seed=9, on_cpu=True, layer_std=LAYER_STD), 0, 1), 0, 1, cap=512)
    assert tp.generate_greedy(prompt, 12) == want
    # the pass's logits too, bit for bit
    plain.reset()
    tp.reset()
    a, b = plain.forward(prompt[:20]), tp.forward(prompt[:20])
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_one_gpu():
    n = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "mp_gpu_check.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0 and "multi-gpu ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
