"""run under torchrun on 2+ GPUs (tests/test_gpu_parallel.py launches it): tensor-parallel dense and expert-parallel MoE
greedy tokens must equal the one-GPU engines' tokens"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from btb_b200 import engine as E  # noqa: E402
from tests.util import LAYER_STD, lively  # noqa: E402
from btb_b200 import moe as MO  # noqa: E402
from btb_b200 import parallel as P  # noqa: E402


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    prompt = torch.arange(3, 48)
    cfg = E.DenseConfig("tp-check", hidden=256 * world, layers=2, q_heads=4 * world, kv_heads=world, head_dim=128,
                        inter=512 * world, vocab=512 * world)
    full = E.synth_weights(cfg, seed=4, on_cpu=True, layer_std=LAYER_STD)
    want = E.CardEngine(full, cap=512, step_kernel=False).generate_greedy(prompt, 16)
    lively(want)
    tp = P.TPEngine(cfg, P.shard_dense(E.synth_weights(cfg, seed=4, on_cpu=True, layer_std=LAYER_STD), rank, world), rank, world, cap=512)
    got = tp.generate_greedy(prompt, 16)
    assert got == want, (rank, got, want)
    mcfg = MO.MoEConfig("ep-check", 256, 2, 8, 2, 128, 128, 512, experts=8 * world, top_k=4, router_mode=0, glu_kind=0,
                        expert_fmt="fp8")
    want = MO.MoEEngine(MO.synth_moe_weights(mcfg, seed=6, on_cpu=True, layer_std=LAYER_STD), cap=512).generate_greedy(prompt, 16)
    lively(want)
    ep = MO.MoEEngine(MO.synth_moe_weights(mcfg, seed=6, on_cpu=True, layer_std=LAYER_STD, ep_rank=rank, ep_size=world), cap=512)  # noqa: E501
    got = ep.generate_greedy(prompt, 16)
    assert got == want, (rank, got, want)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("multi-gpu ok", world, flush=True)
    # leave without tearing the communicator down collectively: every rank is past its last collective
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
