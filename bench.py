"""Decode benchmark of the B200 hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
                    [--workload qwen3-4b-bf16|qwen3-4b-p12|gpt-oss-20b|qwen3-30b-a3b|llama-70b]
                    [--batch B [--wide-tc 0|1]] [--speculative N] [--case gemv:RxC[:M[:fmt]]|attn:N|moe:fp8|moe:mx4|sample:V]

A step is one greedy decode step (one token) at batch 1 of the Qwen3-4B-shaped model with seeded random bf16 weights
(N(0, 0.02), norm weights 1) after a 128-token uniform-random prompt: the configuration the metric is quoted on.
Rank 0 prints ONE JSON line. `value` is tokens/s with everything resident on the card (CUDA events around K replays of
the captured step graph, max over ranks); `e2e` is the same through the public one-token call with the token crossing
the bus both ways every step; `roofline` is the GEMV kernel's achieved weight-streaming rate (CUDA events around one
token's worth of GEMV launches over the model's real weights, 8 GB >> L2) against the measured HBM copy peak;
`cpu_baseline` is the CPU tier's arithmetic (oracle port of btb's 16-lane AVX-512 GEMV, all host cores) on the same
model. With --impl reference the CPU tier is the thing timed.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bf16 decode tok/s @bs1 (Qwen3-4B shape)"
PROMPT = 128
# each configuration's own prompt length (config 5's 32768 rows stand in the cache as seeded synthetic rows)
PROMPTS = {"qwen3-4b-bf16": 128, "qwen3-4b-p12": 2048, "gpt-oss-20b": 1024, "qwen3-30b-a3b": 512, "llama-70b": 128}


def measured_hbm_peak() -> tuple[float, str]:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class Clocks:
    """samples nvidia-smi while the timed region runs"""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, index: int):
        self.rows: list[list[str]] = []
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )  # fmt: skip
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].startswith("Active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}  # fmt: skip


# ---- the CPU tier (oracle port of btb's CPU path) -------------------------------------------------------------------


def cpu_tier_step_fn(cfg, host_w):
    """one decode step on the host: f32 activations over bf16 weights, 16-lane GEMV on every core (the arithmetic of
    btb's CPU tier, btb/engine/host.py:98-134 -> native/src/gemv.rs), a numpy attention over an f32 cache"""
    import numpy as np

    from oracle import oracle as O

    H, D, Hq, Hk = cfg.hidden, cfg.head_dim, cfg.q_heads, cfg.kv_heads
    cap = 512
    K = np.zeros((cfg.layers, Hk, cap, D), np.float32)
    V = np.zeros_like(K)
    inv = (1.0 / (np.float32(cfg.theta) ** (np.arange(0, D, 2, dtype=np.float32) / np.float32(D)))).astype(np.float32)
    state = {"n": PROMPT}

    def rms(x, eps):
        return x * (1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + np.float32(eps)))

    def step(tok: int) -> int:
        n = state["n"]
        h = O.bits_to_f32(host_w["embed"][tok : tok + 1])
        ang = np.float32(n) * inv
        cos, sin = np.cos(np.concatenate([ang, ang])), np.sin(np.concatenate([ang, ang]))
        rot = lambda a: np.concatenate([-a[..., D // 2 :], a[..., : D // 2]], -1)  # noqa: E731
        for i in range(cfg.layers):
            L = host_w["layers"][i]
            x = rms(h, cfg.eps).astype(np.float32)
            qkv = O.cpu_gemv_bf16(L["qkv"], x)[0]
            q = rms(qkv[: Hq * D].reshape(Hq, D), cfg.eps)
            k = rms(qkv[Hq * D : (Hq + Hk) * D].reshape(Hk, D), cfg.eps)
            v = qkv[(Hq + Hk) * D :].reshape(Hk, D)
            q, k = q * cos + rot(q) * sin, k * cos + rot(k) * sin
            K[i, :, n], V[i, :, n] = k, v
            G = Hq // Hk
            s = np.einsum("gud,gnd->gun", q.reshape(Hk, G, D), K[i, :, : n + 1]) * np.float32(D**-0.5)
            p = np.exp(s - s.max(-1, keepdims=True))
            att = np.einsum("gun,gnd->gud", p / p.sum(-1, keepdims=True), V[i, :, : n + 1]).reshape(1, Hq * D)
            h = h + O.cpu_gemv_bf16(L["o"], att.astype(np.float32))
            x = rms(h, cfg.eps).astype(np.float32)
            gu = O.cpu_gemv_bf16(L["gu"], x)[0]
            g, u = gu[: cfg.inter], gu[cfg.inter :]
            m = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)[None]
            h = h + O.cpu_gemv_bf16(L["down"], m)
        x = rms(h, cfg.eps).astype(np.float32)
        logits = O.cpu_gemv_bf16(host_w["embed"], x)[0]
        state["n"] = n + 1
        return int(np.argmax(logits))

    return step


def host_weights_from_engine(mw):
    import numpy as np
    import torch

    def b(t):
        return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)

    return {"embed": b(mw.embed),
            "layers": [{"qkv": b(L.qkv), "o": b(L.o), "gu": b(L.gu), "down": b(L.down)} for L in mw.layers]}  # fmt: skip


def host_weights_synth(cfg, seed=0):
    """the same shapes and distribution drawn on the host (the reference arm needs no card)"""
    import numpy as np
    import torch

    g = torch.Generator().manual_seed(seed)

    def lin(r, c):
        t = torch.empty(r, c, dtype=torch.bfloat16)
        t.normal_(0.0, 0.02, generator=g)
        return t.view(torch.int16).numpy().view(np.uint16)

    H, D = cfg.hidden, cfg.head_dim
    out = {"embed": lin(cfg.vocab, H), "layers": []}
    for _ in range(cfg.layers):
        out["layers"].append({"qkv": lin(cfg.qkv_rows, H), "o": lin(H, cfg.q_heads * D), "gu": lin(2 * cfg.inter, H),
                              "down": lin(H, cfg.inter)})  # fmt: skip
    return out


def time_cpu_tier(cfg, host_w, steps: int, warmup: int = 1) -> tuple[float, int]:
    from oracle import oracle as O

    O.build()
    step = cpu_tier_step_fn(cfg, host_w)
    tok = 1
    for _ in range(warmup):
        tok = step(tok)
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = step(tok)
    dt = time.perf_counter() - t0
    return steps / dt, os.cpu_count() or 1


# ---- arms ---------------------------------------------------------------------------------------------------------------


def run_reference(args, rank: int) -> None:
    from btb_b200.engine import QWEN3_4B as cfg

    if rank != 0:
        return
    hw = host_weights_synth(cfg)
    steps = max(1, min(args.steps, 64))
    tps, cores = time_cpu_tier(cfg, hw, steps, warmup=args.warmup)
    from oracle import oracle as O

    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 / tps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 activations over bf16 weights", "data": "synthetic",
        # the same workload record as the GPU arm's: what differs (the CPU tier, its cores) is in cpu_baseline
        "config": {"workload": f"{cfg.name}-shape bf16, batch 1, greedy decode after a 128-token prompt",
                   "parallelism": "1 device", "graph_steps": 1, "step_kernel": 0,
                   "l2": f"weights a rank streams per step {cfg.weight_bytes_per_token('bf16') / 1e9:.2f} GB > L2 126 MB (inputs "
                         "larger than L2)", "pdl": None, "prefill": None, "bytes_per_token": cfg.weight_bytes_per_token("bf16")},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": cores, "kind": "port",
                         "sample": f"{steps} full decode steps, isa {O.isa()}"},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def tp_synth_shard(cfg, rank: int, world: int):
    """this rank's share of a seeded dense model, drawn shard by shard on the card (the whole model may not fit one
    GPU): every rank draws the same per-tensor streams and keeps its rows"""
    import torch

    from btb_b200 import engine as E
    from btb_b200 import parallel as P

    def lin(seed: int, r: int, c: int, lo: int, hi: int):
        g = torch.Generator(device="cuda").manual_seed(seed)
        out = torch.empty(hi - lo, c, dtype=torch.bfloat16, device="cuda")
        step = 4096
        for a in range(0, r, step):  # draw in row blocks, keep the overlap with [lo, hi)
            b = min(r, a + step)
            blk = (torch.randn(b - a, c, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
            x, y = max(a, lo), min(b, hi)
            if x < y:
                out[x - lo : y - lo] = blk[x - a : y - a]
        return out

    H, D, I = cfg.hidden, cfg.head_dim, cfg.inter
    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device="cuda")  # noqa: E731
    vl, vh = P.row_shard(cfg.vocab, rank, world)
    hl, hh = P.row_shard(H, rank, world)
    il, ih = P.row_shard(I, rank, world)
    ql, qh = P.row_shard(cfg.q_heads * D, rank, world)
    kl, kh = P.row_shard(cfg.kv_heads * D, rank, world)
    table = lin(1, cfg.vocab, H, 0, cfg.vocab)  # the embedding table whole on every rank; the head is this rank's rows of it
    mw = E.ModelWeights(cfg, table, ones(H), head=table[vl:vh])
    for i in range(cfg.layers):
        s0 = 100 + 10 * i
        qkv = torch.cat([lin(s0, cfg.q_heads * D, H, ql, qh), lin(s0 + 1, cfg.kv_heads * D, H, kl, kh),
                         lin(s0 + 2, cfg.kv_heads * D, H, kl, kh)])
        gu = torch.cat([lin(s0 + 4, I, H, il, ih), lin(s0 + 5, I, H, il, ih)])
        mw.layers.append(E.LayerWeights(ones(H), ones(H), qkv, lin(s0 + 3, H, cfg.q_heads * D, hl, hh), gu,
                                        lin(s0 + 6, H, I, hl, hh), ones(D) if cfg.qk_norm else None,
                                        ones(D) if cfg.qk_norm else None))
    return mw


def run_b200(args, rank: int, world: int, local_rank: int) -> None:
    import torch

    from btb_b200 import capi
    from btb_b200 import engine as E

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist  # noqa: PLC0415

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import dataclasses

    K, W = args.steps, max(args.warmup, 3)
    n_prompt = args.prompt or PROMPTS[args.workload]
    cap = (((512 if args.speculative else n_prompt) + 2 * (K + W) + 96 + 511) // 512) * 512
    storage, parallelism = "bf16", ("replicas only" if world > 1 else "1 device")
    if args.pdl is not None:
        capi.set_tuning(pdl=args.pdl)
    if args.l2_warm_kb is not None:
        capi.set_tuning(l2_warm_kb=args.l2_warm_kb)
    if args.l2_warm_ctas is not None:
        capi.set_tuning(l2_warm_ctas=args.l2_warm_ctas)
    if args.workload == "qwen3-4b-bf16" and world > 1 and args.batch == 1 and not args.replicas:
        # one model over the ranks: every linear cut by output rows, one token stream (strong scaling)
        from btb_b200 import parallel as P

        cfg = E.QWEN3_4B if not args.layers else dataclasses.replace(E.QWEN3_4B, layers=args.layers)
        mw = tp_synth_shard(cfg, rank, world)
        eng = P.TPEngine(cfg, mw, rank, world, cap=cap)
        parallelism = f"tp{world}"
    elif args.workload.startswith("qwen3-4b"):
        cfg = E.QWEN3_4B if not args.layers else dataclasses.replace(E.QWEN3_4B, layers=args.layers)
        storage = "p12" if args.workload.endswith("p12") else "bf16"
        mw = E.synth_weights(cfg, seed=0, storage=storage)
        if args.batch > 1:
            run_batch(args, mw, cfg, storage, cap, rank, world, dist)
            return
        eng = E.CardEngine(mw, cap=cap, step_kernel=bool(args.step_kernel))
    elif args.workload in ("gpt-oss-20b", "qwen3-30b-a3b"):
        from btb_b200 import moe as MO

        cfg = MO.GPT_OSS_20B if args.workload == "gpt-oss-20b" else MO.QWEN3_30B_A3B
        if args.layers:
            cfg = dataclasses.replace(cfg, layers=args.layers)
        storage = cfg.expert_fmt
        mw = MO.synth_moe_weights(cfg, seed=0, ep_rank=rank, ep_size=world)
        eng = MO.MoEEngine(mw, cap=cap)
        parallelism = f"ep{world}" if world > 1 else "1 device"
    else:
        from btb_b200 import parallel as P

        cfg = E.LLAMA31_70B if not args.layers else dataclasses.replace(E.LLAMA31_70B, layers=args.layers)
        ctx = args.context or 32768
        cap = ((ctx + 2 * (K + W) + 64 + 511) // 512) * 512
        shard = tp_synth_shard(cfg, rank, world)
        eng = P.TPEngine(cfg, shard, rank, world, cap=cap)
        mw = shard
        parallelism = f"tp{world}" if world > 1 else "1 device"
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (n_prompt,), generator=g)
    prefill = None
    eng.reset()
    if args.speculative:
        run_speculative(args, eng, cfg, storage, parallelism, rank, world, dist)
        return
    if args.workload == "llama-70b":
        # the metric excludes prefill: the 32768-row context is seeded synthetic cache rows (bf16 N(0, 1)), not a
        # prefilled prompt - a chain-pass prefill of that length through the decode kernels would take minutes
        ctx = args.context or 32768
        gk = torch.Generator(device="cuda").manual_seed(1)
        for i in range(cfg.layers):
            eng.K[i][:ctx].normal_(generator=gk)
            eng.V[i][:ctx].normal_(generator=gk)
        eng.n0.fill_(ctx)
        eng.bufs(1)["ids"][0] = 1
    else:
        # the prompt is really prefilled (outside the timed region: the metric is the rate after the first token): on the
        # tensor cores where the engine has the GEMM path (one GPU, bf16 weights), else by chain passes of 32 rows
        gemm = args.prefill == "gemm" or (args.prefill == "auto" and type(eng) is E.CardEngine and storage == "bf16"
                                          and n_prompt >= 256)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        last = eng.prefill_gemm(prompt) if gemm else eng.prefill(prompt)
        torch.cuda.synchronize()
        prefill = {"tokens": n_prompt, "ms": (time.perf_counter() - t0) * 1000.0,
                   "how": "tensor-core GEMMs over 256-row chunks (tcgen05)" if gemm else "chain passes of 32 rows"}
        first = int(last.float().argmax(-1)) if not hasattr(eng, "tp_bufs") else 1
        eng.bufs(1)["ids"][0] = first
    graph = eng.step_graph(args.graph_steps, publish=True)
    reps = lambda n: -(-n // args.graph_steps)  # noqa: E731

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(reps(W)):
        graph.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with Clocks(local_rank) as clk:
        e0.record()
        for _ in range(reps(K)):
            graph.replay()
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    steps_done = reps(K) * args.graph_steps
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    assert capi.status() == 0, "a kernel recorded a device-side refusal"
    tps = world * steps_done / (ms / 1000.0)

    # e2e: the public one-token call, the token crossing the bus both ways every step
    tok = int(eng.pin_tok[0])
    for _ in range(3):
        tok = eng.step(tok)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        tok = eng.step(tok)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t[0])
    e2e = world * K / e2e_s

    # roofline: one token's GEMV launches - the variants the step itself launches (norm folded into the qkv, gate/up and
    # head GEMVs, SwiGLU in the gate/up GEMV's epilogue) - over the model's own weights, nothing else on the stream
    dense_model = args.workload.startswith("qwen3-4b") and not hasattr(eng, "tp_bufs")
    peak, which = measured_hbm_peak()
    roof = gemv_roofline(eng, mw, cfg, storage, peak, which) if dense_model else None

    line = {
        "metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": world, "steps": steps_done, "warmup": W,
        "ms_per_step": ms / steps_done, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if storage == "bf16" else f"bf16 ({STORED.get(storage, storage)} weights widened in registers)",
        "data": "synthetic",
        "config": {"workload": f"{cfg.name}-shape {storage}, batch 1, greedy decode after a {n_prompt}-token prompt"
                   if args.workload != "llama-70b" else f"{cfg.name}-shape bf16, batch 1, greedy decode over a "
                   f"{args.context or 32768}-row synthetic cache (seeded rows, not a prefilled prompt)",
                   "parallelism": parallelism, "graph_steps": args.graph_steps, "step_kernel": args.step_kernel,
                   "l2": f"weights a rank streams per step {cfg.weight_bytes_per_token(storage) / max(1, world if parallelism.startswith(('tp', 'ep')) else 1) / 1e9:.2f}"
                         " GB > L2 126 MB (inputs larger than L2)", "pdl": args.pdl,
                   "prefill": prefill if n_prompt != 128 else None,
                   "bytes_per_token": cfg.weight_bytes_per_token(storage)},
        "clocks": clk.summary(),
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8},
        "gpu_launches": eng.launches_per_step * steps_done,
        "roofline": roof,
        "token_roofline_frac": (cfg.weight_bytes_per_token(storage) * tps / world / 1e9) / peak,
    }  # fmt: skip
    if not dense_model:
        line["roofline"] = None
        line["metric"] = f"decode tok/s @bs1 ({cfg.name} shape)"
    if args.workload != "qwen3-4b-bf16" and args.workload.startswith("qwen3-4b"):
        line["metric"] = "decode tok/s @bs1 (Qwen3-4B shape, pack12 weights)"
    if world > 1 and parallelism != "replicas only":
        line["value"] = tps / world  # one model over all ranks: the job decodes one stream
        line["e2e"]["value"] = e2e / world
        line["scaling"] = "strong"
        line["token_roofline_frac"] = (cfg.weight_bytes_per_token(storage) / world * (tps / world) / 1e9) / peak
        if hasattr(eng, "tp_bufs"):
            line["roofline"] = None
            if args.workload == "qwen3-4b-bf16":
                line["metric"] = METRIC
            line["collective"] = tp_collective(eng, cfg, world, dist)
    if rank == 0 and world == 1 and not args.no_cpu and args.workload == "qwen3-4b-bf16":
        hw = host_weights_from_engine(mw) if storage == "bf16" else host_weights_synth(cfg)
        from oracle import oracle as O

        ctps, cores = time_cpu_tier(cfg, hw, steps=args.cpu_steps, warmup=1)
        line["cpu_baseline"] = {"value": ctps, "unit": "tok/s", "cores": cores, "kind": "port",
                                "sample": f"{args.cpu_steps} full decode steps of the same model, isa {O.isa()}"}  # fmt: skip
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        # every rank is past its last collective: leave without a collective teardown
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


STORED = {"p12": "pack12", "mx4": "MXFP4 expert", "fp8": "FP8 block-scaled"}


def gemv_roofline(eng, mw, cfg, storage, peak, which) -> dict:
    """CUDA events around the step's own GEMV launches over the model's own matrices (36 distinct matrices a kind: far
    past L2): the five kinds one after another as the step orders them (the `achieved` figure: algorithmic bytes of all
    145 launches over their time) and each kind alone (the split)"""
    import torch

    from btb_b200 import capi
    from btb_b200 import engine as E
    from btb_b200.capi import call, ptr

    g = eng.bufs(1)
    s = capi.stream_ptr()
    H, A, I, V = cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.inter, cfg.vocab

    def parts(W):
        if isinstance(W, E.P12Matrix):
            return (ptr(W.lo), ptr(W.hi4), W.table, ptr(W.esc_idx), ptr(W.esc_val), ptr(W.esc_row))
        return (ptr(W), 0, 0, 0, 0, 0)

    def normed(W, nw, out, R, swiglu=False):
        call("btb_b200_gemv_norm_swiglu" if swiglu else "btb_b200_gemv_norm", *parts(W), ptr(g["h"]), ptr(g["y"]), ptr(nw),
             cfg.eps, 0, ptr(g["h2"]), ptr(out), 1, 1, R, H, capi.stream_ptr())

    kinds = {
        "qkv (norm folded in)": lambda L: normed(L.qkv, L.ln1, g["qkv"], cfg.qkv_rows),
        "o": lambda L: eng._matvec(L.o, g["att"], g["y"], 1, H, A, capi.stream_ptr()),
        "gate/up (norm in, SwiGLU out)": lambda L: normed(L.gu, L.ln2, g["m"], 2 * I, True),
        "down": lambda L: eng._matvec(L.down, g["m"], g["y"], 1, H, I, capi.stream_ptr()),
    }
    bpw = 2.0 if storage == "bf16" else 1.5
    shape = {"qkv (norm folded in)": (cfg.qkv_rows, H), "o": (H, A), "gate/up (norm in, SwiGLU out)": (2 * I, H), "down": (H, I)}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, rounds=5):
        """ms a round of `fn`'s launches, replayed as a captured graph (as the step runs them: no host launch gaps)"""
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(2):
            graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(rounds):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return max(e0.elapsed_time(e1) / rounds, 1e-6)

    def whole():
        for L in mw.layers:
            for f in kinds.values():
                f(L)
        normed(mw.embed, mw.norm, g["logits"], V)

    split = {}
    for name, f in kinds.items():
        ms = timed(lambda f=f: [f(L) for L in mw.layers])
        R, C_ = shape[name]
        by = R * C_ * bpw + 2 * (C_ + (R // 2 if "SwiGLU" in name else R))
        split[name] = {"us": ms * 1000 / cfg.layers, "gbs": by * cfg.layers / ms / 1e6, "frac": by * cfg.layers / ms / 1e6 / peak}
    ms = timed(lambda: normed(mw.embed, mw.norm, g["logits"], V), rounds=20)
    split["head (norm folded in)"] = {"us": ms * 1000, "gbs": (V * H * 2 + 2 * (H + V)) / ms / 1e6,
                                      "frac": (V * H * 2 + 2 * (H + V)) / ms / 1e6 / peak}  # fmt: skip
    gemv_ms = timed(whole)
    n_gemv = 4 * cfg.layers + 1
    # algorithmic bytes of one token's GEMVs: the weights as stored, plus each launch's x and y vectors
    abytes = eng.weight_bytes() + cfg.layers * 2 * (3 * H + cfg.qkv_rows + A + 2 * I + H) + 2 * (H + V)
    achieved = abytes / (gemv_ms / 1000.0) / 1e9
    return {"bound": "hbm", "kernel": "gemv_stream: the step's own GEMV launches (norm prologue, SwiGLU epilogue, plain), "
            "one token's 145 in step order", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_source": which, "frac_of_8tbs": achieved / 8000.0, "launches": n_gemv,
            "avg_launch_us": gemv_ms * 1000.0 / n_gemv, "per_kind": split,
            # DRAM bytes a launch: the ncu capture's read+write over algorithmic bytes, scaled to the average launch
            "traffic": TRAFFIC[storage] * abytes / n_gemv if TRAFFIC.get(storage) else None}


def tp_collective(eng, cfg, world, dist) -> dict:
    """what the tensor-parallel step exchanges, and one hop of it timed on its own: every rank sends its slice of a
    hidden-size vector to every rank and takes everyone's (CUDA events around 200 hops in a row, max over ranks)"""
    import torch

    from btb_b200 import capi
    from btb_b200.capi import call, ptr

    t = eng.tp_bufs(1)
    H, A, I = cfg.hidden, cfg.q_heads * cfg.head_dim, cfg.inter
    src = torch.zeros(1, H // world, dtype=torch.bfloat16, device="cuda")
    dst = torch.zeros(1, H, dtype=torch.bfloat16, device="cuda")
    s = capi.stream_ptr()
    hops = 200
    # the probe borrows the `yd` and `yo` vectors of width 1 in turn (a rank may send hop k + 1 while another still takes
    # hop k: two buffers keep them apart, as the step's own order of hops does) with a pass count of its own, started well
    # past the marks the decode left (every rank has made the same passes, so every rank starts at the same number)
    torch.cuda.synchronize()
    start = int(eng.passes[0, 0].item()) * 4 * cfg.layers + 4 * cfg.layers + 1000
    probe = torch.full((1,), start, dtype=torch.int32, device="cuda")
    sends = [eng.heap.send_desc(eng.off[1][k], H, eng.rank * (H // world), ptr(probe), 1, 1) for k in ("yd", "yo")]
    recv = capi.Recv(ptr(probe), 1, 1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    e0.record()
    for k in range(hops):
        call("btb_b200_xchg_send", ptr(src), 1, H // world, sends[k & 1], s)
        call("btb_b200_xchg_unpack", t[("yd", "yo")[k & 1]], ptr(dst), 1, H, recv, s)
        call("btb_b200_xchg_tick", ptr(probe), s)
    e1.record()
    torch.cuda.synchronize()
    us = torch.tensor([e0.elapsed_time(e1) * 1000.0 / hops], device="cuda")
    dist.all_reduce(us, op=dist.ReduceOp.MAX)
    assert capi.status() == 0, "the exchange probe timed out"
    per_step = cfg.layers * 4 * (A + 2 * H + I)  # bytes of marked words a step assembles in every rank's copies
    return {"kind": "peer stores of marked words into every rank's copy (NVLink writes; no collective call, no fence or "
                    "flag, no reduction), folded into the producing kernels' epilogues and the consuming kernels' prologues",
            "hops_per_step": 4 * cfg.layers + 1, "bytes_per_step_received_per_rank": per_step * (world - 1) // world,
            "us_per_hop_alone": float(us[0]), "note": "a hop alone = 3 launches (send, take, tick) on an idle stream; "
            "inside the step the send and the take are parts of the GEMV kernels"}


def run_ref_kernels(args) -> None:
    """the REFERENCE's own card kernels (oracle/_ref: its CUDA sources compiled for this card by oracle/build_ref.sh) and
    this library's, launched through the same typed launchers with the reference's own grids at the Qwen3-4B shape, each
    kind over 24 distinct matrices as one captured graph: the same-box baseline the new kernels have to beat. A checker's
    leg, not the product's: nothing here is on the decode path."""
    import torch

    from btb_b200 import launcher as L
    from tests import refkernels

    if not refkernels.available():
        print(json.dumps({"ref_gpu_kernels": None, "why": "oracle/_ref is not built (oracle/build_ref.sh)"}))
        return
    cfg_H, A, I, Hq, Hk, D = 2560, 4096, 9728, 32, 8, 128
    gen = torch.Generator(device="cuda").manual_seed(0)
    rnd = lambda *sh: (torch.randn(*sh, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)  # noqa: E731
    N = 24
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def timed(fn, rounds=5):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(rounds):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1000.0 / rounds / N  # us a launch

    out: dict = {}
    launchers = {"reference": refkernels.RefLauncher(), "b200": L.B200Launcher()}
    for name, (R, C_) in {"gemv_bf16_m1 19456x2560": (2 * I, cfg_H), "gemv_bf16_m1 2560x4096": (cfg_H, A),
                          "gemv_bf16_m1 2560x9728": (cfg_H, I)}.items():  # fmt: skip
        ws = [rnd(R, C_) for _ in range(N)]
        x, y = rnd(1, C_), torch.zeros(1, R, dtype=torch.bfloat16, device="cuda")
        for who, lz in launchers.items():
            us = timed(lambda lz=lz: [L.btb_gemv_bf16(lz, 1, ((R + 3) // 4, 1, 1), (128, 1, 1), w.data_ptr(), x.data_ptr(),
                                                      y.data_ptr(), R, C_) for w in ws])  # fmt: skip
            out.setdefault(name, {})[who] = {"us": us, "gbs": R * C_ * 2 / us / 1e3}
        del ws
    # the tensor-core matvec at 8 live rows (the reference's grid: a block of 4 warps a 64 rows, btb/engine/cuda.py:1473-1477)
    R, C_ = 2 * I, cfg_H
    ws = [rnd(R, C_) for _ in range(N)]
    x32, y32 = torch.zeros(32, C_, dtype=torch.bfloat16, device="cuda"), torch.zeros(32, R, dtype=torch.bfloat16, device="cuda")
    x32[:8] = rnd(8, C_)
    for who, lz in launchers.items():
        us = timed(lambda lz=lz: [L.btb_gemv_mma_bf16(lz, ((R + 63) // 64, 1, 1), (128, 1, 1), w.data_ptr(), x32.data_ptr(),
                                                      y32.data_ptr(), R, C_, 8) for w in ws])  # fmt: skip
        out.setdefault("gemv_mma_bf16 19456x2560 (8 rows)", {})[who] = {"us": us, "gbs": R * C_ * 2 / us / 1e3}
    del ws
    # decode attention, one row over 4096 cached rows (24 arenas: the keys come from DRAM)
    n0v, cap = 4096, 4608
    S = cap // 512
    Ks, Vs = [rnd(cap, Hk, D) * 50 for _ in range(N)], [rnd(cap, Hk, D) * 50 for _ in range(N)]
    q, att = rnd(1, Hq, D) * 50, torch.zeros(1, Hq * D, dtype=torch.bfloat16, device="cuda")
    pm, pl = torch.zeros(S * Hq, device="cuda"), torch.zeros(S * Hq, device="cuda")
    pa, cnt = torch.zeros(S * Hq * D, device="cuda"), torch.zeros(Hq, dtype=torch.int32, device="cuda")
    n0, par = torch.tensor([n0v], dtype=torch.int32, device="cuda"), torch.tensor([-1], dtype=torch.int32, device="cuda")
    G = Hq // Hk
    for who, lz in launchers.items():
        us = timed(lambda lz=lz: [L.btb_attn_flash(lz, D, ((G + 7) // 8, S, Hk), (256, 1, 1), q.data_ptr(), K_.data_ptr(),
                                                   V_.data_ptr(), att.data_ptr(), n0.data_ptr(), par.data_ptr(), 1, Hq, Hk, D,
                                                   Hk * D, float(D**-0.5), pm.data_ptr(), pl.data_ptr(), pa.data_ptr(),
                                                   cnt.data_ptr(), 0, 0) for K_, V_ in zip(Ks, Vs)])  # fmt: skip
        out.setdefault("attn_flash_d128, 1 row over 4096 cached rows", {})[who] = {"us": us, "gbs": 2 * n0v * Hk * D * 2 / us / 1e3}
    # residual + RMSNorm over one row
    h, yv, wn, xo = rnd(N, cfg_H), rnd(N, cfg_H), rnd(cfg_H), torch.zeros(1, cfg_H, dtype=torch.bfloat16, device="cuda")
    for who, lz in launchers.items():
        us = timed(lambda lz=lz: [L.btb_add_rmsnorm(lz, (1, 1, 1), (256, 1, 1), h[i].data_ptr(), yv[i].data_ptr(), wn.data_ptr(),
                                                    1e-6, xo.data_ptr(), cfg_H, 0) for i in range(N)])  # fmt: skip
        out.setdefault("add_rmsnorm 1x2560", {})[who] = {"us": us}
    tokens = ref_kernel_tokens(args, launchers["reference"])
    print(json.dumps({"ref_gpu_kernels": out, "sms": sms, "how": "CUDA events around a captured graph of 24 launches a kind "
                      "over 24 distinct inputs, 5 replays; the reference's kernels compiled for sm_100a with its own flags",
                      "tokens": tokens}))


def ref_kernel_tokens(args, ref, n_prompt: int = 48, n_new: int = 16) -> dict:
    """The configuration the metric is quoted on (Qwen3-4B shape, every layer, seeded weights) decoded on the same weights
    three ways, all fed the same tokens: (A) the REFERENCE's own card kernels launched one by one in the reference's order
    (btb/engine/cuda.py:1601-1837: add_rmsnorm, gemv, norm_rope_kv, attn_flash, gemv, add_rmsnorm, gemv, silu_mul, gemv;
    final norm, head, lowest-index argmax), a row a pass; (B) the same launches with ONLY the attention served by this
    library (the one kernel whose sums the reference makes on tensor-core tiles, held to 2^-6 a call); (C) this library's
    engine (its fused launches). B and C must agree bit for bit at every pick - every kernel but the attention is the
    reference's own, so the fusions and the GEMVs change no bit at full shape - and A against C shows what the attention's
    bound becomes after 36 layers of random weights."""
    import dataclasses

    import torch

    from btb_b200 import engine as E
    from btb_b200 import launcher as L

    cfg = E.QWEN3_4B if not args.layers else dataclasses.replace(E.QWEN3_4B, layers=args.layers)
    mw = E.synth_weights(cfg, seed=0, storage="bf16", layer_std=0.05)
    cap = 512
    eng = E.CardEngine(mw, cap=cap)
    prompt = torch.randint(0, cfg.vocab, (n_prompt,), generator=torch.Generator().manual_seed(0))
    H, Hq, Hk, D, I, V = cfg.hidden, cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.inter, cfg.vocab
    bf = lambda *sh: torch.zeros(*sh, dtype=torch.bfloat16, device="cuda")  # noqa: E731
    S, G = cap // 512, Hq // Hk
    p = lambda t: t.data_ptr() if t is not None else 0  # noqa: E731
    mine_lz = L.B200Launcher()

    class Path:
        """the reference's launch sequence over buffers of its own; `attn` serves the attention"""

        def __init__(self, attn):
            self.attn = attn
            self.K = [bf(cap, Hk, D) for _ in range(cfg.layers)]
            self.V = [bf(cap, Hk, D) for _ in range(cfg.layers)]
            self.h, self.x, self.y, self.qkv = bf(1, H), bf(1, H), bf(1, H), bf(1, cfg.qkv_rows)
            self.q, self.att, self.gu, self.m, self.logits = bf(1, Hq, D), bf(1, Hq * D), bf(1, 2 * I), bf(1, I), bf(1, V)
            self.pm, self.pl = torch.zeros(S * Hq, device="cuda"), torch.zeros(S * Hq, device="cuda")
            self.pa, self.cnt = torch.zeros(S * Hq * D, device="cuda"), torch.zeros(Hq, dtype=torch.int32, device="cuda")
            self.n0, self.dep = torch.zeros(1, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
            self.par = torch.tensor([-1], dtype=torch.int32, device="cuda")

        def gemv(self, w, xin, out, R, C_):
            L.btb_gemv_bf16(ref, 1, ((R + 3) // 4, 1, 1), (128, 1, 1), p(w), p(xin), p(out), R, C_)

        def step(self, tok: int) -> torch.Tensor:
            z = self
            z.h.copy_(mw.embed[tok : tok + 1])
            yp = None
            for i, Lw in enumerate(mw.layers):
                L.btb_add_rmsnorm(ref, (1, 1, 1), (256, 1, 1), p(z.h), p(yp), p(Lw.ln1), cfg.eps, p(z.x), H, 0)
                z.gemv(Lw.qkv, z.x, z.qkv, cfg.qkv_rows, H)
                L.btb_norm_rope_kv(ref, D, (Hq + 2 * Hk, 1, 1), (32, 1, 1), p(z.qkv), p(Lw.wq), p(Lw.wk), cfg.eps, p(eng.cos),
                                   p(eng.sin), p(z.n0), p(z.dep), p(z.K[i]), p(z.V[i]), p(z.q), 1, Hq, Hk, D, Hk * D, 0)
                L.btb_attn_flash(z.attn, D, ((G + 7) // 8, S, Hk), (256, 1, 1), p(z.q), p(z.K[i]), p(z.V[i]), p(z.att), p(z.n0),
                                 p(z.par), 1, Hq, Hk, D, Hk * D, float(D**-0.5), p(z.pm), p(z.pl), p(z.pa), p(z.cnt), 0, 0)
                z.gemv(Lw.o, z.att, z.y, H, Hq * D)
                L.btb_add_rmsnorm(ref, (1, 1, 1), (256, 1, 1), p(z.h), p(z.y), p(Lw.ln2), cfg.eps, p(z.x), H, 0)
                z.gemv(Lw.gu, z.x, z.gu, 2 * I, H)
                L.btb_silu_mul(ref, (min(4096, (I + 255) // 256), 1, 1), (256, 1, 1), p(z.gu), p(z.m), 1, I)
                z.gemv(Lw.down, z.m, z.y, H, I)
                yp = z.y
            L.btb_add_rmsnorm(ref, (1, 1, 1), (256, 1, 1), p(z.h), p(yp), p(mw.norm), cfg.eps, p(z.x), H, 0)
            z.gemv(mw.embed, z.x, z.logits, V, H)
            z.n0.add_(1)
            return z.logits[0].clone()

    A, B = Path(ref), Path(mine_lz)
    la = lb = None
    for t in prompt.tolist():
        la, lb = A.step(int(t)), B.step(int(t))
    eng.reset()
    lc = eng.prefill(prompt)[0].clone()
    bits_equal, worst, scale, decided, agree, toks = True, 0.0, 1.0, 0, 0, []
    for i in range(n_new):
        fa = la.float()
        top = torch.topk(fa, 2)
        tok = int((fa == top.values[0]).nonzero()[0])  # the lowest index among equals
        toks.append(tok)
        bits_equal = bits_equal and bool(torch.equal(lb.view(torch.int16), lc.view(torch.int16)))
        d = float((fa - lc.float()).abs().max())
        if d > worst:
            worst, scale = d, float(fa.abs().max())
        if float(top.values[0] - top.values[1]) > 2 * d:  # a pick the difference seen here cannot turn
            decided += 1
            agree += int(int((lc.float() == lc.float().max()).nonzero()[0]) == tok)
        if i + 1 < n_new:
            la, lb = A.step(tok), B.step(tok)
            lc = eng.forward(torch.tensor([tok]))[0].clone()
    torch.cuda.synchronize()
    return {"workload": f"{cfg.name}-shape bf16, {cfg.layers} layers, {n_prompt}-token prompt, {n_new} greedy picks, every "
                        "path fed the reference path's tokens",
            "distinct_tokens": len(set(toks)),
            "engine_bits_equal_reference_kernels_with_this_attention": bits_equal,
            "all_reference_kernels_vs_engine": {"max_logit_difference": worst, "max_logit_there": scale,
                                                "picks_decided_beyond_the_difference": decided, "of_those_equal": agree},
            "tokens_equal_reference_kernels": bits_equal and agree == decided}


def run_case(args) -> None:
    """one kernel on a small case, for a profiler capture or a quick look: `gemv:RxC[:M[:fmt]]` rotates over enough
    seeded matrices to stay out of L2 (fmt bf16 | p12 | fp8 | tc: the tensor-core matvec | tcp12: the same over pack12 weights); `attn:N` is the step's fused
    attention row over N cached rows at the Qwen3-4B head shape, `attnv:N:T` a verify pass's T rows over N cached rows. Prints us a launch (CUDA events) and, for a GEMV, the weight-streaming rate."""
    import torch

    from btb_b200 import capi
    from btb_b200 import engine as E
    from btb_b200.capi import call, ptr

    kind, _, rest = args.case.partition(":")
    sp = capi.stream_ptr()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out: dict = {"case": args.case}
    if kind == "gemv":
        parts = rest.split(":")
        R, C_ = (int(v) for v in parts[0].split("x"))
        M = int(parts[1]) if len(parts) > 1 else 1
        fmt = parts[2] if len(parts) > 2 else "bf16"
        per = R * C_ * {"p12": 1.5, "tcp12": 1.5, "fp8": 1.0}.get(fmt, 2)
        nmat = max(2, int(400e6 // per) + 1)
        gen = torch.Generator(device="cuda").manual_seed(0)
        ws = []
        for _ in range(nmat):
            w = torch.randn(R, C_, device="cuda", generator=gen).mul_(0.02).to(torch.bfloat16)
            if fmt in ("p12", "tcp12"):
                from btb_b200 import pack12

                w = E.P12Matrix(pack12.pack_bf16(w), R, C_, "cuda")
            elif fmt == "fp8":  # e4m3 bytes without NaN codes, bf16-valued scales a 128 x 128 block (config 4's draw)
                q = torch.randint(0, 256, (R, C_), device="cuda", generator=gen, dtype=torch.uint8)
                q = torch.where((q & 0x7F) == 0x7F, q & 0xF0, q)
                sc = (torch.randn(R // 128, C_ // 128, device="cuda", generator=gen) * 0.02).to(torch.bfloat16).float()
                w = E.FP8Matrix(q, sc)
            ws.append(w)
        x = torch.randn(M, C_, device="cuda", generator=gen).to(torch.bfloat16)
        y = torch.zeros(M, R, device="cuda", dtype=torch.bfloat16)

        ws_tc = None
        if fmt in ("tc", "tcp12"):
            ws_tc = torch.zeros(max(int(capi.lib().btb_b200_gemv_tc_workspace_bytes(R, C_)) // 4, 4), device="cuda")

        def one(w):
            if fmt == "tc":
                call("btb_b200_gemv_tc_bf16", ptr(w), ptr(x), ptr(y), M, R, C_, ptr(ws_tc), sp)
            elif fmt == "tcp12":
                call("btb_b200_gemv_tc_p12", ptr(w.lo), ptr(w.hi4), w.table, ptr(w.esc_idx), ptr(w.esc_val), ptr(w.esc_row),
                     ptr(x), ptr(y), M, R, C_, ptr(ws_tc), sp)  # fmt: skip
            elif fmt == "p12":
                call("btb_b200_gemv_p12", ptr(w.lo), ptr(w.hi4), w.table, ptr(w.esc_idx), ptr(w.esc_val), ptr(w.esc_row),
                     ptr(x), ptr(y), M, R, C_, sp)  # fmt: skip
            elif fmt == "fp8":
                call("btb_b200_gemv_fp8", ptr(w.w), ptr(w.scales), w.sr, w.sc, ptr(x), ptr(y), M, R, C_, sp)
            else:
                call("btb_b200_gemv_bf16", ptr(w), ptr(x), ptr(y), M, R, C_, sp)

        for it in range(3):
            e0.record()
            for w in ws:
                one(w)
            e1.record()
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000 / nmat
        out.update(us_per_launch=us, gbs=per / us / 1e3, matrices=nmat, bytes_per_launch=per + 2 * M * (R + C_))
    elif kind == "attn":
        n0v = int(rest)
        c = E.QWEN3_4B
        Hq, Hk, D, cap = c.q_heads, c.kv_heads, c.head_dim, ((n0v + 64 + 511) // 512) * 512
        gen = torch.Generator(device="cuda").manual_seed(0)
        rnd = lambda *sh: torch.randn(*sh, device="cuda", generator=gen).to(torch.bfloat16)  # noqa: E731
        qkv, K_, V_ = rnd(1, (Hq + 2 * Hk) * D), rnd(cap, Hk, D), rnd(cap, Hk, D)
        wq, wk, cos, sin = rnd(D), rnd(D), rnd(cap, D), rnd(cap, D)
        q, att = torch.zeros(1, Hq, D, device="cuda", dtype=torch.bfloat16), torch.zeros(1, Hq * D, device="cuda", dtype=torch.bfloat16)
        S = cap // 512
        pm, pl, pa = torch.zeros(S * Hq, device="cuda"), torch.zeros(S * Hq, device="cuda"), torch.zeros(S * Hq * D, device="cuda")
        cnt = torch.zeros(Hq, dtype=torch.int32, device="cuda")
        n0 = torch.tensor([n0v], dtype=torch.int32, device="cuda")
        depth = torch.zeros(1, dtype=torch.int32, device="cuda")
        for it in range(3):
            e0.record()
            for _ in range(20):
                call("btb_b200_attn_step", ptr(qkv), ptr(wq), ptr(wk), 1e-6, ptr(cos), ptr(sin), ptr(n0), ptr(depth),
                     ptr(K_), ptr(V_), ptr(q), ptr(att), Hq, Hk, D, D, Hk * D, 0, float(D**-0.5), ptr(pm), ptr(pl), ptr(pa),
                     ptr(cnt), 0, 0, 0, cap, sp)  # fmt: skip
            e1.record()
            torch.cuda.synchronize()
        out.update(us_per_launch=e0.elapsed_time(e1) * 1000 / 20, cached_rows=n0v)
    elif kind == "attnv":
        # a verify pass's attention: `attnv:N:T` = T tree rows (a chain) over N cached rows, Qwen3-4B head shape,
        # through btb_b200_norm_rope_kv + btb_b200_attn_decode; the cache's rows rotate over layers' worth of arenas so
        # that the keys come from DRAM
        n0v, T = (int(v) for v in rest.split(":"))
        c = E.QWEN3_4B
        Hq, Hk, D, cap = c.q_heads, c.kv_heads, c.head_dim, ((n0v + 64 + 511) // 512) * 512
        gen = torch.Generator(device="cuda").manual_seed(0)
        rnd = lambda *sh: torch.randn(*sh, device="cuda", generator=gen).to(torch.bfloat16)  # noqa: E731
        arenas = max(2, int(300e6 // (2 * cap * Hk * D * 2)) + 1)
        Ks, Vs = [rnd(cap, Hk, D) for _ in range(arenas)], [rnd(cap, Hk, D) for _ in range(arenas)]
        M = E.pad_rows(T)
        q, att = rnd(M, Hq, D), torch.zeros(M, Hq * D, device="cuda", dtype=torch.bfloat16)
        S = cap // 512
        pm, pl = torch.zeros(S * M * Hq, device="cuda"), torch.zeros(S * M * Hq, device="cuda")
        pa, cnt = torch.zeros(S * M * Hq * D, device="cuda"), torch.zeros(M * Hq, dtype=torch.int32, device="cuda")
        n0 = torch.tensor([n0v], dtype=torch.int32, device="cuda")
        par = torch.arange(-1, M - 1, dtype=torch.int32, device="cuda")
        for it in range(3):
            e0.record()
            for K_, V_ in zip(Ks, Vs):
                call("btb_b200_attn_decode", ptr(q), ptr(K_), ptr(V_), ptr(att), ptr(n0), ptr(par), T, Hq, Hk, D, D, Hk * D,
                     float(D**-0.5), ptr(pm), ptr(pl), ptr(pa), ptr(cnt), 0, 0, 0, cap, sp)  # fmt: skip
            e1.record()
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000 / arenas
        kv = 2 * (n0v + T) * Hk * D * 2
        out.update(us_per_launch=us, cached_rows=n0v, rows=T, kv_bytes=kv, gbs=kv / us / 1e3, arenas=arenas)
    elif kind == "moe":
        # the picked experts' gate/up matvecs of one MoE layer: moe:fp8 (Qwen3-30B-A3B shape, 8 picks of 128 experts)
        # or moe:mx4 (gpt-oss-20b shape, 4 picks of 32); the picks rotate so that the rows come from DRAM
        from btb_b200 import moe as MO

        cfg = MO.QWEN3_30B_A3B if rest.split(":")[0] == "fp8" else MO.GPT_OSS_20B
        gen = torch.Generator(device="cuda").manual_seed(0)
        down = ":dn" in args.case  # moe:fp8:dn / moe:mx4:dn: the layer's DOWN stack (an activated row a pick)
        st = (MO.synth_expert_stack(cfg, gen, cfg.experts, cfg.hidden, cfg.inter, "cuda") if down
              else MO.synth_expert_stack(cfg, gen, cfg.experts, 2 * cfg.inter, cfg.hidden, "cuda"))
        k, E = cfg.top_k, cfg.experts
        rounds = max(2, E // k)
        picks = [torch.arange(i * k, (i + 1) * k, dtype=torch.int32, device="cuda") % E for i in range(rounds)]
        # the row the engine's experts are given: the normed bf16 row widened to f32 (moe:fp8:f32 for any f32 row)
        xf = torch.randn(k if down else 1, st.C, device="cuda", generator=gen)
        if not args.case.endswith(":f32"):
            xf = xf.bfloat16().float()
        yv = torch.zeros(k, st.R, device="cuda")
        per = k * st.R * st.C * {"fp8": 1.0, "mx4": 17 / 32, "bf16": 2.0}[st.fmt]
        for it in range(3):
            e0.record()
            for idx in picks:
                call("btb_b200_moe_gemv", MO.FMT[st.fmt], ptr(st.w), ptr(st.scales), st.w_stride, st.s_stride, st.sr, st.sc,
                     ptr(idx), k, E, ptr(xf), 1 if down else k, ptr(yv), st.R, st.C, 0, 1, sp)  # fmt: skip
            e1.record()
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000 / rounds
        out.update(us_per_launch=us, gbs=per / us / 1e3, bytes_per_launch=per, picks=k, experts=E)
    elif kind == "sample":
        V = int(rest)
        from btb_b200.sampling import CardSampler, Sampling

        smp = CardSampler("cuda")
        smp.set(Sampling(temperature=0.8, top_k=40, top_p=0.9, seed=7))
        lg = torch.randn(1, V, device="cuda").to(torch.bfloat16)
        n0, tok = torch.zeros(1, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int64, device="cuda")
        for it in range(3):
            e0.record()
            for _ in range(20):
                smp.pick(lg, 1, n0, None, tok, sp)
            e1.record()
            torch.cuda.synchronize()
        out.update(us_per_launch=e0.elapsed_time(e1) * 1000 / 20, vocab=V)
    elif kind == "verify":
        # the verify pass's pick over R tree nodes with 4 drafted children each (verify:V[:R]): the drafter a perturbed copy
        # of the target, every other node a point-mass row
        from btb_b200.sampling import Sampling, Verify

        parts = rest.split(":")
        V, R = int(parts[0]), int(parts[1]) if len(parts) > 1 else 8
        gen = torch.Generator(device="cuda").manual_seed(0)
        lg = (torch.randn(R, V, device="cuda", generator=gen) * 3).to(torch.bfloat16)
        q = torch.softmax(lg.float() + torch.randn(R, V, device="cuda", generator=gen), -1)
        kids = torch.multinomial(q, 4).tolist()
        s_ = Sampling(temperature=0.8, top_k=40, top_p=0.9, seed=7)
        v = Verify(s_, q, kids, [r % 2 == 0 for r in range(R)])
        keys = [s_.key_for(100 + r) for r in range(R)]
        v.pick(lg, keys)
        for it in range(3):
            e0.record()
            for _ in range(10):
                outv = v.pick(lg, keys)
            e1.record()
            torch.cuda.synchronize()
        acc = int(((outv >> 24) > 0).sum())
        out.update(us_per_call=e0.elapsed_time(e1) * 1000 / 10, vocab=V, nodes=R, children=4, accepted_nodes=acc,
                   note="a call is the host class's: small uploads of kids / keys / parameters and one launch")
    else:
        raise SystemExit(f"unknown case {args.case}")
    assert capi.status() == 0
    print(json.dumps(out), flush=True)


def run_batch(args, mw, cfg, storage, cap, rank, world, dist) -> None:
    """small-batch decode: --batch sequences with independent seeded prompts decoded side by side, a pass of B rows a
    step (every weight streamed once for all of them)"""
    import torch

    from btb_b200 import capi
    from btb_b200 import engine as E
    from btb_b200.batch import BatchEngine

    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    eng = BatchEngine(mw, B, cap=cap)
    eng.wide_tc = bool(args.wide_tc)
    prompts = [torch.randint(0, cfg.vocab, (PROMPT,), generator=torch.Generator().manual_seed(100 + b)) for b in range(B)]
    eng.prefill_all(prompts)
    # outside the timed region: the first step's logits of the pass as timed against the same step through the fp32-chain
    # GEMVs (the two families sum in different orders: they agree to rounding, and a wrong partial sum does not)
    check = None
    if eng.wide_tc:
        gB = eng.bufs(E.pad_rows(B))
        keep_n, keep_ids = eng.n0b.clone(), gB["ids"].clone()

        def first_step(tc: bool):
            eng.wide_tc = tc
            eng._batch_step(capi.stream_ptr())
            torch.cuda.synchronize()
            out = gB["logits"][:B].float().clone(), eng.pin_toks.clone()
            eng.n0b.copy_(keep_n)
            gB["ids"].copy_(keep_ids)
            return out

        (lc, tc_), (lt, tt) = first_step(False), first_step(True)
        diff, top = float((lt - lc).abs().max()), float(lc.abs().max())
        check = {"first_step_logits_max_abs_diff_vs_fp32_chain": diff, "max_abs_logit": top,
                 "picks_equal": int((tc_ == tt).sum()), "of": B}
        assert diff <= 0.1 * max(1.0, top), f"the tensor-core pass is off the fp32-chain pass: {check}"
    graph = eng.batch_graph()
    for _ in range(W):
        graph.replay()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with Clocks(int(os.environ.get("LOCAL_RANK", "0"))) as clk:
        e0.record()
        for _ in range(K):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    t0 = time.perf_counter()
    for _ in range(K):  # the public loop: every step's B tokens read back before the next
        graph.replay()
        torch.cuda.current_stream().synchronize()
        _ = eng.pin_toks.tolist()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([ms, e2e_s * 1000.0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0]), float(t[1]) / 1000.0
    assert capi.status() == 0, "a kernel recorded a device-side refusal"
    peak, _ = measured_hbm_peak()
    tps = world * B * K / (ms / 1000.0)
    line = {
        "metric": f"decode tok/s @bs{B} ({cfg.name} shape" + (", pack12 weights)" if storage == "p12" else ")"),
        "value": tps, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if storage == "bf16" else f"bf16 ({STORED.get(storage, storage)} weights widened in registers)",
        "data": "synthetic",
        "config": {"workload": f"{cfg.name}-shape {storage}, batch {B} (independent seeded prompts of {PROMPT} tokens), "
                   "greedy decode", "parallelism": "replicas only" if world > 1 else "1 gpu", "batch": B,
                   "matvec": "tensor cores (tcgen05)" if eng.wide_tc else "fp32 chains",
                   "l2": "weights per step > L2 126 MB", "bytes_per_step": cfg.weight_bytes_per_token(storage)},
        "clocks": clk.summary(),
        "e2e": {"value": world * B * K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 8 * B},
        "gpu_launches": eng.launches_per_step * K, "roofline": None,
        "step_roofline_frac": (cfg.weight_bytes_per_token(storage) * K / (ms / 1000.0) / 1e9) / peak,
        "check": check,
    }  # fmt: skip
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


def run_speculative(args, eng, cfg, storage, parallelism, rank, world, dist) -> None:
    """greedy decode with an n-gram tree of `--speculative` drafts verified a pass: the prompt is a seeded 64-token
    pattern repeated to 512 tokens so that the n-grams have something to propose"""
    import torch

    from btb_b200 import capi
    from btb_b200.draft import generate_speculative

    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (64,), generator=g).repeat(8)
    K, W = args.steps, max(args.warmup, 3)
    generate_speculative(eng, prompt, W, budget=args.speculative)
    ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    with Clocks(int(os.environ.get("LOCAL_RANK", "0"))) as clk:
        t0 = time.perf_counter()
        toks, stats = generate_speculative(eng, prompt, K + 1, budget=args.speculative, events=ev)
        wall = time.perf_counter() - t0
    ms = ev[0].elapsed_time(ev[1])
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    assert capi.status() == 0, "a kernel recorded a device-side refusal"
    tps = K / (ms / 1000.0)
    line = {
        "metric": f"decode tok/s @bs1 ({cfg.name} shape, n-gram tree of {args.speculative} drafts a pass)", "value": tps,
        "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16" if storage == "bf16" else f"bf16 ({STORED.get(storage, storage)} weights widened in registers)",
        "data": "synthetic",
        "config": {"workload": f"{cfg.name}-shape {storage}, batch 1, speculative greedy decode after a 512-token prompt "
                   "(a seeded 64-token pattern repeated)", "parallelism": parallelism, "passes": stats["passes"],
                   "tokens_per_pass": stats["tokens_per_pass"], "l2": "weights per pass > L2 126 MB"},
        "clocks": clk.summary(),
        # the loop is the public call: every pass reads its picks back and sends the next tree's ids
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 8 * (1 + args.speculative) * stats["passes"] / K,
                "d2h_bytes_per_step": 8 * (1 + args.speculative) * stats["passes"] / K, "wall_s": wall},
        "gpu_launches": None, "roofline": None,
    }  # fmt: skip
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


# per-launch DRAM traffic of the dominant kernel from the committed ncu summary (profiles/), filled once captured
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of the captured launch: 103.03 MB over 99.66 MB for
# the 19456 x 2560 bf16 GEMV (profiles/gemv_stream_bf16_m1.md); traffic grows in proportion to the rows streamed
TRAFFIC: dict[str, float | None] = {"bf16": 1.034, "p12": None}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="qwen3-4b-bf16",
                    choices=["qwen3-4b-bf16", "qwen3-4b-p12", "gpt-oss-20b", "qwen3-30b-a3b", "llama-70b"])
    ap.add_argument("--step-kernel", type=int, default=0, help="1: the whole step as one persistent kernel")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0: the config's)")
    ap.add_argument("--context", type=int, default=0, help="llama-70b: rows of synthetic cache standing before the step")
    ap.add_argument("--graph-steps", type=int, default=1)
    ap.add_argument("--pdl", type=int, default=None)
    ap.add_argument("--l2-warm-kb", type=int, default=None, help="weights the attention launch pulls into L2 ahead (KB)")
    ap.add_argument("--l2-warm-ctas", type=int, default=None)
    ap.add_argument("--cpu-steps", type=int, default=4)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--batch", type=int, default=1, help="qwen3-4b workloads: sequences decoded side by side")
    ap.add_argument("--wide-tc", type=int, default=1, help="--batch: the tensor-core matvec for the pass of B rows")
    ap.add_argument("--case", default="", help="one kernel on a small case: gemv:RxC[:M[:fmt]], attn:N, moe:fp8|mx4, sample:V")
    ap.add_argument("--speculative", type=int, default=0, help="verify an n-gram tree of this many drafts a pass")
    ap.add_argument("--ref-kernels", action="store_true", help="time the reference's own card kernels beside this library's")
    ap.add_argument("--prompt", type=int, default=0, help="prompt tokens (0: the configuration's own length)")
    ap.add_argument("--prefill", default="auto", choices=["auto", "gemm", "chain"])
    ap.add_argument("--replicas", action="store_true", help="--gpus N: N independent copies instead of one model over N ranks")
    ap.add_argument("--tune", default="", help="the library's launch tunables, k=v[,k=v...] (btb_b200_set_tuning)")
    args = ap.parse_args()
    if args.tune and args.impl != "reference":
        from btb_b200 import capi  # noqa: PLC0415

        capi.set_tuning(**{k: int(v) for k, v in (kv.split("=") for kv in args.tune.split(","))})
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.ref_kernels:
        run_ref_kernels(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args, rank)
    else:
        run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
