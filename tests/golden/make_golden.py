"""Generates the golden fixtures of this folder from the reference checkout.

Run once where the reference is mounted (``python tests/golden/make_golden.py <reference checkout>``); the outputs are
committed and the tests read only them. Everything here is produced by IMPORTING the reference's own Python codecs
(``btb.pack12``, ``btb.mxfp4``, ``btb.fp8``, ``btb.sampling``, ``btb.draft``) or by reading its banked test
fixtures (``tests/fixtures/tiny_qwen3*``, ``tests/fixtures/receipts_qwen3.pt``), never by re-deriving a value.

Outputs
  codecs.npz       pack12 cases (packed parts + the reference's unpack), MXFP4 exhaustive byte x scale dequantize,
                   FP8 byte x scale `held` values
  tiny_qwen3.npz   the tiny Qwen3 fixture's weights (bf16 bits), its pack12 and FP8 stores' parts, and the receipts
                   banked by the reference's CPU path (prompt/tree/next logits, per-layer K/V, greedy tokens)
  sampling.npz     key_for() values for seeded (seed, position) pairs
  drafts.json      n-gram chains and merged trees from the reference's proposer over seeded token streams
  moe.npz          the MoE block's host pieces run from the reference's own source: both routers' picks and weights, both
                   gated activations in the row dtype, the down product's rounding, bias and ordered sum
  tiny_gpt_oss.npz the tiny gpt-oss fixture's tensors as stored (MXFP4 experts) and its banked receipts
"""

from __future__ import annotations

import json
import os
import struct
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def codecs(ref: str, out: dict) -> None:
    from btb import fp8, mxfp4, pack12

    g = torch.Generator().manual_seed(1234)
    cases = {
        "a": torch.randn(48, 64, generator=g) * 0.02,  # the configs' weight distribution
        "b": torch.randn(7, 24, generator=g) * torch.logspace(-12, 6, 24),  # many high bytes: dense escapes
        "c": torch.randn(5, 9, generator=g),  # odd element count
        "d": torch.zeros(4, 8),  # one high byte only
        "e": torch.randn(96, 160, generator=g) * torch.logspace(-10, 4, 160),  # escapes across many 2048-element tiles
    }
    for name, t in cases.items():
        t = t.to(torch.bfloat16)
        lo, hi4, tbl, ei, ev = pack12.pack_bf16(t)
        back = pack12.unpack_bf16(
            torch.from_numpy(lo), torch.from_numpy(hi4), torch.from_numpy(tbl), t.numel(), tuple(t.shape),
            torch.from_numpy(ei), torch.from_numpy(ev),
        )  # fmt: skip
        assert torch.equal(back.view(torch.int16), t.view(torch.int16))
        out[f"p12_{name}_src"] = bits(t)
        out[f"p12_{name}_lo"], out[f"p12_{name}_hi4"], out[f"p12_{name}_tbl"] = lo, hi4, tbl
        out[f"p12_{name}_esc_idx"], out[f"p12_{name}_esc_val"] = ei, ev
        out[f"p12_{name}_unpacked"] = bits(back)
    # MXFP4: every byte under every scale (the reference's own exhaustive test shape)
    blocks = np.repeat(np.arange(256, dtype=np.uint8)[None, :, None], 256, axis=0)  # [scale, byte, 1]
    blocks = np.broadcast_to(blocks, (256, 256, 16)).copy().reshape(256, 256, 1, 16)
    scales = np.repeat(np.arange(256, dtype=np.uint8)[:, None, None], 256, axis=1)  # [scale, byte, 1]
    deq = mxfp4.dequantize(blocks, scales)  # [256, 256, 32]
    db = deq.view(np.uint32)
    assert (db[:, :, 0::2] == db[:, :, :1]).all() and (db[:, :, 1::2] == db[:, :, 1:2]).all()  # one byte repeated
    out["mx4_pair"] = np.ascontiguousarray(deq[:, :, :2]).view(np.uint32)  # [scale, byte, (lo nibble, hi nibble)]
    # a seeded matrix, for the layout (rows, blocks along K, low nibble first)
    rng = np.random.default_rng(7)
    mb = rng.integers(0, 256, size=(6, 4, 16), dtype=np.uint8)
    ms = rng.integers(110, 135, size=(6, 4), dtype=np.uint8)
    out["mx4_m_blocks"], out["mx4_m_scales"] = mb, ms
    out["mx4_m_deq"] = mxfp4.dequantize(mb, ms).view(np.uint32)
    # FP8: every byte under seeded scales (bf16-valued, as the configs draw them, and arbitrary f32 ones)
    sc = torch.cat([
        (torch.randn(24, generator=g) * 0.02).to(torch.bfloat16).float(),
        torch.randn(24, generator=g) * torch.logspace(-6, 3, 24),
        torch.tensor([1.0, 2.0 ** -20, 448.0, 1e-30, 3.0e38, -0.75, 0.0, 2.0 ** -140]),
    ])  # fmt: skip
    q = torch.arange(256, dtype=torch.uint8).reshape(1, 256).repeat(sc.numel(), 1)  # row i under scale i
    held = fp8.held(q, sc.reshape(-1, 1))
    out["fp8_scales"] = sc.numpy()
    out["fp8_held"] = bits(held)  # [n_scales, 256]
    # a blocked matrix: 8x12 in 2x3 grid
    qm = torch.from_numpy(rng.integers(0, 256, size=(8, 12), dtype=np.uint8))
    qm[(qm & 0x7F) == 0x7F] = 0x3C
    sm = (torch.randn(2, 3, generator=g) * 0.02).to(torch.bfloat16).float()
    out["fp8_m_w"], out["fp8_m_scales"] = qm.numpy(), sm.numpy()
    out["fp8_m_held"] = bits(fp8.held(qm, sm))


def tiny(ref: str, out: dict) -> None:
    from safetensors import safe_open

    fx = os.path.join(ref, "tests", "fixtures")

    def read_all(d: str) -> dict:
        idx = json.load(open(os.path.join(fx, d, "model.safetensors.index.json")))
        res = {}
        for shard in sorted(set(idx["weight_map"].values())):
            with safe_open(os.path.join(fx, d, shard), "pt") as f:
                for k in f.keys():
                    res[k] = f.get_tensor(k)
        return res

    out["config"] = np.frombuffer(open(os.path.join(fx, "tiny_qwen3", "config.json"), "rb").read(), np.uint8)
    for k, v in read_all("tiny_qwen3").items():
        assert v.dtype == torch.bfloat16, (k, v.dtype)
        out["w/" + k] = bits(v)
    for k, v in read_all("tiny_qwen3-pack12").items():
        out["p12/" + k] = v.numpy() if v.dtype == torch.uint8 else bits(v)
    for k, v in read_all("tiny_qwen3-f8_e4m3").items():
        if v.dtype == torch.float8_e4m3fn:
            out["f8/" + k] = v.view(torch.uint8).numpy()
        elif v.dtype == torch.bfloat16:
            out["f8/" + k] = bits(v)
        else:
            out["f8/" + k] = v.numpy()
    rc = torch.load(os.path.join(fx, "receipts_qwen3.pt"), weights_only=False)
    for store in ("bf16", "p12"):
        r = rc[store]
        out[f"rc/{store}/prompt_logits"] = r["prompt_logits"].numpy()
        out[f"rc/{store}/chunk_logits"] = r["chunk_logits"].numpy()
        out[f"rc/{store}/next"] = r["next"].numpy()
        out[f"rc/{store}/greedy"] = np.asarray(r["greedy"], np.int64)
        for i, (k, v) in r["keys"].items():
            out[f"rc/{store}/k{i}"] = k.float().numpy()
            out[f"rc/{store}/v{i}"] = v.float().numpy()
    sys.path.insert(0, os.path.join(ref, "tests"))
    import helpers

    out["rc/prompt"] = np.asarray(helpers.PROMPT_DENSE[0], np.int64)
    out["rc/chunk"] = np.asarray(helpers.CHUNK, np.int64)
    out["rc/parents"] = np.asarray(helpers.PARENTS, np.int64)
    out["rc/depth"] = np.asarray(helpers.DEPTH, np.int64)
    out["rc/path"] = np.asarray(helpers.PATH, np.int64)


def sampling(ref: str, out: dict) -> None:
    from btb import sampling as S

    seeds = [0, 1, 7, 2**31 - 1, 123456789]
    pos = [0, 1, 2, 17, 4095, 100000]
    out["key_seeds"], out["key_pos"] = np.asarray(seeds, np.int64), np.asarray(pos, np.int64)
    out["keys"] = np.asarray([[S.Sampling(temperature=1.0, seed=s).key_for(p) for p in pos] for s in seeds], np.uint64)
    out["keys_salt3"] = np.asarray([[S.Sampling(temperature=1.0, seed=s).key_for(p, 3) for p in pos] for s in seeds],
                                   np.uint64)
    idx = torch.arange(0, 4096, dtype=torch.int64)
    key = int(out["keys"][2][3])
    out["uniform_key"] = np.asarray([key], np.uint64)
    out["uniform"] = S._hash_uniform(key, idx).numpy()


def verify(ref: str, out: dict) -> None:
    """seeded verify-pass picks through the reference's `Verify.pick_torch` on the CPU (its torch statement of the card's
    btb_sample_verify): children drawn from a perturbed copy of the target by the reference's own `draw_torch`, rows with
    and without a drafter distribution, with and without top-k / top-p"""
    from btb.sampling import Sampling, Verify

    cases = [(12, 4, 300, Sampling(temperature=0.8, top_p=0.9, seed=5), 8, 0.7),
             (12, 4, 100, Sampling(temperature=1.2, top_k=6, seed=2), 4, 0.7),
             (3000, 3, 24, Sampling(temperature=0.7, top_k=50, top_p=0.95, seed=11), 6, 0.7),
             (3000, 3, 24, Sampling(temperature=1.0, seed=3), 3, 0.7),
             (12, 4, 300, Sampling(temperature=0.8, seed=8), 3, 3.0),  # a drafter far from the target: rejections
             (3000, 3, 24, Sampling(temperature=0.9, top_p=0.8, seed=4), 5, 2.0)]  # fmt: skip
    for ci, (V, R, n, s, width, noise) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + ci)
        logits = torch.randn(R, V, generator=g) * 3
        dl = logits + torch.randn(R, V, generator=g) * noise
        K, H, KEYS, OUT = [], [], [], []
        for i in range(n):
            keys = [s.key_for(i * R + r) for r in range(R)]
            ids, q = s.draw_torch(dl, [s.key_for(i * R + r, salt=1) for r in range(R)], width)
            hasq = [(i + r) % 3 != 0 for r in range(R)]
            kids = ids.tolist()
            got = Verify(s, q, kids, hasq).pick_torch(logits, keys)
            K.append(np.asarray(kids, np.int32)), H.append(np.asarray(hasq, np.uint32))
            KEYS.append(np.asarray(keys, np.uint64)), OUT.append(got.numpy().astype(np.uint32))
        out[f"v{ci}/logits"], out[f"v{ci}/dl"] = logits.numpy(), dl.numpy()
        out[f"v{ci}/params"] = np.asarray([s.temperature, s.top_k, s.top_p, s.seed, width], np.float64)
        out[f"v{ci}/kids"], out[f"v{ci}/hasq"] = np.stack(K), np.stack(H)
        out[f"v{ci}/keys"], out[f"v{ci}/out"] = np.stack(KEYS), np.stack(OUT)
        # the drafter's distribution does not depend on the keys: the same at every trial of a case, kept once
        out[f"v{ci}/q"] = s.dist_torch(dl).numpy()


def drafts(ref: str) -> dict:
    """seeded token streams through the reference's n-gram proposer and its chain merge: the chains proposed after
    every few tokens and the trees built from them"""
    import random

    import ast

    from btb.draft import NGramProposer

    # btb.engine.generate imports a transformers class this image's version lacks; its tree builder is a plain
    # function, so it is taken from the module's source and run on its own
    src = open(os.path.join(ref, "btb", "engine", "generate.py")).read()
    fn = next(n for n in ast.parse(src).body if isinstance(n, ast.FunctionDef) and n.name == "_chains_tree")
    ns: dict = {}
    exec("from __future__ import annotations\n" + ast.get_source_segment(src, fn), ns)  # noqa: S102
    _chains_tree = ns["_chains_tree"]

    cases = []
    for seed, vocab, n, kw in ((0, 6, 160, {}), (1, 3, 120, {"n_max": 3, "n_min": 1, "followers": 2}),
                               (2, 40, 200, {"n_max": 5, "n_min": 2, "followers": 4})):  # fmt: skip
        rng = random.Random(seed)
        pattern = [rng.randrange(vocab) for _ in range(17)]
        toks = [pattern[i % 17] if rng.random() < 0.8 else rng.randrange(vocab) for i in range(n)]
        prop = NGramProposer(toks[:8], **kw)
        steps = []
        for i, t in enumerate(toks[8:]):
            prop.extend(t)
            if i % 5 == 0:
                for v, budget in ((4, 8), (8, 5), (3, 31)):
                    chains = prop.propose_chains(v)
                    g, par, dep, ch, _tags = _chains_tree(chains, budget)
                    steps.append({"at": i, "v": v, "budget": budget, "chains": [[list(c), tag] for c, tag in chains],
                                  "guesses": list(g), "parents": list(par), "depth": list(dep),
                                  "children": {str(k): list(x) for k, x in ch.items()}})  # fmt: skip
        cases.append({"kw": kw, "head": toks[:8], "tail": toks[8:], "steps": steps})
    return {"cases": cases}


def _method(ref: str, rel: str, cls: str, name: str):
    """a method of a class in a reference module that this image cannot import whole (it needs a newer transformers),
    taken from the module's source and run on its own as a plain function of (self, ...)"""
    import ast
    from typing import Any

    src = open(os.path.join(ref, rel)).read()
    c = next(n for n in ast.parse(src).body if isinstance(n, ast.ClassDef) and n.name == cls)
    fn = next(n for n in c.body if isinstance(n, ast.FunctionDef) and n.name == name)
    fn.decorator_list = []
    ns: dict = {"torch": torch, "Any": Any}
    exec("from __future__ import annotations\n" + ast.unparse(fn), ns)  # noqa: S102
    return ns[name]


def moe(ref: str, out: dict) -> None:
    """the host's MoE pieces (btb/engine/host.py `_Router`, `_Experts`; families/qwen4/router.py `Qwen4Router`) executed
    from the reference's source on seeded rows"""
    from types import SimpleNamespace as NS

    g = torch.Generator().manual_seed(4321)
    # routers: f32 logits in (what the host GEMV hands them), bf16 rows
    for tag, E, k in (("a", 32, 4), ("b", 128, 8), ("c", 8, 2)):
        lg = torch.randn(6, E, generator=g) * 2.0
        hidden = torch.zeros(6, 4, dtype=torch.bfloat16)
        lin = lambda x, lg=lg: lg  # noqa: E731  the router's matvec is pinned elsewhere; the picks are what is banked here
        r1 = _method(ref, "btb/engine/host.py", "_Router", "forward")
        _lg, scores, idx = r1(NS(lin=lin, top_k=k), hidden)
        out[f"route_{tag}_logits"] = lg.numpy()
        out[f"route_{tag}_m1_idx"], out[f"route_{tag}_m1_w"] = idx.numpy().astype(np.int32), bits(scores)
        r0 = _method(ref, "btb/engine/families/qwen4/router.py", "Qwen4Router", "forward")
        _l, wts, ex = r0(NS(lin=lin, top_k=k, hidden_dim=4, norm_topk_prob=True), hidden)
        out[f"route_{tag}_m0_idx"], out[f"route_{tag}_m0_w"] = ex.numpy().astype(np.int32), bits(wts)
    # the gated activations in the row dtype, with and without the bias
    gate1 = _method(ref, "btb/engine/host.py", "_Experts", "gpt_oss_gate")
    silu_gate = _method(ref, "btb/engine/host.py", "_Experts", "_silu_gate")
    act = _method(ref, "btb/engine/host.py", "_Experts", "_act")
    bias_of = _method(ref, "btb/engine/host.py", "_Experts", "_bias")
    down = _method(ref, "btb/engine/host.py", "_Experts", "_down")
    n, I, H, E = 8, 48, 40, 6
    gu = torch.randn(n, 2 * I, generator=g) * 3.0  # past the clamp at 7 on both sides
    rows = torch.randint(0, E, (n,), generator=g)
    b_gu = (torch.randn(E, 2 * I, generator=g) * 0.5).to(torch.bfloat16)
    b_dn = (torch.randn(E, H, generator=g) * 0.5).to(torch.bfloat16)
    out["act_gu"], out["act_rows"] = gu.numpy(), rows.numpy().astype(np.int32)
    out["act_bias_gu"], out["act_bias_dn"] = bits(b_gu), bits(b_dn)
    for kind, gate in ((0, None), (1, gate1)):
        for biased in (False, True):
            me = NS(biased=biased, gate=gate, alpha=1.702, limit=7.0, gate_up_proj_bias=b_gu, _bias=bias_of,
                    act_fn=torch.nn.functional.silu)  # fmt: skip
            me._silu_gate = lambda x, me=me: silu_gate(me, x)
            got = act(me, gu.to(torch.bfloat16), rows)
            assert got.dtype == torch.bfloat16
            out[f"act_k{kind}_b{int(biased)}"] = bits(got)
    # the down product's rounding and bias, the routing weight, and the sum one expert at a time in ascending id
    # (host.py `_one_row`: out[i] = _down(dn_buf[i], hit[i], dt) * weights[slot]; final[0] += out[i], hit ascending)
    T, k = 5, 4
    dn = torch.randn(T, k, H, generator=g) * 2.0
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])  # the router's order, not sorted
    w = torch.softmax(torch.randn(T, k, generator=g), -1).to(torch.bfloat16)
    out["comb_dn"], out["comb_idx"], out["comb_w"] = dn.numpy(), idx.numpy().astype(np.int32), bits(w)
    for biased in (False, True):
        me = NS(biased=biased, down_proj_bias=b_dn, _bias=bias_of)
        fin = torch.zeros(T, H, dtype=torch.bfloat16)
        for t in range(T):
            hit = sorted(int(e) for e in idx[t])
            slot = {e: idx[t].tolist().index(e) for e in hit}
            for e in hit:
                fin[t] += down(me, dn[t, slot[e]], e, torch.bfloat16) * w[t][slot[e]]
        out[f"comb_b{int(biased)}"] = bits(fin)


def tiny_moe(ref: str, out: dict) -> None:
    """the reference's tiny gpt-oss fixture as stored, and its banked receipts (transformers' f32 forward)"""
    from safetensors import safe_open

    fx = os.path.join(ref, "tests", "fixtures")
    d = os.path.join(fx, "tiny_gpt_oss")
    idx = json.load(open(os.path.join(d, "model.safetensors.index.json")))
    out["config"] = np.frombuffer(open(os.path.join(d, "config.json"), "rb").read(), np.uint8)
    for shard in sorted(set(idx["weight_map"].values())):
        with safe_open(os.path.join(d, shard), "pt") as f:
            for k in f.keys():
                v = f.get_tensor(k)
                out["w/" + k] = v.numpy() if v.dtype == torch.uint8 else bits(v)
    rc = torch.load(os.path.join(fx, "receipts_gpt_oss.pt"), weights_only=False)["host"]
    out["rc/prompt"], out["rc/cont"] = np.asarray(rc["prompt"][0], np.int64), np.asarray(rc["cont"][0], np.int64)
    out["rc/prompt_logits"], out["rc/next"] = rc["prompt_logits"].numpy(), rc["next"].numpy()
    out["rc/greedy"] = np.asarray(rc["greedy"], np.int64)


def main() -> None:
    if len(sys.argv) < 2 and not os.environ.get("BTB_REFERENCE"):
        raise SystemExit("usage: make_golden.py <reference checkout> (or BTB_REFERENCE=<checkout>)")
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ["BTB_REFERENCE"]
    sys.path.insert(0, ref)
    a: dict = {}
    codecs(ref, a)
    np.savez_compressed(os.path.join(HERE, "codecs.npz"), **a)
    b: dict = {}
    tiny(ref, b)
    np.savez_compressed(os.path.join(HERE, "tiny_qwen3.npz"), **b)
    c: dict = {}
    sampling(ref, c)
    np.savez_compressed(os.path.join(HERE, "sampling.npz"), **c)
    with open(os.path.join(HERE, "drafts.json"), "w") as f:
        json.dump(drafts(ref), f, separators=(",", ":"))
    d: dict = {}
    moe(ref, d)
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **d)
    e: dict = {}
    tiny_moe(ref, e)
    np.savez_compressed(os.path.join(HERE, "tiny_gpt_oss.npz"), **e)
    v: dict = {}
    verify(ref, v)
    np.savez_compressed(os.path.join(HERE, "verify.npz"), **v)
    for f in ("codecs.npz", "tiny_qwen3.npz", "sampling.npz", "drafts.json", "moe.npz", "tiny_gpt_oss.npz", "verify.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
