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


def main() -> None:
    ref = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
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
    for f in ("codecs.npz", "tiny_qwen3.npz", "sampling.npz", "drafts.json"):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
