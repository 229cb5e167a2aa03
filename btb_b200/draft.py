"""n-gram drafting and the speculative greedy loop over the card engine.

Mirrors btb's host-side drafting (btb/draft.py:8-113 `NGramProposer`, btb/engine/generate.py:94-117 `_chains_tree`,
:682-795 the verify pass and the walk, btb/engine/cuda.py:3535-3575 the in-place commit): continuations of the text's
tail are looked up by n-gram, merged into a tree of at most `budget` guesses, verified in ONE pass whose row t is
bit-for-bit the step at its position (the kernels are row-invariant), and the accepted branch's cache rows are
gathered to the front. The tokens are therefore exactly the greedy loop's; only the number of passes changes.
"""

from __future__ import annotations

from collections.abc import Iterable, Sequence
from typing import Any

import torch

from . import capi
from .capi import call, ptr


class NGramProposer:
    """per order n in [n_min, n_max]: each n-gram's followers with their count and the position after the latest
    occurrence (btb/draft.py:8-74)"""

    def __init__(self, corpus_ids: Iterable[int], n_max: int = 4, n_min: int = 2, followers: int = 4) -> None:
        self.corpus: list[int] = []
        self.n_max, self.n_min, self.followers = n_max, n_min, max(1, int(followers))
        self.maps: dict[int, dict[tuple[int, ...], dict[int, list[int]]]] = {n: {} for n in range(n_min, n_max + 1)}
        for t in corpus_ids:
            self.extend(int(t))

    def extend(self, tok: int) -> None:
        self.corpus.append(tok)
        hi = len(self.corpus)
        for n in range(self.n_min, self.n_max + 1):
            i = hi - n - 1
            if i >= 0:
                key = tuple(self.corpus[i : i + n])
                slot = self.maps[n].setdefault(key, {})
                e = slot.get(tok)
                if e is None:
                    slot[tok] = [1, i + n]
                else:
                    e[0] += 1
                    e[1] = i + n

    def _followers(self, n: int, key: tuple[int, ...]) -> list[tuple[int, int]]:
        d = self.maps[n].get(key)
        if not d:
            return []
        return sorted(((c, p) for c, p in d.values()), reverse=True)[: self.followers]

    def propose_chains(self, v: int) -> list[tuple[list[int], str]]:
        """distinct continuations of up to v tokens: longest order first, most frequent follower first; a chain equal
        to or a prefix of an earlier one is dropped (btb/draft.py:76-97)"""
        out: list[tuple[list[int], str]] = []
        if v <= 0:
            return out
        for n in range(self.n_max, self.n_min - 1, -1):
            if len(self.corpus) < n:
                continue
            key = tuple(self.corpus[-n:])
            for _c, at in self._followers(n, key):
                c = self.corpus[at : at + v]
                if c and not any(o[: len(c)] == c for o, _ in out):
                    out.append((list(c), f"ngram{n}"))
        return out


def chains_tree(chains: Sequence[tuple[Sequence[int], str]], budget: int):
    """chains merged by shared prefix: node 0 the root, node j > 0 carrying guesses[j - 1]; (guesses, parents, depth,
    children), at most `budget` guesses (btb/engine/generate.py:94-117)"""
    guesses: list[int] = []
    parents, depth = [-1], [0]
    children: dict[int, list[int]] = {}
    for toks, _tag in chains:
        node = 0
        for d, t in enumerate(toks):
            t = int(t)
            nxt = next((c for c in children.get(node, []) if guesses[c - 1] == t), None)
            if nxt is None:
                if len(guesses) >= budget:
                    break
                nxt = len(guesses) + 1
                guesses.append(t)
                parents.append(node)
                depth.append(d + 1)
                children.setdefault(node, []).append(nxt)
            node = nxt
    return guesses, parents, depth, children


def walk(picks: Sequence[int], guesses: Sequence[int], children: dict[int, list[int]]) -> list[int]:
    """the accepted branch: from the root, the child whose guess is the node's own pick, as long as there is one
    (btb/engine/generate.py:765-795)"""
    node, path = 0, [0]
    while True:
        nxt = next((c for c in children.get(node, []) if guesses[c - 1] == picks[node]), None)
        if nxt is None:
            return path
        node = nxt
        path.append(nxt)


def generate_speculative(eng: Any, prompt: Any, max_new: int, budget: int = 8, v_max: int = 8,
                         events: Any = None) -> tuple[list[int], dict]:
    """greedy decode with n-gram tree drafts; returns (tokens, stats). The tokens are the plain greedy loop's.
    events: a pair of CUDA events recorded after the prefill's pick and after the last commit (the decode alone)."""
    prompt = [int(t) for t in torch.as_tensor(prompt).tolist()]
    eng.reset()
    last = eng.prefill(torch.tensor(prompt))
    g1 = eng.bufs(1)
    s = capi.stream_ptr()
    eng._pick({"logits": last.contiguous(), "pick": g1["pick"], "depth": eng._before}, 1, s, g1["tok"])
    cur = int(g1["tok"][0].item())
    toks = [cur]
    prop = NGramProposer(prompt + [cur])
    passes = 0
    if events is not None:
        events[0].record()
    c = eng.cfg
    row_el = c.kv_heads * c.head_dim
    while len(toks) < max_new:
        guesses, parents, depth, children = chains_tree(prop.propose_chains(v_max), min(budget, 31))
        T = 1 + len(guesses)
        g = eng.bufs(_pad(T))
        eng.forward(torch.tensor([cur] + guesses), depth=depth, parents=parents, advance=False)
        eng._pick(g, T, s, g["tok"])
        picks = g["tok"][:T].tolist()
        path = walk(picks, guesses, children)[: max_new - len(toks)]  # no row past the last token asked for
        pt = torch.tensor(path, dtype=torch.int32, device=eng.dev)
        call("btb_b200_kv_commit", ptr(eng.K), ptr(eng.V), eng.K[0].numel(), c.layers, ptr(eng.n0), ptr(pt), len(path),
             row_el, eng.rs, 0, eng.cap, s)
        call("btb_b200_publish", ptr(eng.n0), 0, 0, 0, 0, len(path), s)
        new = [picks[n] for n in path]
        for t in new:
            prop.extend(t)
        toks += new
        cur = new[-1]
        passes += 1
    if events is not None:
        events[1].record()
    torch.cuda.synchronize()
    return toks[:max_new], {"passes": passes, "tokens_per_pass": (len(toks) - 1) / max(1, passes)}


def _pad(T: int) -> int:
    from .engine import pad_rows

    return pad_rows(T)
