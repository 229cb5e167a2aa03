"""n-gram drafting and the speculative greedy loop over the card engine.

Mirrors btb's host-side drafting (btb/draft.py:8-113 `NGramProposer`, btb/engine/generate.py:94-117 `_chains_tree`,
:682-795 the verify pass and the walk, btb/engine/cuda.py:3535-3575 the in-place commit): continuations of the text's
tail are looked up by n-gram, merged into a tree of at most `budget` guesses, verified in ONE pass whose row t is
bit-for-bit the step at its position (the kernels are row-invariant), and the accepted branch's cache rows are
gathered to the front. The tokens are therefore exactly the greedy loop's; only the number of passes changes.
"""

from __future__ import annotations

import ctypes as C
from collections.abc import Iterable, Sequence
from typing import Any

import torch

from . import capi
from .capi import call, ptr


class NGramProposer:
    """the library's n-gram index behind btb's proposer interface (btb/draft.py:8-113): `extend(token)` and
    `propose_chains(v)` -> [(tokens, "ngram<order>"), ...]"""

    def __init__(self, corpus_ids: Iterable[int], n_max: int = 4, n_min: int = 2, followers: int = 4) -> None:
        L = capi.lib()
        self._h = L.btb_b200_ngram_new(int(n_max), int(n_min), int(followers))
        if not self._h:
            raise ValueError(f"n-gram orders {n_min}..{n_max} are not served")
        self._free = L.btb_b200_ngram_free
        self.n_max, self.n_min, self.followers = n_max, n_min, max(1, int(followers))
        ids = [int(t) for t in corpus_ids]
        if ids:
            call("btb_b200_ngram_extend", self._h, (C.c_longlong * len(ids))(*ids), len(ids))

    def __del__(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._free(h)

    def __len__(self) -> int:
        return int(capi.lib().btb_b200_ngram_length(self._h))

    def extend(self, tok: int) -> None:
        call("btb_b200_ngram_extend", self._h, (C.c_longlong * 1)(int(tok)), 1)

    def propose_chains(self, v: int) -> list[tuple[list[int], str]]:
        """distinct continuations of the text's tail, up to v tokens each: longest order first, most frequent follower
        first; a chain equal to or a prefix of an earlier one is dropped"""
        most = (self.n_max - self.n_min + 1) * self.followers
        if v <= 0:
            return []
        toks, offs, order = (C.c_int * (most * v))(), (C.c_int * (most + 1))(), (C.c_int * most)()
        n = C.c_int(0)
        call("btb_b200_ngram_chains", self._h, int(v), most, toks, offs, order, C.byref(n))
        return [(list(toks[offs[c] : offs[c + 1]]), f"ngram{order[c]}") for c in range(n.value)]

    def tree(self, v: int, budget: int) -> tuple[list[int], list[int], list[int]]:
        """`propose_chains(v)` merged into a tree of at most `budget` guesses, in one call: (guesses, parents, depth)"""
        g, par, dep = (C.c_int * max(budget, 1))(), (C.c_int * (budget + 1))(), (C.c_int * (budget + 1))()
        n = C.c_int(0)
        call("btb_b200_ngram_tree", self._h, int(v), int(budget), g, par, dep, C.byref(n))
        return list(g[: n.value]), list(par[: n.value + 1]), list(dep[: n.value + 1])


def chains_tree(chains: Sequence[tuple[Sequence[int], str]], budget: int):
    """chains merged by shared prefix (btb/engine/generate.py:94-117): node 0 the root, node j > 0 carrying
    guesses[j - 1]; (guesses, parents, depth, children), at most `budget` guesses. Takes any proposer's chains - the
    reference's own `NGramProposer.propose_chains` output included."""
    flat = [int(t) for toks, _tag in chains for t in toks]
    offs = [0]
    for toks, _tag in chains:
        offs.append(offs[-1] + len(toks))
    g, par, dep = (C.c_int * max(budget, 1))(), (C.c_int * (budget + 1))(), (C.c_int * (budget + 1))()
    n = C.c_int(0)
    call("btb_b200_chains_tree", (C.c_int * max(len(flat), 1))(*flat), (C.c_int * len(offs))(*offs), len(chains),
         int(budget), g, par, dep, C.byref(n))  # fmt: skip
    guesses, parents, depth = list(g[: n.value]), list(par[: n.value + 1]), list(dep[: n.value + 1])
    return guesses, parents, depth, children_of(parents)


def children_of(parents: Sequence[int]) -> dict[int, list[int]]:
    """each node's children in node order, from the parents list"""
    children: dict[int, list[int]] = {}
    for j, p in enumerate(parents):
        if p >= 0:
            children.setdefault(p, []).append(j)
    return children


def walk(picks: Sequence[int], guesses: Sequence[int], children: dict[int, list[int]]) -> list[int]:
    """the accepted branch (btb/engine/generate.py:765-795): from the root, the child whose guess is the node's own pick,
    as long as there is one"""
    n = 1 + len(guesses)
    parents = [-1] * n
    for p, cs in children.items():
        for c in cs:
            parents[c] = int(p)
    path, m = (C.c_int * n)(), C.c_int(0)
    call("btb_b200_tree_walk", (C.c_longlong * n)(*[int(t) for t in picks[:n]]), (C.c_int * max(n - 1, 1))(*guesses),
         (C.c_int * n)(*parents), n, path, C.byref(m))  # fmt: skip
    return list(path[: m.value])


def generate_speculative(eng: Any, prompt: Any, max_new: int, budget: int = 8, v_max: int = 8,
                         events: Any = None, proposer: Any = None) -> tuple[list[int], dict]:
    """greedy decode with n-gram tree drafts; returns (tokens, stats). The tokens are the plain greedy loop's.
    events: a pair of CUDA events recorded after the prefill's pick and after the last commit (the decode alone).
    proposer: a factory `proposer(ids) -> object with extend(token) and propose_chains(v)` - btb's own
    `btb.draft.NGramProposer` fits as it is; None: the library's native index."""
    prompt = [int(t) for t in torch.as_tensor(prompt).tolist()]
    eng.reset()
    last = eng.prefill(torch.tensor(prompt))
    g1 = eng.bufs(1)
    s = capi.stream_ptr()
    eng._pick({"logits": last.contiguous(), "pick": g1["pick"], "depth": eng._before}, 1, s, g1["tok"])
    cur = int(g1["tok"][0].item())
    toks = [cur]
    prop = (proposer or NGramProposer)(prompt + [cur])
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
