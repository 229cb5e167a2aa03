"""The paged KV cache on the card with a shared-prefix tree: conversations that begin alike hold the same pages once.

What this mirrors of btb: `PagePool` (btb/engine/kvpool.py:22, 53-149: PAGE = 64 rows of every layer, holders counted, the
lowest free page handed out first), a conversation's `Table` of rows (`page * PAGE + offset`, its logical positions in
order, btb/engine/paged.py:1-16) read by the kernels through the row map `tbl[logical] -> cache row`
(native/cuda/btb_kernels.cu:261-327, btb_attn_flash.cuh:652-658), and the prefix tree that lets a new conversation take
over the pages of the longest prompt prefix already computed (btb/engine/prefix.py, radix.py). btb spreads pages over the
card, pinned RAM and the host and moves them under a memory ledger; a B200 holds 180 GB, so here every page lives in HBM
and the bookkeeping is all there is: no tiers, nothing to move.

Sharing is by whole pages: a page enters the tree when its 64 rows are written, keyed by its 64 token ids under its
parent page, and is never written again; a conversation's last, partial page is its own. Pages no conversation holds
stay in the tree until the pool runs short, then the least recently used leaves go first.
"""

from __future__ import annotations

import heapq
from dataclasses import dataclass, field
from typing import Any

import torch

from . import capi
from .capi import call, ptr
from .engine import CardEngine, ModelWeights

PAGE = 64  # rows a page (btb/engine/kvpool.py:22)


class PoolError(RuntimeError):
    """no free page and nothing left to evict, or a holder's count gone wrong"""


@dataclass(eq=False)
class Page:
    id: int
    refs: int = 0  # holders: conversations' tables and the tree's nodes
    tick: int = 0


class PagePool:
    """`n_pages` pages of PAGE rows; `alloc` hands out the lowest free one, `unref` takes a page back with its last holder"""

    def __init__(self, n_pages: int):
        self.pages = [Page(i) for i in range(n_pages)]
        self.free = list(range(n_pages))
        heapq.heapify(self.free)
        self.clock = 0

    def __len__(self) -> int:
        return len(self.pages) - len(self.free)

    def alloc(self) -> Page:
        if not self.free:
            raise PoolError("no free page")
        p = self.pages[heapq.heappop(self.free)]
        p.refs = 1
        self.touch(p)
        return p

    def touch(self, p: Page) -> None:
        self.clock += 1
        p.tick = self.clock

    def ref(self, p: Page) -> None:
        if p.refs <= 0:
            raise PoolError(f"page {p.id} referenced after it was freed")
        p.refs += 1

    def unref(self, p: Page) -> bool:
        if p.refs <= 0:
            raise PoolError(f"page {p.id} let go more often than it was held")
        p.refs -= 1
        if p.refs == 0:
            heapq.heappush(self.free, p.id)
            return True
        return False

    def check(self) -> list[str]:
        free = set(self.free)
        bad = [f"page {p.id} is free with {p.refs} holders" for p in self.pages if p.id in free and p.refs]
        bad += [f"page {p.id} is held by no one and not free" for p in self.pages if p.id not in free and p.refs <= 0]
        return bad


@dataclass(eq=False)
class Node:
    """a full page in the tree: the 64 token ids it holds, under the page before it"""

    page: Page | None
    parent: "Node | None"
    key: tuple = ()
    children: dict = field(default_factory=dict)


class PrefixTree:
    """full pages by the token ids that filled them, each under its predecessor: the longest chain matching a prompt's
    start is cache already computed. The tree is a holder of every page in it."""

    def __init__(self, pool: PagePool):
        self.pool = pool
        self.root = Node(None, None)

    def match(self, ids: list[int]) -> list[Node]:
        """the nodes of the longest chain of whole pages that `ids` begins with"""
        node, out = self.root, []
        for a in range(0, len(ids) - PAGE + 1, PAGE):
            nxt = node.children.get(tuple(ids[a : a + PAGE]))
            if nxt is None:
                break
            out.append(nxt)
            node = nxt
        for n in out:
            self.pool.touch(n.page)
        return out

    def insert(self, parent: Node, key: tuple, page: Page) -> Node:
        """`page`, just filled with `key`'s tokens after `parent`'s, joins the tree (which now holds it too); if an equal
        page is there already (two conversations computed it side by side) that one is returned and `page` stays the
        caller's alone"""
        have = parent.children.get(key)
        if have is not None:
            return have
        self.pool.ref(page)
        node = Node(page, parent, key)
        parent.children[key] = node
        return node

    def evict(self, want: int) -> int:
        """lets go of up to `want` pages nobody but the tree holds, least recently used leaves first; returns how many"""
        done = 0
        while done < want:
            leaves = [n for n in self._nodes() if not n.children and n.page.refs == 1]
            if not leaves:
                break
            n = min(leaves, key=lambda x: x.page.tick)
            del n.parent.children[n.key]
            self.pool.unref(n.page)
            done += 1
        return done

    def _nodes(self):
        stack = list(self.root.children.values())
        while stack:
            n = stack.pop()
            yield n
            stack.extend(n.children.values())

    def __len__(self) -> int:
        return sum(1 for _ in self._nodes())


class Conversation:
    """one token stream's place in the cache: its pages in logical order and how many rows stand"""

    def __init__(self, eng: "PagedEngine"):
        self.eng = eng
        self.pages: list[Page] = []
        self.ids: list[int] = []  # the tokens whose rows stand in the cache
        self.node: Node = eng.tree.root  # the tree node of the last page that is in the tree
        self.shared = 0  # rows taken over from the tree when the conversation was attached

    def __len__(self) -> int:
        return len(self.ids)

    def release(self) -> None:
        for p in self.pages:
            self.eng.pool.unref(p)
        self.pages, self.ids = [], []


class PagedEngine(CardEngine):
    """the card engine over a page pool: the kernels read and write the cache through a row map, conversations that
    begin alike share pages, and `attach` prefills only what the tree does not hold"""

    def __init__(self, weights: ModelWeights, n_pages: int = 64, device: Any = "cuda", **kw: Any):
        super().__init__(weights, cap=n_pages * PAGE, device=device, **kw)
        self.pool = PagePool(n_pages)
        self.tree = PrefixTree(self.pool)
        # the row map of the conversation being decoded: logical row -> cache row (every layer's arena alike)
        self.tbl = torch.zeros(self.cap, dtype=torch.int32, device=self.dev)
        self.conv: Conversation | None = None
        self._bound: tuple = (0, 0)

    # -- pages -----------------------------------------------------------------------------------------------------------
    def _page(self) -> Page:
        if not self.pool.free and not self.tree.evict(1):
            raise PoolError("every page is held by a conversation")
        return self.pool.alloc()

    def _bind(self, c: Conversation, rows_ahead: int) -> None:
        """pages for `rows_ahead` more rows, and the row map on the card"""
        need = -(-(len(c) + rows_ahead) // PAGE)
        while len(c.pages) < need:
            c.pages.append(self._page())
        if self._bound != (id(c), len(c.pages)):  # the map changes only with the conversation or its page list
            rows = torch.tensor([p.id * PAGE for p in c.pages], dtype=torch.int32)
            tbl = (rows[:, None] + torch.arange(PAGE, dtype=torch.int32)[None, :]).reshape(-1)
            self.tbl[: tbl.numel()].copy_(tbl)
            self._bound = (id(c), len(c.pages))
        if self.conv is not c:
            self.n0.fill_(len(c))
        self.conv = c

    def _note(self, c: Conversation, toks: list[int]) -> None:
        """`toks`' rows now stand after the conversation's: pages they completed join the tree"""
        before = len(c) // PAGE
        c.ids.extend(int(t) for t in toks)
        for i in range(before, len(c) // PAGE):
            if i < c.shared // PAGE:
                continue
            c.node = self.tree.insert(c.node, tuple(c.ids[i * PAGE : (i + 1) * PAGE]), c.pages[i])

    # -- the public surface ----------------------------------------------------------------------------------------------
    def attach(self, prompt: Any) -> tuple[Conversation, torch.Tensor]:
        """a new conversation over `prompt`: the pages of its longest prefix already in the tree are taken over, the rest
        is prefilled. Returns the conversation and the last prompt row's logits [1, V]. At least the last token is always
        computed (its logits are wanted)."""
        ids = [int(t) for t in torch.as_tensor(prompt).tolist()]
        c = Conversation(self)
        nodes = self.tree.match(ids[: max(0, len(ids) - 1)])
        for n in nodes:
            self.pool.ref(n.page)
            c.pages.append(n.page)
        c.ids = ids[: len(nodes) * PAGE]
        c.shared = len(c.ids)
        if nodes:
            c.node = nodes[-1]
        rest = ids[c.shared :]
        self._bind(c, len(rest))
        last = None
        for a in range(0, len(rest), 32):
            chunk = rest[a : a + 32]
            last = self.forward(torch.tensor(chunk))[-1:].clone()
            self._note(c, chunk)
        return c, last

    def resume(self, c: Conversation, rows_ahead: int = 1) -> None:
        """make `c` the conversation the next steps decode"""
        self._bind(c, rows_ahead)

    def decode(self, c: Conversation, first: int, max_new: int) -> list[int]:
        """greedy tokens after `first` (the pick from the prompt's last logits): `first` itself, then max_new - 1 steps"""
        toks = [int(first)]
        while len(toks) < max_new:
            self.resume(c, 1)
            nxt = self.step(toks[-1])
            self._note(c, [toks[-1]])
            toks.append(nxt)
        return toks

    # -- the kernels' row map ----------------------------------------------------------------------------------------------
    def _attention(self, g: dict, i: int, wq: Any, wk: Any, T: int, s: int, win: int = 0, sinks: Any = None,
                   out: Any = None, warm: tuple = ()) -> None:  # fmt: skip
        c = self.cfg
        Hq, Hk, D = c.q_heads, c.kv_heads, c.head_dim
        out = g["att"] if out is None else out
        if T == 1 and self.fuse_attn and D in (64, 128):
            self._k("btb_b200_attn_step", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                    ptr(self.n0), ptr(g["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), ptr(out), Hq, Hk, D,
                    self.hs, self.rs, 0, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]), ptr(g["part_acc"]),
                    ptr(g["cnt"]), win, ptr(self.tbl), ptr(sinks), self.cap, s)  # fmt: skip
            return
        self._k("btb_b200_norm_rope_kv", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                ptr(self.n0), ptr(g["depth"]), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), T, Hq, Hk, D, self.hs,
                self.rs, 0, ptr(self.tbl), self.cap, s)  # fmt: skip
        self._k("btb_b200_attn_decode", ptr(g["q"]), ptr(self.K[i]), ptr(self.V[i]), ptr(out), ptr(self.n0),
                ptr(g["par"]), T, Hq, Hk, D, self.hs, self.rs, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]),
                ptr(g["part_acc"]), ptr(g["cnt"]), win, ptr(self.tbl), ptr(sinks), self.cap, s)  # fmt: skip
