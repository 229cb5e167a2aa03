"""Small-batch decode: B sequences side by side on one card - each with its own cache and length (`BatchEngine`), or as
rows of one cache in btb's rows layout, forks of a shared prefix included (`RowsEngine`).

btb's batched greedy loop (btb/engine/generate.py:985-1046) decodes B rows a step over a cache whose rows stand at
their own lengths (btb/engine/cache.py:334-337). Here a step is ONE pass of B rows through the same kernels as the
one-sequence step - every weight is streamed once for all B tokens - and only the attention differs: row b reads
sequence b's cache (`btb_b200_attn_step_batch`). The kernels are row-invariant, so sequence b's tokens are the tokens
the one-sequence engine gives for its prompt (tested).
"""

from __future__ import annotations

from typing import Any

import torch

from . import capi
from .capi import ptr
from .engine import CardEngine, ModelWeights, pad_rows


class BatchEngine(CardEngine):
    """B sequences on one card: caches [L, B, cap, Hk, D], lengths int32 [B], one pass of B rows a step"""

    def __init__(self, weights: ModelWeights, batch: int, cap: int = 4096, device: Any = "cuda"):
        if not 1 <= batch <= 32:
            raise ValueError("1 to 32 sequences a pass")
        super().__init__(weights, cap=cap, step_kernel=False, device=device)
        c = self.cfg
        self.B = int(batch)
        self.Kb = torch.zeros(c.layers, self.B, self.cap, c.kv_heads, c.head_dim, dtype=torch.bfloat16, device=self.dev)
        self.Vb = torch.zeros_like(self.Kb)
        self.n0b = torch.zeros(self.B, dtype=torch.int32, device=self.dev)
        self.seq_stride = self.cap * c.kv_heads * c.head_dim
        self._one = (self.K, self.V, self.n0)  # the one-sequence views the parent's passes use
        self._side_by_side = False
        self.pin_toks = torch.zeros(self.B, dtype=torch.int64).pin_memory()
        self._bgraph: Any = None
        self._zeros = torch.zeros(32, dtype=torch.int32, device=self.dev)  # every row is depth 0 of its own sequence

    # a sequence's own cache and length as the parent's one-sequence state (its prefill runs the parent's passes)
    def _select(self, b: int) -> None:
        self.K, self.V, self.n0 = self.Kb[:, b], self.Vb[:, b], self.n0b[b : b + 1]

    def reset(self) -> None:
        self.n0b.zero_()

    def _attention(self, g: dict, i: int, wq: Any, wk: Any, T: int, s: int, win: int = 0, sinks: Any = None,
                   out: Any = None, warm: tuple = ()) -> None:  # fmt: skip
        if not self._side_by_side:
            return super()._attention(g, i, wq, wk, T, s, win, sinks, out, warm)
        c = self.cfg
        Hq, Hk, D = c.q_heads, c.kv_heads, c.head_dim
        out = g["att"] if out is None else out
        self._k("btb_b200_attn_step_batch", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                ptr(self.n0b), ptr(self._zeros), ptr(self.Kb[i]), ptr(self.Vb[i]), ptr(g["q"]), ptr(out), T,
                self.seq_stride, Hq, Hk, D, self.hs, self.rs, 0, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]),
                ptr(g["part_acc"]), ptr(g["cnt"]), win, ptr(sinks), self.cap, s)  # fmt: skip

    def _batch_step(self, s: int) -> None:
        """ids [B] -> one pass of B rows -> the picks into ids, every length + 1, the tokens to pinned memory"""
        B = self.B
        g = self.bufs(pad_rows(B))
        self._n = 0
        self._side_by_side = True
        try:
            self._embed(g, B, s)
            self.body(B, stream_ptr=s)
            self._pick(g, B, s, g["ids"])
        finally:
            self._side_by_side = False
        self.n0b.add_(1)
        self.pin_toks.copy_(g["ids"][:B], non_blocking=True)
        self.launches_per_step = self._n

    def batch_graph(self) -> Any:
        if self._bgraph is not None:
            return self._bgraph
        M = pad_rows(self.B)
        g = self.bufs(M)
        keep_n, keep_ids = self.n0b.clone(), g["ids"].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._batch_step(capi.stream_ptr(side))
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.n0b.copy_(keep_n)
        g["ids"].copy_(keep_ids)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._batch_step(capi.stream_ptr())
        self.n0b.copy_(keep_n)
        g["ids"].copy_(keep_ids)
        self._bgraph = graph
        return graph

    def prefill_all(self, prompts: list[Any]) -> list[int]:
        """each sequence's prompt through the one-sequence passes into its own cache; returns the first tokens"""
        if len(prompts) != self.B:
            raise ValueError(f"{len(prompts)} prompts for {self.B} sequences")
        g1 = self.bufs(1)
        gB = self.bufs(pad_rows(self.B))
        s = capi.stream_ptr()
        first = []
        self.reset()
        try:
            for b, p in enumerate(prompts):
                self._select(b)
                last = self.prefill(torch.as_tensor(p, dtype=torch.int64))
                self._pick({"logits": last.contiguous(), "pick": g1["pick"], "depth": self._before}, 1, s, g1["tok"])
                first.append(int(g1["tok"][0].item()))
        finally:
            self.K, self.V, self.n0 = self._one
        gB["ids"][: self.B].copy_(torch.tensor(first, dtype=torch.int64))
        return first

    def generate_batch(self, prompts: list[Any], max_new: int) -> list[list[int]]:
        """greedy decode of every sequence, a step for all of them at a time"""
        toks = [[t] for t in self.prefill_all(prompts)]
        graph = self.batch_graph()
        for _ in range(max_new - 1):
            graph.replay()
            torch.cuda.current_stream().synchronize()
            for b in range(self.B):
                toks[b].append(int(self.pin_toks[b]))
        return toks


class RowsEngine(CardEngine):
    """The rows layout (btb/engine/cuda.py:3445-3500 `_card_rows_step`, native/cuda/btb_kernels.cu:228-248): a pass's B
    rows as B sequences of one token each in ONE cache - the forks of a prompt, which share its rows as their prefix, or a
    batch of prompts lying end to end - each row at its own position. Row b's keys are its prefix (`len` cache rows from
    `off`) and then its own steps, step i at cache row base + i * W + col, every row's step i in one stretch of W rows.
    A row reads its keys in logical order, so its bits are its own one-sequence decode's whatever rows step beside it."""

    def __init__(self, weights: ModelWeights, cap: int = 4096, device: Any = "cuda"):
        super().__init__(weights, cap=cap, step_kernel=False, device=device)
        self.rw = torch.zeros(3 + 3 * 32, dtype=torch.int32, device=self.dev)
        self.B = 0
        self._rows = False
        self._rgraph: dict[int, Any] = {}
        self.pin_rows = torch.zeros(32, dtype=torch.int64).pin_memory()
        self.lens: list[int] = []

    # -- forming the rows ------------------------------------------------------------------------------------------------
    def _layout(self, offs: list[int], lens: list[int], base: int) -> None:
        B = len(lens)
        if not 1 <= B <= 32:
            raise ValueError("1 to 32 rows a pass")
        M = pad_rows(B)
        lay = [base, 0, M]
        for b in range(B):
            lay += [b, offs[b], lens[b]]
        lay += [0, 0, -1] * (M - B)  # the rows past B are padding the kernels skip
        self.rw[: len(lay)].copy_(torch.tensor(lay, dtype=torch.int32))
        self.B, self.lens, self.base, self.W = B, list(lens), base, M

    def fork(self, prompt: Any, B: int) -> torch.Tensor:
        """the prompt prefilled once, B rows that share its cache rows as their prefix; returns the prompt's last logits
        [1, V] (the rows' first tokens are the caller's choice: B samples, the B best, ...)"""
        self.reset()
        last = self.prefill(torch.as_tensor(prompt, dtype=torch.int64))
        n = int(torch.as_tensor(prompt).numel())
        self._layout([0] * B, [n] * B, n)
        return last

    def batch(self, prompts: list[Any]) -> list[torch.Tensor]:
        """every prompt prefilled (at positions 0..), its rows moved end to end; returns each prompt's last logits"""
        lens = [int(torch.as_tensor(p).numel()) for p in prompts]
        offs = [sum(lens[:b]) for b in range(len(lens))]
        lasts = []
        for b in reversed(range(len(prompts))):  # back to front: a prompt's rows land past the scratch range [0, len)
            self.reset()
            lasts.append(self.prefill(torch.as_tensor(prompts[b], dtype=torch.int64)).clone())
            if offs[b]:
                for i in range(self.cfg.layers):
                    self.K[i][offs[b] : offs[b] + lens[b]].copy_(self.K[i][: lens[b]].clone())
                    self.V[i][offs[b] : offs[b] + lens[b]].copy_(self.V[i][: lens[b]].clone())
        self._layout(offs, lens, sum(lens))
        return lasts[::-1]

    # -- the pass -----------------------------------------------------------------------------------------------------------
    def _attention(self, g: dict, i: int, wq: Any, wk: Any, T: int, s: int, win: int = 0, sinks: Any = None,
                   out: Any = None, warm: tuple = ()) -> None:  # fmt: skip
        if not self._rows:
            return super()._attention(g, i, wq, wk, T, s, win, sinks, out, warm)
        c = self.cfg
        Hq, Hk, D = c.q_heads, c.kv_heads, c.head_dim
        out = g["att"] if out is None else out
        M = pad_rows(T)
        self._k("btb_b200_norm_rope_kv_rows", ptr(g["qkv"]), ptr(wq), ptr(wk), c.eps, ptr(self.cos), ptr(self.sin),
                ptr(self.rw), ptr(self.K[i]), ptr(self.V[i]), ptr(g["q"]), M, Hq, Hk, D, self.hs, self.rs, 0, self.cap, s)
        self._k("btb_b200_attn_decode_rows", ptr(g["q"]), ptr(self.K[i]), ptr(self.V[i]), ptr(out), ptr(self.rw), M, Hq,
                Hk, D, self.hs, self.rs, float(D**-0.5), ptr(g["part_m"]), ptr(g["part_l"]), ptr(g["part_acc"]),
                ptr(g["cnt"]), win, ptr(sinks), self.cap, s)  # fmt: skip

    def _rows_pass(self, s: int) -> None:
        """ids [B] -> one pass of B rows -> logits [B, V], the greedy picks into ids, the layout's step + 1"""
        B = self.B
        g = self.bufs(pad_rows(B))
        self._n = 0
        self._rows = True
        try:
            self._embed(g, B, s)
            self.body(B, stream_ptr=s)
            self._k("btb_b200_argmax_bf16", ptr(g["logits"]), B, self.cfg.vocab, ptr(g["pick"]), ptr(g["ids"]), s)
        finally:
            self._rows = False
        self.rw[1:2].add_(1)
        self.pin_rows[:B].copy_(g["ids"][:B], non_blocking=True)
        self.launches_per_step = self._n

    def rows_graph(self) -> Any:
        """the pass captured for this width (the layout is data: forming new rows of the same width needs no capture)"""
        M = pad_rows(self.B)
        if M in self._rgraph:
            return self._rgraph[M]
        g = self.bufs(M)
        keep_rw, keep_ids = self.rw.clone(), g["ids"].clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._rows_pass(capi.stream_ptr(side))  # (the eager run writes this step's cache rows, which the replay rewrites)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.rw.copy_(keep_rw)
        g["ids"].copy_(keep_ids)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._rows_pass(capi.stream_ptr())
        self.rw.copy_(keep_rw)
        g["ids"].copy_(keep_ids)
        self._rgraph[M] = graph
        return graph

    def rows_step(self, toks: list[int]) -> torch.Tensor:
        """one token into each row: the rows' logits [B, V] bf16 (a view of the pass's buffer)"""
        if len(toks) != self.B:
            raise ValueError(f"{len(toks)} tokens for {self.B} rows")
        if self.base + (int(self.rw[1]) + 1) * self.W > self.cap:
            raise ValueError("the rows' next step does not fit the cache")
        g = self.bufs(pad_rows(self.B))
        g["ids"][: self.B].copy_(torch.tensor(toks, dtype=torch.int64))
        self.rows_graph().replay()
        return g["logits"][: self.B]

    def generate_rows(self, firsts: list[int], max_new: int) -> list[list[int]]:
        """greedy decode of every row after its first token, a pass for all of them at a time"""
        toks = [[int(t)] for t in firsts]
        g = self.bufs(pad_rows(self.B))
        g["ids"][: self.B].copy_(torch.tensor(firsts, dtype=torch.int64))
        graph = self.rows_graph()
        for _ in range(max_new - 1):
            graph.replay()
            torch.cuda.current_stream().synchronize()
            for b in range(self.B):
                toks[b].append(int(self.pin_rows[b]))
        return toks
