"""The whole-step kernel's program: btb's card graph body (btb/engine/cuda.py:1722-1834 `_card_body`, :2227-2249 the
step's embed / pick / publish) written down as data - one record a phase - for ``btb_b200_step`` to walk.

The records mirror ``StepOp`` / ``StepArgs`` of ``csrc/step.cu`` field for field (ctypes lays a Structure out as the C
compiler does; the sizes are checked against the library's at import of a program).
"""

from __future__ import annotations

import ctypes as C
from typing import Any

import torch

from . import capi
from .capi import ptr

OP_END, OP_GEMV, OP_ROPE, OP_ATTN, OP_PICK = 0, 1, 2, 3, 4
XK_COPY, XK_SILU, XK_NORM = 0, 1, 2
F_BF16, F_P12 = 0, 1
NWS = 16  # warps a CTA of the step kernel

_P = C.c_void_p


class StepOp(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("fmt", C.c_int32), ("xkind", C.c_int32), ("R", C.c_int32), ("C", C.c_int32),
        ("seg", C.c_int32), ("next_gemv", C.c_int32), ("centered", C.c_int32),
        ("eps", C.c_float), ("scale", C.c_float), ("win", C.c_int32), ("pad0", C.c_int32),
        ("w", _P), ("hi4", _P), ("esc_idx", _P), ("esc_val", _P), ("esc_row", _P),
        ("table", C.c_uint8 * 16),
        ("x", _P), ("y", _P), ("h_in", _P), ("y_add", _P), ("norm_w", _P), ("h_out", _P), ("rows", _P),
        ("wq", _P), ("wk", _P), ("K", _P), ("V", _P), ("q", _P), ("att", _P),
    ]  # fmt: skip


class StepArgs(C.Structure):
    _fields_ = [
        ("ops", _P),
        ("n_ops", C.c_int32), ("first_gemv", C.c_int32), ("T", C.c_int32), ("steps", C.c_int32), ("S", C.c_int32),
        ("stage_cap", C.c_int32), ("front_bytes", C.c_int32), ("norm_bytes", C.c_int32),
        ("cap", C.c_int32), ("Hq", C.c_int32), ("Hk", C.c_int32), ("vocab", C.c_int32),
        ("hs", C.c_longlong), ("rs", C.c_longlong),
        ("n0", _P), ("depth", _P), ("par", _P), ("tbl", _P), ("sinks", _P), ("cos_t", _P), ("sin_t", _P),
        ("part_m", _P), ("part_l", _P), ("part_acc", _P), ("cnt", _P),
        ("bar", _P), ("abort_flag", _P), ("logits", _P), ("pick_keys", _P), ("ids", _P), ("tok_out", _P),
        ("pin_tok", _P), ("pin_n0", _P), ("pin_ts", _P),
        ("advance", C.c_int32), ("pick", C.c_int32),
        ("trace", _P), ("trace_cta", C.c_int32), ("pad1", C.c_int32),
    ]  # fmt: skip


def _round_up(a: int, b: int) -> int:
    return -(-a // b) * b


def seg_for(C_: int, fmt: int, stage_cap: int) -> int:
    """a row's segment in elements: equal parts, each a multiple of 256 columns, each stage within `stage_cap`"""
    per_el = 2.0 if fmt == F_BF16 else 1.5
    max_el = max(256, int(stage_cap / per_el) // 256 * 256)
    nseg = -(-C_ // max_el)
    return _round_up(-(-C_ // nseg), 256)


class StepProgram:
    """one pass width's program and launch arguments on the card; ``launch(stream)`` enqueues the whole step"""

    def __init__(self, eng: Any, M: int, steps: int, pick: bool, publish: bool, ring_bytes: int = 160 * 1024,
                 stage_cap: int = 2560):  # fmt: skip
        from .engine import P12Matrix

        lib = capi.lib()
        if lib.btb_b200_step_op_bytes() != C.sizeof(StepOp) or lib.btb_b200_step_args_bytes() != C.sizeof(StepArgs):
            raise RuntimeError("step.py and csrc/step.cu disagree about the program's layout")
        c, g, w = eng.cfg, eng.bufs(M), eng.w
        self.eng, self.M, self.steps = eng, M, steps
        H, Hq, Hk, D, I = c.hidden, c.q_heads, c.kv_heads, c.head_dim, c.inter
        self.D, self.G = D, Hq // Hk
        p12_any = any(isinstance(m, P12Matrix) for L in w.layers for m in (L.qkv, L.o, L.gu, L.down))
        if p12_any:
            stage_cap = _round_up(int(stage_cap * 1.5), 128)
        ops: list[StepOp] = []

        def gemv(W: Any, R: int, C_: int, y: torch.Tensor, **kw: Any) -> None:
            op = StepOp()
            op.kind, op.R, op.C = OP_GEMV, R, C_
            if isinstance(W, P12Matrix):
                op.fmt = F_P12
                op.w, op.hi4 = ptr(W.lo), ptr(W.hi4)
                op.esc_idx, op.esc_val, op.esc_row = ptr(W.esc_idx), ptr(W.esc_val), ptr(W.esc_row)
                op.table = (C.c_uint8 * 16)(*W.table)
            else:
                op.fmt, op.w = F_BF16, ptr(W)
            op.seg = seg_for(C_, op.fmt, stage_cap)
            op.y = ptr(y)
            op.eps = c.eps
            for k, v in kw.items():
                setattr(op, k, v)
            ops.append(op)

        hcur, halt = g["h"], g["h2"]
        y_prev = None
        for i, L in enumerate(w.layers):
            first = i == 0
            gemv(L.qkv, c.qkv_rows, H, g["qkv"], xkind=XK_NORM, h_in=ptr(w.embed) if first else ptr(hcur),
                 rows=ptr(g["ids"]) if first else 0, y_add=ptr(y_prev), norm_w=ptr(L.ln1),
                 h_out=ptr(hcur) if first else ptr(halt))  # fmt: skip
            if not first:
                hcur, halt = halt, hcur
            op = StepOp()
            op.kind, op.x, op.wq, op.wk = OP_ROPE, ptr(g["qkv"]), ptr(L.wq), ptr(L.wk)
            op.K, op.V, op.q, op.eps = ptr(eng.K[i]), ptr(eng.V[i]), ptr(g["q"]), c.eps
            ops.append(op)
            op = StepOp()
            op.kind, op.K, op.V, op.q, op.att = OP_ATTN, ptr(eng.K[i]), ptr(eng.V[i]), ptr(g["q"]), ptr(g["att"])
            op.scale, op.win = float(D**-0.5), 0
            ops.append(op)
            gemv(L.o, H, Hq * D, g["y"], xkind=XK_COPY, x=ptr(g["att"]))
            gemv(L.gu, 2 * I, H, g["gu"], xkind=XK_NORM, h_in=ptr(hcur), y_add=ptr(g["y"]), norm_w=ptr(L.ln2),
                 h_out=ptr(halt))  # fmt: skip
            hcur, halt = halt, hcur
            gemv(L.down, H, I, g["y"], xkind=XK_SILU, x=ptr(g["gu"]))
            y_prev = g["y"]
        gemv(w.embed, c.vocab, H, g["logits"], xkind=XK_NORM, h_in=ptr(hcur), y_add=ptr(y_prev), norm_w=ptr(w.norm),
             h_out=ptr(halt))  # fmt: skip
        if pick:
            op = StepOp()
            op.kind = OP_PICK
            ops.append(op)
        # each GEMV's successor in the program; the last one wraps to the first (the next step's) when steps repeat
        gi = [k for k, o in enumerate(ops) if o.kind == OP_GEMV]
        for a, b in zip(gi, gi[1:]):
            ops[a].next_gemv = b
        ops[gi[-1]].next_gemv = gi[0] if steps > 1 else -1
        for o in ops:
            if o.kind != OP_GEMV:
                o.next_gemv = -1
        arr = (StepOp * len(ops))(*ops)
        self.ops_dev = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(eng.dev)
        # shared memory: [norm scratch | x] overlaid by the attention's scratch, then the rings
        norm_bytes = _round_up(H * 4 + 256 * 4, 128)
        x_bytes = _round_up(M * max(H, Hq * D, I) * 2, 128)
        G = self.G
        attn_bytes = 4 * (G * D + 2 * 8 * 2 * G + NWS * G * 32 + NWS * G * D)
        front = _round_up(max(norm_bytes + x_bytes, attn_bytes), 128)
        S = max(2, min(8, (ring_bytes // NWS) // stage_cap))
        while front + NWS * S * stage_cap + NWS * S * 8 > 224 * 1024 and S > 2:
            S -= 1
        self.state = torch.zeros(4, dtype=torch.int32, device=eng.dev)  # [0] barrier counter, [1] abort flag
        self.tok_out = torch.zeros(max(1, steps), dtype=torch.int64, device=eng.dev)
        a = StepArgs()
        a.ops, a.n_ops, a.first_gemv = ptr(self.ops_dev), len(ops), gi[0]
        a.T, a.steps, a.S, a.stage_cap, a.front_bytes, a.norm_bytes = M, steps, S, stage_cap, front, norm_bytes
        a.cap, a.Hq, a.Hk, a.vocab, a.hs, a.rs = eng.cap, Hq, Hk, c.vocab, eng.hs, eng.rs
        a.n0, a.depth, a.par = ptr(eng.n0), ptr(g["depth"]), ptr(g["par"])
        a.cos_t, a.sin_t = ptr(eng.cos), ptr(eng.sin)
        a.part_m, a.part_l, a.part_acc, a.cnt = ptr(g["part_m"]), ptr(g["part_l"]), ptr(g["part_acc"]), ptr(g["cnt"])
        a.bar, a.abort_flag = ptr(self.state), ptr(self.state) + 4
        a.logits, a.pick_keys, a.ids = ptr(g["logits"]), ptr(g["pick"]), ptr(g["ids"])
        a.tok_out = ptr(self.tok_out)
        if publish:
            a.pin_tok, a.pin_n0, a.pin_ts = ptr(eng.pin_tok), ptr(eng.pin_n0), ptr(eng.pin_ts)
        a.advance, a.pick = M if not pick else 1, 1 if pick else 0
        self.args = a
        self.kinds = [o.kind for o in ops]
        self.n_phases = len(ops)
        self.smem = front + NWS * S * stage_cap + NWS * S * 8

    def trace(self, cta: int = 0) -> torch.Tensor:
        """switch on the per-phase device clock of one CTA; returns the [n_phases, 2] buffer the next launches fill"""
        self._trace = torch.zeros(self.n_phases, 2, dtype=torch.int64, device=self.eng.dev)
        self.args.trace, self.args.trace_cta = ptr(self._trace), cta
        return self._trace

    def launch(self, T: int | None = None, stream: Any = None) -> None:
        """zero the barrier state, then the one launch; T live rows of the width's M (default: all M)"""
        if T is not None:
            self.args.T = T
            if not self.args.pick:
                self.args.advance = T
        s = torch.cuda.current_stream() if stream is None else stream
        with torch.cuda.stream(s):
            self.state.zero_()
        capi.call("btb_b200_step", C.byref(self.args), self.M, self.D, self.G, int(s.cuda_stream))
