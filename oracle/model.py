"""TEST INFRASTRUCTURE - not a product path.

The dense decoder block composed from the oracle's functions, in the two arithmetic modes the reference has:

``CpuTier``   f32 activations over bf16 weights, 16-lane GEMV (btb/engine/host.py:98-134 -> native/src/gemv.rs),
              Hugging Face's Qwen3 block in f32. This is the mode the reference's receipts were banked in
              (tests/integration/test_receipts.py), so it is what pins the oracle to the reference.
``CardPath``  bf16 activations, the card graph's kernel sequence (btb/engine/cuda.py:1722-1834): add_rmsnorm ->
              qkv GEMV -> norm_rope_kv -> attention -> o GEMV -> add_rmsnorm -> gate/up GEMV -> SwiGLU-folded down
              GEMV ... final add_rmsnorm -> head GEMV -> bf16 logits -> lowest-index argmax. This is what the CUDA
              engine is compared with.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import oracle as O


@dataclass
class DenseCfg:
    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    inter: int
    vocab: int
    theta: float = 1e6
    eps: float = 1e-6
    qk_norm: bool = True


def rope_tables_f32(cfg: DenseCfg, n: int) -> tuple[np.ndarray, np.ndarray]:
    """cos/sin [n, D] in f32 as Hugging Face's default rotary makes them: inv_freq = theta^(-2i/D) in f32, the angle
    pos * inv_freq in f32, the halves concatenated"""
    D = cfg.head_dim
    inv = (1.0 / (np.float32(cfg.theta) ** (np.arange(0, D, 2, dtype=np.float32) / np.float32(D)))).astype(np.float32)
    ang = (np.arange(n, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    emb = np.concatenate([ang, ang], axis=-1)
    return np.cos(emb).astype(np.float32), np.sin(emb).astype(np.float32)


def rope_tables_bf16(cfg: DenseCfg, n: int) -> tuple[np.ndarray, np.ndarray]:
    """the card's tables: the f32 tables rounded to bf16 (btb/engine/cuda.py:1166-1182), as bit patterns"""
    c, s = rope_tables_f32(cfg, n)
    return O.f32_to_bits(c), O.f32_to_bits(s)


class Weights:
    """one model's tensors as bf16 bit patterns, by Hugging Face names"""

    def __init__(self, cfg: DenseCfg, tensors: dict[str, np.ndarray]):
        self.cfg = cfg
        self.t = tensors

    def layer(self, i: int, name: str) -> np.ndarray:
        return self.t[f"model.layers.{i}.{name}.weight"]

    def merged_qkv(self, i: int) -> np.ndarray:
        return np.concatenate(
            [self.layer(i, "self_attn.q_proj"), self.layer(i, "self_attn.k_proj"), self.layer(i, "self_attn.v_proj")]
        )

    def merged_gu(self, i: int) -> np.ndarray:
        return np.concatenate([self.layer(i, "mlp.gate_proj"), self.layer(i, "mlp.up_proj")])

    @property
    def embed(self) -> np.ndarray:
        return self.t["model.embed_tokens.weight"]

    @property
    def final_norm(self) -> np.ndarray:
        return self.t["model.norm.weight"]


# --------------------------------------------------------------------------------------------------------------
# the CPU tier (f32 activations)
# --------------------------------------------------------------------------------------------------------------


class CpuTier:
    def __init__(self, w: Weights, cap: int = 512, gemv=None):
        self.w, self.cfg = w, w.cfg
        c = self.cfg
        self.cos, self.sin = rope_tables_f32(c, cap)
        self.K = np.zeros((c.layers, c.kv_heads, cap, c.head_dim), np.float32)
        self.V = np.zeros_like(self.K)
        self.n = 0
        self.gemv = gemv or (lambda wt, x: O.cpu_gemv_bf16(wt, x))

    @staticmethod
    def _rms(x: np.ndarray, w_bits: np.ndarray, eps: float) -> np.ndarray:
        x = x.astype(np.float32)
        var = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32)
        return (O.bits_to_f32(w_bits) * (x * (1.0 / np.sqrt(var + np.float32(eps))).astype(np.float32))).astype(
            np.float32
        )

    def forward(self, ids, positions=None, parents=None) -> np.ndarray:
        """T rows after the cache's n rows; row t at positions[t], seeing the cache and its ancestors (parents, -1
        the root; a chain by default). Rows are written to cache slots n + t. Returns logits [T, V] f32."""
        c = self.cfg
        T = len(ids)
        n0 = self.n
        positions = list(range(n0, n0 + T)) if positions is None else list(positions)
        parents = list(range(-1, T - 1)) if parents is None else list(parents)
        G = c.q_heads // c.kv_heads
        D = c.head_dim
        h = O.bits_to_f32(self.w.embed[np.asarray(ids)]).copy()
        # visibility of pass rows: row t sees pass row u iff u is t or an ancestor of t
        vis = np.zeros((T, T), bool)
        for t in range(T):
            p = t
            while p >= 0:
                vis[t, p] = True
                p = parents[p]
        for i in range(c.layers):
            x = self._rms(h, self.w.layer(i, "input_layernorm"), c.eps)
            q = self.gemv(self.w.layer(i, "self_attn.q_proj"), x).reshape(T, c.q_heads, D)
            k = self.gemv(self.w.layer(i, "self_attn.k_proj"), x).reshape(T, c.kv_heads, D)
            v = self.gemv(self.w.layer(i, "self_attn.v_proj"), x).reshape(T, c.kv_heads, D)
            if c.qk_norm:
                q = self._rms(q, self.w.layer(i, "self_attn.q_norm"), c.eps)
                k = self._rms(k, self.w.layer(i, "self_attn.k_norm"), c.eps)
            cos, sin = self.cos[positions][:, None, :], self.sin[positions][:, None, :]

            def rot(a):
                return np.concatenate([-a[..., D // 2 :], a[..., : D // 2]], axis=-1)

            q = (q * cos + rot(q) * sin).astype(np.float32)
            k = (k * cos + rot(k) * sin).astype(np.float32)
            self.K[i, :, n0 : n0 + T] = k.transpose(1, 0, 2)
            self.V[i, :, n0 : n0 + T] = v.transpose(1, 0, 2)
            att = np.zeros((T, c.q_heads, D), np.float32)
            scale = np.float32(D**-0.5)
            for t in range(T):
                keep = np.concatenate([np.ones(n0, bool), vis[t]])
                for hq in range(c.q_heads):
                    g = hq // G
                    kk = self.K[i, g, : n0 + T][keep]
                    vv = self.V[i, g, : n0 + T][keep]
                    s = (kk @ q[t, hq]).astype(np.float32) * scale
                    p = np.exp(s - s.max()).astype(np.float32)
                    att[t, hq] = (p @ vv) / p.sum(dtype=np.float32)
            y = self.gemv(self.w.layer(i, "self_attn.o_proj"), att.reshape(T, -1))
            h = (h + y).astype(np.float32)
            x = self._rms(h, self.w.layer(i, "post_attention_layernorm"), c.eps)
            gt = self.gemv(self.w.layer(i, "mlp.gate_proj"), x)
            up = self.gemv(self.w.layer(i, "mlp.up_proj"), x)
            act = (gt / (1.0 + np.exp(-gt, dtype=np.float32))).astype(np.float32)
            y = self.gemv(self.w.layer(i, "mlp.down_proj"), (act * up).astype(np.float32))
            h = (h + y).astype(np.float32)
        self.n = n0 + T
        x = self._rms(h, self.w.final_norm, c.eps)
        return self.gemv(self.w.embed, x)

    def keep_path(self, base: int, path) -> None:
        """the accepted branch's rows gathered to the cache's front (btb/engine/cuda.py:3563-3575)"""
        for j, node in enumerate(path):
            self.K[:, :, base + j] = self.K[:, :, base + node].copy()
            self.V[:, :, base + j] = self.V[:, :, base + node].copy()
        self.n = base + len(path)


# --------------------------------------------------------------------------------------------------------------
# the card path (bf16 activations, the card graph's kernel order)
# --------------------------------------------------------------------------------------------------------------


class CardPath:
    """KV position-major [cap, Hk, D] (hs = D, rs = Hk * D), btb/engine/arena.py:1-5"""

    def __init__(self, w: Weights, cap: int = 512, silu_fold: bool = True, tables=None):
        self.w, self.cfg = w, w.cfg
        c = self.cfg
        self.cap = cap
        # `tables`: the engine's own bf16 cos/sin bit patterns, so both sides read the same table
        self.cos, self.sin = rope_tables_bf16(c, cap) if tables is None else tables
        self.K = np.zeros((c.layers, cap, c.kv_heads, c.head_dim), np.uint16)
        self.V = np.zeros_like(self.K)
        self.n = 0
        self.qkv = [w.merged_qkv(i) for i in range(c.layers)]
        self.gu = [w.merged_gu(i) for i in range(c.layers)]
        self.silu_fold = silu_fold

    def forward(self, ids, depth=None, parents=None) -> np.ndarray:
        """one pass of T rows; returns the bf16 logits' bit patterns [T, V]"""
        c = self.cfg
        T = len(ids)
        n0 = self.n
        depth = np.arange(T, dtype=np.int32) if depth is None else np.asarray(depth, np.int32)
        par = np.arange(-1, T - 1, dtype=np.int32) if parents is None else np.asarray(parents, np.int32)
        D, Hq, Hk = c.head_dim, c.q_heads, c.kv_heads
        hs, rs = D, Hk * D
        h = self.w.embed[np.asarray(ids)].copy()
        y_prev = None
        for i in range(c.layers):
            h, x = O.add_rmsnorm(h, y_prev, self.w.layer(i, "input_layernorm"), c.eps)
            qkv = O.gemv_card_bf16(self.qkv[i], x)
            wq = self.w.layer(i, "self_attn.q_norm") if c.qk_norm else None
            wk = self.w.layer(i, "self_attn.k_norm") if c.qk_norm else None
            q = O.norm_rope_kv(qkv, wq, wk, c.eps, self.cos, self.sin, n0, depth, self.K[i], self.V[i], Hq, Hk, D, hs, rs)
            att = O.attn_decode(q, self.K[i], self.V[i], n0, par, Hq, Hk, D, hs, rs, float(D**-0.5))
            y = O.gemv_card_bf16(self.w.layer(i, "self_attn.o_proj"), att)
            h, x = O.add_rmsnorm(h, y, self.w.layer(i, "post_attention_layernorm"), c.eps)
            gu = O.gemv_card_bf16(self.gu[i], x)
            if self.silu_fold:
                y_prev = O.gemv_card_silu_bf16(self.w.layer(i, "mlp.down_proj"), gu)
            else:
                y_prev = O.gemv_card_bf16(self.w.layer(i, "mlp.down_proj"), O.silu_mul(gu))
        h, x = O.add_rmsnorm(h, y_prev, self.w.final_norm, c.eps)
        self.n = n0 + T
        return O.gemv_card_bf16(self.w.embed, x)

    def greedy(self, prompt, n_new: int) -> list[int]:
        """prefill as chain passes of up to 32 rows through the step's own arithmetic, then one row a step"""
        lg = None
        for a in range(0, len(prompt), 32):
            lg = self.forward(prompt[a : a + 32])
        toks = [int(O.argmax_bf16(lg[-1:])[0])]
        while len(toks) < n_new:
            lg = self.forward([toks[-1]])
            toks.append(int(O.argmax_bf16(lg)[0]))
        return toks


# --------------------------------------------------------------------------------------------------------------
# the MoE decoder: the card path's attention, the host's router and experts (btb/engine/host.py:175-191, 508-569)
# --------------------------------------------------------------------------------------------------------------


@dataclass
class MoECfg(DenseCfg):
    experts: int = 8
    top_k: int = 2
    router_mode: int = 0
    glu_kind: int = 0
    expert_fmt: str = "mx4"
    alpha: float = 1.702
    limit: float = 7.0


class MoECardPath:
    """layers: dicts with ln1, ln2, qkv, o, router (bf16 bits), wq, wk (or None), gu / dn: (fmt, w, scales) stacked
    over ALL experts as stored. embed, norm: bf16 bits."""

    def __init__(self, cfg: MoECfg, embed, norm, layers, cap: int = 512, tables=None):
        self.cfg, self.embed, self.norm, self.layers = cfg, embed, norm, layers
        self.cos, self.sin = rope_tables_bf16(cfg, cap) if tables is None else tables
        self.K = np.zeros((cfg.layers, cap, cfg.kv_heads, cfg.head_dim), np.uint16)
        self.V = np.zeros_like(self.K)
        self.n = 0

    @staticmethod
    def expert_gemv(stack, e: int, x: np.ndarray) -> np.ndarray:
        fmt, w, sc = stack
        if fmt == "mx4":
            R, G = w.shape[1], w.shape[2]
            return O.cpu_gemv_mxfp4(w[e], sc[e], R, G * 32, x)
        if fmt == "fp8":
            R, C_ = w.shape[1], w.shape[2]
            return O.cpu_gemv_fp8(w[e], sc[e], R, C_, x)
        return O.cpu_gemv_bf16(w[e], x)

    def moe_block(self, L, x_bits: np.ndarray) -> np.ndarray:
        c = self.cfg
        xf = O.bits_to_f32(x_bits)
        logits = O.cpu_gemv_bf16(L["router"], xf)
        idx, w = O.moe_route(logits, c.experts, c.top_k, c.router_mode)
        T = xf.shape[0]
        dn = np.zeros((T, c.top_k, c.hidden), np.float32)
        for t in range(T):
            for s in range(c.top_k):
                e = int(idx[t, s])
                gu = self.expert_gemv(L["gu"], e, xf[t : t + 1])
                hmid = O.moe_act(gu, c.glu_kind, None, c.alpha, c.limit)
                dn[t, s] = self.expert_gemv(L["dn"], e, hmid)[0]
        return O.moe_combine(dn, idx, w)

    def forward(self, ids, depth=None, parents=None) -> np.ndarray:
        c = self.cfg
        T, n0 = len(ids), self.n
        depth = np.arange(T, dtype=np.int32) if depth is None else np.asarray(depth, np.int32)
        par = np.arange(-1, T - 1, dtype=np.int32) if parents is None else np.asarray(parents, np.int32)
        D, Hq, Hk = c.head_dim, c.q_heads, c.kv_heads
        hs, rs = D, Hk * D
        h = self.embed[np.asarray(ids)].copy()
        y_prev = None
        for i, L in enumerate(self.layers):
            h, x = O.add_rmsnorm(h, y_prev, L["ln1"], c.eps)
            qkv = O.gemv_card_bf16(L["qkv"], x)
            q = O.norm_rope_kv(qkv, L.get("wq"), L.get("wk"), c.eps, self.cos, self.sin, n0, depth, self.K[i], self.V[i],
                               Hq, Hk, D, hs, rs)
            att = O.attn_decode(q, self.K[i], self.V[i], n0, par, Hq, Hk, D, hs, rs, float(D**-0.5))
            y = O.gemv_card_bf16(L["o"], att)
            h, x = O.add_rmsnorm(h, y, L["ln2"], c.eps)
            y_prev = self.moe_block(L, x)
        h, x = O.add_rmsnorm(h, y_prev, self.norm, c.eps)
        self.n = n0 + T
        return O.gemv_card_bf16(self.embed, x)

    def greedy(self, prompt, n_new: int) -> list[int]:
        lg = None
        for a in range(0, len(prompt), 32):
            lg = self.forward(prompt[a : a + 32])
        toks = [int(O.argmax_bf16(lg[-1:])[0])]
        while len(toks) < n_new:
            lg = self.forward([toks[-1]])
            toks.append(int(O.argmax_bf16(lg)[0]))
        return toks


# --------------------------------------------------------------------------------------------------------------
# gpt-oss in f32: what the reference's banked receipts for its tiny gpt-oss fixture were computed with
# (tests/make_fixtures.py:1331-1366 `bank_gpt_oss`: transformers' GptOssForCausalLM in float32, eager attention,
# experts dequantized from the stored MXFP4). The pieces are the oracle's own: the 16-lane GEMVs over the weights as
# stored (native/src/gemv.rs:46-58, 1038-1119), the router's top-k then softmax (btb/engine/host.py:187-191), the
# clamped GLU over interleaved lanes (host.py:444-450) and the sum in ascending expert id (host.py:565-569) - here
# without the row dtype's roundings, since the receipts' activations are f32.
# --------------------------------------------------------------------------------------------------------------


class GptOssF32:
    def __init__(self, cfg: dict, w: dict, cap: int = 128):
        self.c, self.w = cfg, w
        self.L, self.H, self.D = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["head_dim"]
        self.Hq, self.Hk = cfg["num_attention_heads"], cfg["num_key_value_heads"]
        self.E, self.k = cfg["num_local_experts"], cfg["num_experts_per_tok"]
        self.eps, self.win = np.float32(cfg["rms_norm_eps"]), int(cfg["sliding_window"])
        self.limit, self.alpha = np.float32(cfg.get("swiglu_limit", 7.0)), np.float32(1.702)
        self.inv_freq, self.att_scale = self._yarn(cfg)
        self.K = np.zeros((self.L, cap, self.Hk, self.D), np.float32)
        self.V = np.zeros_like(self.K)
        self.n = 0

    @classmethod
    def from_fixture(cls, npz) -> "GptOssF32":
        import json

        cfg = json.loads(npz["config"].tobytes())
        return cls(cfg, {k[2:]: npz[k] for k in npz.files if k.startswith("w/")})

    @staticmethod
    def _yarn(cfg: dict):
        """the YaRN inverse frequencies and the attention factor applied to cos and sin (transformers'
        `_compute_yarn_parameters`: interpolated and extrapolated frequencies blended by a linear ramp between the
        dimensions that make beta_fast and beta_slow rotations over the original context)"""
        import math

        rs = cfg["rope_scaling"]
        base, dim, factor = float(cfg["rope_theta"]), int(cfg["head_dim"]), float(rs["factor"])
        orig = int(rs["original_max_position_embeddings"])

        def corr(rot: float) -> float:
            return (dim * math.log(orig / (rot * 2 * math.pi))) / (2 * math.log(base))

        low, high = corr(float(rs["beta_fast"])), corr(float(rs["beta_slow"]))
        if rs.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, dim - 1)
        if low == high:
            high += 0.001
        ramp = np.clip((np.arange(dim // 2, dtype=np.float32) - np.float32(low)) / np.float32(high - low), 0, 1)
        pos_freqs = np.float32(base) ** (np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim))
        extra, inter = np.float32(1) / pos_freqs, np.float32(1) / (np.float32(factor) * pos_freqs)
        keep = (np.float32(1) - ramp).astype(np.float32)
        inv = (inter * (np.float32(1) - keep) + extra * keep).astype(np.float32)
        return inv, np.float32(0.1 * math.log(factor) + 1.0)

    def _lin(self, name: str, x: np.ndarray) -> np.ndarray:
        y = O.cpu_gemv_bf16(self.w[name + ".weight"], np.ascontiguousarray(x, np.float32))
        b = self.w.get(name + ".bias")
        return y if b is None else (y + O.bits_to_f32(b)[None, :]).astype(np.float32)

    def _norm(self, name: str, h: np.ndarray) -> np.ndarray:
        var = np.mean(h * h, axis=-1, keepdims=True, dtype=np.float32)
        return (O.bits_to_f32(self.w[name + ".weight"])[None, :] * (h * (np.float32(1) / np.sqrt(var + self.eps)))).astype(np.float32)

    def _rope(self, x: np.ndarray, pos: np.ndarray) -> np.ndarray:
        ang = pos[:, None].astype(np.float32) * self.inv_freq[None, :]
        cos, sin = (np.cos(ang) * self.att_scale)[:, None, :], (np.sin(ang) * self.att_scale)[:, None, :]
        a, b = x[..., : self.D // 2], x[..., self.D // 2 :]
        return np.concatenate([a * cos - b * sin, b * cos + a * sin], -1).astype(np.float32)

    def _experts(self, p: str, x: np.ndarray) -> np.ndarray:
        T = x.shape[0]
        logits = self._lin(p + "router", x)
        idx, _w = O.moe_route(logits, self.E, self.k, 1)  # the picks: top-k by value, lower index first among equals
        out = np.zeros((T, self.H), np.float32)
        gb, gs = self.w[p + "experts.gate_up_proj_blocks"], self.w[p + "experts.gate_up_proj_scales"]
        db, ds = self.w[p + "experts.down_proj_blocks"], self.w[p + "experts.down_proj_scales"]
        gbias, dbias = O.bits_to_f32(self.w[p + "experts.gate_up_proj_bias"]), O.bits_to_f32(self.w[p + "experts.down_proj_bias"])
        for t in range(T):
            top = logits[t, idx[t]]
            ex = np.exp(top - top.max(), dtype=np.float32)
            wts = ex / ex.sum(dtype=np.float32)
            for s in np.argsort(idx[t], kind="stable"):  # ascending expert id
                e = int(idx[t, s])
                gu = O.cpu_gemv_mxfp4(gb[e], gs[e], gb.shape[1], gb.shape[2] * 32, x[t : t + 1])[0] + gbias[e]
                g, u = np.minimum(gu[0::2], self.limit), np.clip(gu[1::2], -self.limit, self.limit)
                hmid = ((u + np.float32(1)) * (g * (np.float32(1) / (np.float32(1) + np.exp(-g * self.alpha, dtype=np.float32))))).astype(np.float32)
                y = O.cpu_gemv_mxfp4(db[e], ds[e], db.shape[1], db.shape[2] * 32, hmid[None, :])[0] + dbias[e]
                out[t] += (y * wts[s]).astype(np.float32)
        return out

    def forward(self, ids) -> np.ndarray:
        """a chain of rows after the cache's; f32 logits [T, V]"""
        T, n0 = len(ids), self.n
        pos = np.arange(n0, n0 + T)
        G = self.Hq // self.Hk
        h = O.bits_to_f32(self.w["model.embed_tokens.weight"][np.asarray(ids)])
        sliding = [t == "sliding_attention" for t in self.c["layer_types"]]
        for i in range(self.L):
            p = f"model.layers.{i}."
            x = self._norm(p + "input_layernorm", h)
            q = self._rope(self._lin(p + "self_attn.q_proj", x).reshape(T, self.Hq, self.D), pos)
            k = self._rope(self._lin(p + "self_attn.k_proj", x).reshape(T, self.Hk, self.D), pos)
            v = self._lin(p + "self_attn.v_proj", x).reshape(T, self.Hk, self.D)
            self.K[i, n0 : n0 + T], self.V[i, n0 : n0 + T] = k, v
            sinks = O.bits_to_f32(self.w[p + "self_attn.sinks"])
            att = np.zeros((T, self.Hq, self.D), np.float32)
            for t in range(T):
                last = n0 + t
                first = max(0, last + 1 - self.win) if sliding[i] else 0
                for hq in range(self.Hq):
                    kk, vv = self.K[i, first : last + 1, hq // G], self.V[i, first : last + 1, hq // G]
                    s = np.append((kk @ q[t, hq]) * np.float32(self.D**-0.5), sinks[hq]).astype(np.float32)
                    pr = np.exp(s - s.max(), dtype=np.float32)
                    pr = pr / pr.sum(dtype=np.float32)
                    att[t, hq] = pr[:-1] @ vv  # the sink takes its share of the mass and contributes no value
            h = h + self._lin(p + "self_attn.o_proj", att.reshape(T, -1))
            x = self._norm(p + "post_attention_layernorm", h)
            h = h + self._experts(p + "mlp.", x)
        self.n = n0 + T
        return self._lin("lm_head", self._norm("model.norm", h))

    def greedy(self, prompt, n_new: int) -> list[int]:
        lg = self.forward(list(prompt))
        toks = [int(np.argmax(lg[-1]))]
        while len(toks) < n_new:
            toks.append(int(np.argmax(self.forward([toks[-1]])[-1])))
        return toks
