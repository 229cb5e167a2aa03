"""The oracle's sampled pick pinned: its keys and uniforms against values banked from the reference's Python
(tests/golden/sampling.npz), its exp against libm, its kept sets against the sort-based definition of the masks
(btb/sampling.py:96-109) and the known answers of the reference's own unit tests (native/src/sample.rs:515-567)."""

import os

import numpy as np

from oracle import oracle as O

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampling.npz"))


def test_keys_and_uniforms_are_the_reference_values():
    for a, seed in enumerate(G["key_seeds"]):
        for b, pos in enumerate(G["key_pos"]):
            assert O.sample_key(int(seed), int(pos)) == int(G["keys"][a][b])
            assert O.sample_key(int(seed), int(pos), 3) == int(G["keys_salt3"][a][b])
    u = O.sample_uniform(int(G["uniform_key"][0]), range(4096))
    assert np.array_equal(u.view(np.uint32), G["uniform"].astype(np.float32).view(np.uint32))
    assert 0.0 < u.min() and u.max() < 1.0


def test_exp_holds_to_a_few_ulps():
    t = -np.arange(2000, dtype=np.float32) * np.float32(0.04)
    a, b = O.sample_exp(t).astype(np.float64), np.exp(t.astype(np.float64))
    assert np.all(np.abs(a - b) <= 4e-7 * np.maximum(b, 1e-30) + 1e-38)
    assert O.sample_exp([-88.0])[0] == 0.0


def test_masks_keep_the_right_tokens_and_a_key_repeats():
    # probabilities halving from 0.5: top-p 0.8 keeps three, top-k 2 keeps two
    x = np.log(np.float32(0.5) / np.float32(2.0) ** np.arange(8, dtype=np.float32))[None]
    keys = np.arange(400, dtype=np.uint64)
    xs = np.repeat(x, 400, 0)
    tp, _, _ = O.sample_pick(xs, keys, 1.0, 0, 0.8)
    tk, _, _ = O.sample_pick(xs, keys, 1.0, 2, 1.0)
    assert set(tp.tolist()) == {0, 1, 2} and set(tk.tolist()) == {0, 1}
    assert np.array_equal(tp, O.sample_pick(xs, keys, 1.0, 0, 0.8)[0])


def test_draws_follow_the_distribution():
    p = np.asarray([0.5, 0.3, 0.15, 0.05], np.float32)
    n = 20000
    tok, _, _ = O.sample_pick(np.repeat(np.log(p)[None], n, 0), np.arange(n, dtype=np.uint64), 1.0)
    f = np.bincount(tok, minlength=4) / n
    assert np.all(np.abs(f - p) < 0.02)


def _kept_by_sorting(x, temperature, top_k, top_p):
    """the masks as btb/sampling.py:96-109 states them, in float64"""
    s = x.astype(np.float64) / temperature
    keep = np.ones_like(s, bool)
    if top_k > 0:
        keep &= s >= np.sort(s)[::-1][min(top_k, s.size) - 1]
    if top_p < 1.0:
        z = np.where(keep, np.exp(s - s.max()), 0.0)
        order = np.argsort(-s, kind="stable")
        pr = z[order] / z.sum()
        drop = np.cumsum(pr) - pr >= top_p
        drop[0] = False
        k2 = np.zeros_like(keep)
        k2[order[~drop]] = True
        keep &= k2
    return keep


def test_thresholds_agree_with_the_sorted_definition():
    rng = np.random.default_rng(0)
    for V, T, k, p in ((1000, 0.8, 40, 0.9), (5000, 1.0, 0, 0.7), (257, 1.5, 3, 0.5), (70, 0.3, 0, 0.99),
                       (3001, 0.7, 50, 1.0), (9, 1.0, 20, 1.0)):  # fmt: skip
        x = (rng.standard_normal((4, V)) * 3).astype(np.float32)
        _, floors, _ = O.sample_pick(x, np.arange(4, dtype=np.uint64), T, k, p)
        for r in range(4):
            s = x[r] * (np.float32(1.0) / np.float32(T))
            u = s.view(np.uint32)
            o = np.where(u & 0x80000000, ~u, u | 0x80000000)
            got = o >= floors[r].max()
            want = _kept_by_sorting(x[r], T, k, p)
            # the fixed-point masses and the f32 target can move the nucleus' edge by a token
            assert abs(int(got.sum()) - int(want.sum())) <= 1 and (got & want).sum() >= min(got.sum(), want.sum())
            if p >= 1.0:
                assert np.array_equal(got, want)


def test_picked_token_is_kept_and_rows_pick_alike_alone_and_together():
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((16, 3000)) * 2).astype(np.float32)
    keys = np.arange(16, dtype=np.uint64)
    together, floors, _ = O.sample_pick(x, keys, 0.8, 40, 0.9)
    for r in range(16):
        alone, _, _ = O.sample_pick(x[r : r + 1], keys[r : r + 1], 0.8, 40, 0.9)
        assert alone[0] == together[r]
        s = x[r, together[r]] * (np.float32(1.0) / np.float32(0.8))
        u = np.float32(s).view(np.uint32)
        o = ~u if u & 0x80000000 else u | 0x80000000
        assert o >= floors[r].max()
