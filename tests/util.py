"""Shared by the model-level GPU tests: how small test models are drawn, and a guard against degenerate sequences."""

# Layers' linears of the small test models are drawn at this deviation (the embedding keeps 0.02). At 0.02 a
# hidden-256 model of two or three layers falls into a fixed point and greedy decoding repeats one token, and a token
# comparison then cannot see an off-by-one cache row or a wrong commit.
LAYER_STD = 0.1


def lively(tokens, what: str = "greedy sequence") -> None:
    """the expected sequence must hold many distinct tokens, or comparing against it proves nothing"""
    toks = list(tokens)
    need = min(8, max(2, len(toks) // 3))
    assert len(set(toks)) >= need, f"{what} is degenerate: {len(set(toks))} distinct tokens in {len(toks)}: {toks}"


def oracle_trace(orc, prompt, n_new: int):
    """the oracle's greedy decode with every step's logits kept: (tokens, [f32 logits row of each pick])"""
    import numpy as np

    from oracle import oracle as O

    lg = None
    for a in range(0, len(prompt), 32):
        lg = orc.forward(list(prompt[a : a + 32]))
    rows = [O.bits_to_f32(lg[-1])]
    toks = [int(O.argmax_bf16(lg[-1:])[0])]
    while len(toks) < n_new:
        lg = orc.forward([toks[-1]])
        rows.append(O.bits_to_f32(lg[-1]))
        toks.append(int(O.argmax_bf16(lg)[0]))
    return toks, [np.asarray(r, np.float32) for r in rows]


def same_tokens_or_near_tie(got, want, rows, min_equal: int = 4) -> None:
    """the card's tokens are the oracle's - or part at a pick the oracle itself calls a near tie. The card computes expf,
    rsqrtf and the attention's dot products in another order than the CPU oracle (the logit tests bound that at 2^-6 of
    the row's largest logit), so where the oracle's two best logits sit inside that bound the argmax may go either way;
    from there on the sequences differ legitimately. A wrong cache row or commit shows up as a pick the oracle does NOT
    call close, or before `min_equal` tokens have matched."""
    got, want = list(got), list(want)
    for i, (g, w) in enumerate(zip(got, want)):
        if g == w:
            continue
        row = rows[i]
        tol = 2.0**-6 * max(1.0, float(abs(row).max()))
        assert i >= min_equal, f"tokens part at pick {i}: {got} != {want}"
        assert float(row[w] - row[g]) <= tol, f"pick {i}: the oracle prefers {w} over {g} by {float(row[w] - row[g])} > {tol}"
        return
    assert len(got) == len(want)
