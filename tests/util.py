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
