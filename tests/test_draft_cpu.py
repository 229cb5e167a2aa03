"""The library's native n-gram index, chain merge and accept walk (host code behind the C-ABI) against fixtures made by
the reference's own code (tests/golden/make_golden.py: btb/draft.py NGramProposer, btb/engine/generate.py _chains_tree)."""

import json
import os

from btb_b200.draft import NGramProposer, chains_tree, walk

HERE = os.path.dirname(os.path.abspath(__file__))


def test_proposer_and_tree_match_reference():
    cases = json.load(open(os.path.join(HERE, "golden", "drafts.json")))["cases"]
    n = 0
    for case in cases:
        prop = NGramProposer(case["head"], **case["kw"])
        steps = iter(case["steps"])
        cur = next(steps)
        for i, t in enumerate(case["tail"]):
            prop.extend(t)
            while cur is not None and cur["at"] == i:
                chains = prop.propose_chains(cur["v"])
                assert [[c, tag] for c, tag in chains] == cur["chains"]
                g, par, dep, ch = chains_tree(chains, cur["budget"])
                assert (g, par, dep) == (cur["guesses"], cur["parents"], cur["depth"])
                assert {str(k): v for k, v in ch.items()} == cur["children"]
                assert len(g) <= cur["budget"]
                assert prop.tree(cur["v"], cur["budget"]) == (g, par, dep)  # the one-call form
                n += 1
                cur = next(steps, None)
    assert n > 100


def test_tree_is_parents_first_and_walk_follows_picks():
    chains = [([5, 6, 7], "a"), ([5, 6, 8], "b"), ([9], "c"), ([5, 6], "d")]
    g, par, dep, ch = chains_tree(chains, 8)
    assert g == [5, 6, 7, 8, 9] and par == [-1, 0, 1, 2, 2, 0] and dep == [0, 1, 2, 3, 3, 1]
    assert all(p < j for j, p in enumerate(par))
    # node picks: root says 5, node1 says 6, node2 says 8 -> path through the second chain; its leaf's pick ends it
    picks = [5, 6, 8, 0, 1, 0]
    assert walk(picks, g, ch) == [0, 1, 2, 4]
    assert walk([4, 0, 0, 0, 0, 0], g, ch) == [0]
    assert walk([9, 0, 0, 0, 0, 3], g, ch) == [0, 5]
    assert chains_tree(chains, 2)[0] == [5, 6]
    assert chains_tree([], 8) == ([], [-1], [0], {})


def test_host_sampling_keys_are_the_reference_keys():
    """btb_b200.sampling.Sampling.key_for against key_for() values banked from the reference (sampling.npz)"""
    import numpy as np

    from btb_b200.sampling import Sampling

    g = np.load(os.path.join(HERE, "golden", "sampling.npz"))
    for a, seed in enumerate(g["key_seeds"]):
        for b, pos in enumerate(g["key_pos"]):
            s = Sampling(temperature=1.0, seed=int(seed))
            assert s.key_for(int(pos)) == int(g["keys"][a][b])
            assert s.key_for(int(pos), 3) == int(g["keys_salt3"][a][b])
    assert Sampling().greedy and not Sampling(temperature=0.7).greedy
    assert Sampling(temperature=1.0, top_k=5).masked and Sampling(temperature=1.0, top_p=0.9).masked
    import pytest

    with pytest.raises(ValueError):
        Sampling(temperature=-1.0)
    with pytest.raises(ValueError):
        Sampling(temperature=1.0, top_p=1.5)
