"""The host-side n-gram drafter of the speculative decoder (hx_pld_draft) against the CPU restatement of the
reference's pld_draft (gpt2_infer.c:2972-2994), and the token-level replay of its accept rule."""
import numpy as np

import helix_b200 as hb
import oracle_lib as ol


def test_drafter_known_cases():
    # longest suffix first, most recent occurrence first, continuation capped by m and by the end of the sequence
    assert list(hb.pld_draft([1, 2, 3, 4, 1, 2, 3])) == [4, 1, 2, 3]
    assert list(hb.pld_draft([1, 2, 3, 4, 1, 2, 3], m=2)) == [4, 1]
    assert list(hb.pld_draft([5, 6, 7])) == []                       # nothing repeats
    assert list(hb.pld_draft([7])) == []                             # shorter than k_min + 1
    assert list(hb.pld_draft([9, 9, 9, 9])) == [9]                   # the match may overlap the suffix, not start in it
    assert list(hb.pld_draft([1, 2, 1, 2, 1, 2], m=3)) == [1, 2]
    # k = 3 has no match, k = 2 has: [8, 3] occurs at 1 -> continuation 4, 5, ...
    assert list(hb.pld_draft([0, 8, 3, 4, 5, 6, 8, 3], k_max=3)) == [4, 5, 6, 8, 3]
    # the most recent occurrence wins over an earlier, longer continuation
    assert list(hb.pld_draft([4, 1, 7, 7, 4, 1, 5, 4, 1], k_max=2, m=3)) == [5, 4, 1]


def test_drafter_matches_restatement_on_random_sequences():
    rng = np.random.default_rng(17)
    for trial in range(400):
        T = int(rng.integers(1, 60))
        ids = rng.integers(0, int(rng.integers(2, 9)), T).astype(np.int32)
        k_min = int(rng.integers(1, 3)); k_max = k_min + int(rng.integers(0, 4)); m = int(rng.integers(1, 20))
        got = hb.pld_draft(ids, k_min, k_max, m)
        want = ol.pld_draft(ids, k_min, k_max, m)
        assert list(got) == list(want), (ids, k_min, k_max, m)
        assert len(got) <= min(m, 16)


def test_spec_counters_replay():
    # a continuation that repeats the prompt: every draft is right, so few forwards produce many tokens
    prompt = np.array([3, 1, 4, 1, 5, 9, 2, 6], np.int32)
    greedy = np.array(list(prompt) * 3, np.int32)
    st = ol.spec_counters(prompt, greedy, k_min=1, k_max=3, m=6)
    assert st["emitted"] + (st["steps"] - st["forwards"]) + 1 == len(greedy)      # verify tokens + single steps + prefill token
    assert st["accepted"] > 0 and st["forwards"] < len(greedy) // 2
    # a continuation that never follows a draft: every hit costs a forward and yields exactly one token
    greedy2 = np.arange(100, 124, dtype=np.int32)
    st2 = ol.spec_counters(np.array([1, 2, 1, 2, 1], np.int32), greedy2)
    assert st2["accepted"] == 0 and st2["emitted"] == st2["forwards"]
