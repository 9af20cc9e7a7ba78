"""Batched decode of independent sequences (chunks of 64 through the tcgen05 GEMM) against the CPU restatement run one
sequence at a time."""
import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("which,nseq", [("tiny", 20), ("ragged", 5), ("wide", 16), ("tiny", 70), ("wide", 40)])
def test_batched_decode_matches_single_sequence_checker(which, nseq, tiny_file, ragged_file, wide_file):
    path = dict(tiny=tiny_file, ragged=ragged_file, wide=wide_file)[which]
    T, G = 9, 7                                       # teacher-forced prompt positions, then free-running steps
    om = ol.OracleModel(path, kv_cap=32)
    rng = np.random.default_rng(40 + nseq)
    prompts = rng.integers(0, om.NV, (nseq, T)).astype(np.int32)
    want = np.stack([om.generate(prompts[i], G + 1) for i in range(nseq)])     # [nseq][G+1]

    gm = hb.Model.load(path, kv_cap=32, batch=nseq)
    nxt = None
    for p in range(T):                                # every sequence at the same position, different tokens
        nxt = gm.decode_batch(prompts[:, p], np.full(nseq, p))
    assert np.array_equal(nxt, want[:, 0])
    out, ms = gm.decode_batch_loop(nxt, T, G)         # feeds the arg-max back on the device
    assert np.array_equal(out.T, want[:, 1:])
    # ragged positions: sequence i restarts at its own position with its own token
    pos = np.array([T + G - 1 - (i % 3) for i in range(nseq)], np.int32)
    ids = np.array([(want[i, G - 1 - (i % 3)]) for i in range(nseq)], np.int32)
    again = gm.decode_batch(ids, pos)
    assert np.array_equal(again, np.array([want[i, G - (i % 3)] for i in range(nseq)]))
    gm.close(); om.close()


def test_prefill_into_slots_then_batched_decode(ragged_file):
    """Every sequence of a batch gets its own prompt through the chunked prefill into its own KV slot, then all slots
    decode together; tokens must equal the checker's greedy continuation of each prompt on its own."""
    nseq, G = 4, 6
    om = ol.OracleModel(ragged_file, kv_cap=64)
    rng = np.random.default_rng(77)
    lens = [19, 16, 5, 33]                            # ragged chunks, one exact chunk, shorter than a chunk, two chunks + 1
    prompts = [rng.integers(0, om.NV, n).astype(np.int32) for n in lens]
    want = [om.generate(p, G + 1) for p in prompts]
    gm = hb.Model.load(ragged_file, kv_cap=64, batch=nseq)
    first = np.array([gm.prefill_seq(s, prompts[s]) for s in range(nseq)], np.int32)
    assert list(first) == [int(w[0]) for w in want]
    toks, pos = first.copy(), np.array(lens, np.int32)
    for g in range(G):                                # ragged positions: each sequence continues at its own length
        toks = gm.decode_batch(toks, pos)
        assert list(toks) == [int(w[g + 1]) for w in want], g
        pos += 1
    gm.close(); om.close()
