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


@pytest.mark.parametrize("which,lens", [
    ("ragged", [19, 16, 5, 33]),                      # ragged chunks, a quarter chunk, shorter than a token group, half a chunk + 1
    ("ragged", [64, 129, 70, 3]),                     # one exact chunk, two chunks + 1, a chunk and a bit
    ("gqa4", [200, 61, 130, 257, 9]),                 # head_dim 128 in groups of 4: several key tiles and runs per sequence
    ("wide", [150, 66]),
])
def test_prefill_into_slots_then_batched_decode(which, lens, ragged_file, gqa4_file, wide_file):
    """Every sequence of a batch gets its own prompt through the chunked prefill into its own KV slot, then all slots
    decode together; tokens must equal the checker's greedy continuation of each prompt on its own."""
    path = dict(ragged=ragged_file, gqa4=gqa4_file, wide=wide_file)[which]
    nseq, G = len(lens), 6
    cap = max(lens) + 16
    om = ol.OracleModel(path, kv_cap=cap)
    rng = np.random.default_rng(77)
    prompts = [rng.integers(0, om.NV, n).astype(np.int32) for n in lens]
    want = [om.generate(p, G + 1) for p in prompts]
    gm = hb.Model.load(path, kv_cap=cap, batch=nseq)
    first = np.array([gm.prefill_seq(s, prompts[s]) for s in range(nseq)], np.int32)
    assert list(first) == [int(w[0]) for w in want]
    toks, pos = first.copy(), np.array(lens, np.int32)
    for g in range(G):                                # ragged positions: each sequence continues at its own length
        toks = gm.decode_batch(toks, pos)
        assert list(toks) == [int(w[g + 1]) for w in want], g
        pos += 1
    gm.close(); om.close()
