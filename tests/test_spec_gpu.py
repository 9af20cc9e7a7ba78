"""Prompt-lookup speculative decode (hx_generate_spec) on the GPU: the tokens must be the plain greedy sequence --
the reference's gate for its HX_SPEC path (gpt2_infer.c:2965-2967) -- and the counters must be those of the
reference's accept rule replayed on that sequence (oracle_lib.spec_counters restates spec_step, :3076-3118)."""
import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol
from conftest import TINY, WIDE, RAGGED, make_model_file

pytestmark = pytest.mark.gpu

CASES = {"tiny": (TINY, 3), "wide": (WIDE, 12), "ragged": (RAGGED, 11),
         "d512-dh128": (dict(NL=3, DM=512, NH=4, NKV=1, DH=128, DFF=768, NV=2011), 41)}
N_NEW = 64


def periodic_prompt(vocab, seed):
    base = np.random.default_rng(seed).integers(0, vocab, 5).astype(np.int32)
    return np.concatenate([base, base, base[:3]]).astype(np.int32)


@pytest.fixture(scope="module", params=sorted(CASES))
def model(request, tmp_path_factory):
    cfg, seed = CASES[request.param]
    path = make_model_file(tmp_path_factory, cfg, seed, "spec_" + request.param)
    gm = hb.Model.load(path, kv_cap=128)
    om = ol.OracleModel(path, kv_cap=128)
    yield request.param, cfg, gm, om
    gm.close(); om.close()


@pytest.mark.parametrize("pseed", [5, 6])
def test_spec_tokens_are_the_greedy_tokens(model, pseed):
    name, cfg, gm, om = model
    prompt = periodic_prompt(cfg["NV"], pseed)
    plain, _, _ = gm.generate(prompt, N_NEW)
    want = om.generate(prompt, N_NEW)
    assert list(plain) == list(want)
    gm.reset()
    spec, st, _, _ = gm.generate_spec(prompt, N_NEW)
    assert list(spec) == list(plain)
    replay = ol.spec_counters(prompt, plain, kv_cap=128)
    print(name, pseed, st, "replay", replay)
    assert st["hits"] > 0 and st["forwards"] > 0
    if st["near_ties"] == 0:
        assert {k: st[k] for k in ol.SPEC_COUNTERS} == replay
        assert st["single_steps"] == st["steps"] - st["forwards"]
    assert st["emitted"] + st["single_steps"] + 1 == N_NEW
    # the sequence can be continued by the plain path afterwards: cache and cursor are where greedy leaves them
    more, _ = gm.decode_loop(int(spec[-1]), len(prompt) + N_NEW - 1, 4)
    gm.reset()
    plain2, _, _ = gm.generate(prompt, N_NEW + 4)
    assert list(more) == list(plain2[N_NEW:])


def test_spec_settings_and_limits(model):
    name, cfg, gm, om = model
    prompt = periodic_prompt(cfg["NV"], 6)
    plain, _, _ = gm.generate(prompt, 40)
    for kw in (dict(k_max=1, k_min=1, m=1), dict(k_max=5, k_min=2, m=15), dict(k_max=3, k_min=1, m=40),
               dict(min_margin=1e30)):                       # an impossible margin: every step falls back to the plain kernel
        gm.reset()
        spec, st, _, _ = gm.generate_spec(prompt, 40, **kw)
        assert list(spec) == list(plain), kw
        if kw.get("min_margin"):
            assert st["accepted"] == 0 and st["emitted"] == 0 and st["single_steps"] == 39
    # a draft never runs past the KV capacity (kv_cap 128): generate right up to it
    gm.reset()
    n_max = 128 - len(prompt) + 1
    plain, _, _ = gm.generate(prompt, n_max)
    gm.reset()
    spec, st, _, _ = gm.generate_spec(prompt, n_max)
    assert list(spec) == list(plain)
    with pytest.raises(hb.HxError):
        gm.generate_spec(prompt, n_max + 1)
