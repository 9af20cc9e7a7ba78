"""The tokenizer (hx_tokenizer_*) against the reference's gpt2_tok.c: committed golden ids (written by
tests/golden/make_tok_golden.py from the compiled reference) and, where the compiled reference is present, live
comparison on random texts.  The vocabulary is the synthetic one of tests/tok_fixture.py."""
import json
import os
import subprocess

import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol
import tok_fixture as tf

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("tok"))
    vpath, mpath, nv = tf.write_files(d)
    t = hb.Tokenizer(vpath, mpath)
    yield t, vpath, mpath, nv
    t.close()


def test_golden_ids_of_the_reference_tokenizer(tok):
    t, _, _, nv = tok
    gold = json.load(open(os.path.join(G, "tok_golden.json")))
    assert gold["vocab_size"] == nv == t.vocab_size()
    assert len(gold["cases"]) == len(tf.texts())
    for case in gold["cases"]:
        data = bytes.fromhex(case["utf8_hex"])
        assert list(t.encode(data)) == case["ids"], data
        assert t.decode(case["ids"]) == data


def test_live_against_the_compiled_reference(tok):
    if not os.path.exists(ol.REF_TOK):
        pytest.skip("oracle/_ref/gpt2_tok not built")
    t, vpath, mpath, _ = tok
    rng = np.random.default_rng(21)
    alphabet = list(" \n\t\r abcdefghijklmnopqrstuvwxyzTHEQUICK0123456789'.,;:!?-_()[]{}<>|=+*/\\\"éüñ日本語данные") + ["it's", " we'll", " ", "　", "  "]
    for _ in range(120):
        text = "".join(alphabet[int(rng.integers(0, len(alphabet)))] for _ in range(int(rng.integers(1, 120))))
        data = text.encode("utf-8")
        p = subprocess.run([ol.REF_TOK, vpath, mpath, "encode"], input=data, capture_output=True)
        assert p.returncode == 0, p.stderr
        assert list(t.encode(data)) == [int(x) for x in p.stdout.split()], text


def test_control_tokens_and_limits(tok, tmp_path):
    t, vpath, mpath, nv = tok
    im_start, im_end = nv - 2, nv - 1
    text = "<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n"
    ids = list(t.encode(text, with_specials=True))
    assert ids[0] == im_start and ids.count(im_start) == 2 and ids.count(im_end) == 1
    k = ids.index(im_end)
    assert ids[1:k] == list(t.encode("user\nhello")) and t.decode(ids) == text.encode()
    assert im_start not in list(t.encode(text))                       # without the split the brackets are ordinary text
    assert list(t.encode("")) == [] and t.decode([]) == b""
    assert t.decode([nv + 5, -1]) == b""                              # unknown ids contribute nothing
    with pytest.raises(hb.HxError):
        hb.Tokenizer(str(tmp_path / "missing.json"), mpath)
    # a vocabulary that lacks a byte: the text cannot be encoded, and the call says so instead of emitting a wrong id
    v = json.load(open(vpath)); del v["a"]
    json.dump(v, open(tmp_path / "v2.json", "w"))
    t2 = hb.Tokenizer(str(tmp_path / "v2.json"), mpath)
    with pytest.raises(hb.HxError, match="no vocabulary entry"):
        t2.encode("xax")
    t2.close()
