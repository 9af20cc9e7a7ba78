"""The serve worker (hx_worker / hx_serve) against the reference's own --serve mode (run_serve,
helixc/runtime/gpt2_infer.c:3284-3400) run unmodified on the same B200 with its own PTX: the same request frames
must give the same event stream -- event kinds, sequence numbers, token ids (greedy and seeded sampling), context
lengths, error events -- and logits that agree to the decode tolerance.  Without the compiled reference worker the
stream is checked against the CPU restatement (greedy tokens, sampler replay on the restatement's logits)."""
import json
import os
import subprocess

import numpy as np
import pytest

import helix_b200 as hb
import oracle_lib as ol
from test_ref_worker_gpu import KOVC, SIDE, have_worker

pytestmark = pytest.mark.gpu

CFG = dict(NL=2, DM=256, NH=4, NKV=2, DH=64, DFF=512, NV=1000)
PROMPT = [11, 502, 73, 999, 0, 640, 27]
SAMPLING = dict(temperature=0.8, top_k=20, top_p=0.95, rep_penalty=1.1, seed=7)
SAMPLING2 = dict(temperature=1.2, top_p=0.9, min_p=0.01, freq_penalty=0.2, pres_penalty=0.1, seed=99)
FRAMES = [
    {"ids": PROMPT, "n_gen": 8, "request_id": "a", "detail": "token"},
    # the reference resets its sampler before it reads a frame's sampling fields: this first sampling frame draws from
    # the unseeded generator, the next one is reset with THIS frame's seed
    dict({"ids": PROMPT, "n_gen": 10, "request_id": "b", "detail": "token"}, **SAMPLING),
    dict({"ids": PROMPT, "n_gen": 10, "request_id": "b2", "detail": "token"}, **SAMPLING2),
    {"n_gen": 3, "request_id": "c", "detail": "token"},                               # nothing to run
    {"prompt": "hello", "n_gen": 3, "request_id": "d", "detail": "token"},            # no tokenizer linked
    {"ids": PROMPT, "n_gen": 200, "request_id": "e", "detail": "token"},              # beyond --max-ctx
    {"ids": [5, 6], "request_id": "f", "detail": "token"},                            # n_gen defaults to 20
    {"cmd": "quit"},
    {"ids": PROMPT, "n_gen": 2, "request_id": "never", "detail": "token"},
]
MAX_CTX = 128


def events(text):
    return [json.loads(l) for l in text.splitlines() if l.startswith("{")]


@pytest.fixture(scope="module")
def model_file(tmp_path_factory):
    d = tmp_path_factory.mktemp("serve")
    path = str(d / "m.weights")
    ol.write_v3(path, CFG, ol.synth_tensors(CFG, seed=41))
    return path


@pytest.fixture(scope="module")
def ours(model_file):
    assert os.path.exists(hb.worker_path()), "helix_b200/hx_worker is not built"
    stdin = "".join(json.dumps(f) + "\n" for f in FRAMES)
    p = subprocess.run([hb.worker_path(), model_file, "--serve", "--max-ctx", str(MAX_CTX)], input=stdin, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "GPT2_SERVE_READY" in p.stderr, p.stderr[-2000:]
    return events(p.stdout)


def test_stream_shape_and_restatement(ours, model_file):
    kinds = [e["_ev"] for e in ours]
    want = (["hello", "tokenize"] + ["forward_begin", "token"] * 8 + ["done"] + (["hello", "tokenize"] + ["forward_begin", "token"] * 10 + ["done"]) * 2 +
            ["error", "error", "error"] + ["hello", "tokenize"] + ["forward_begin", "token"] * 20 + ["done"])
    assert kinds == want
    assert [e["seq"] for e in ours] == list(range(len(ours)))            # one counter for the life of the worker
    errs = [e for e in ours if e["_ev"] == "error"]
    assert [(e["where"], e["message"], e["fatal"]) for e in errs] == [
        ("load", "bad request json", False), ("tokenize", "no in-process tokenizer and no pre-tokenized ids", False),
        ("forward", "context exceeds --max-ctx; raise --max-ctx", False)]
    done = [e for e in ours if e["_ev"] == "done"]
    assert (done[0]["n_prompt"], done[0]["n_gen"], done[0]["n_total"], done[0]["nonfinite"]) == (7, 8, 15, 0)
    om = ol.OracleModel(model_file, kv_cap=MAX_CTX)
    assert done[0]["gen_ids"] == [int(t) for t in om.generate(np.array(PROMPT, np.int32), 8)]
    assert done[3]["gen_ids"] == [int(t) for t in om.generate(np.array([5, 6], np.int32), 20)]
    # the two sampling requests replayed with the restatement's logits and the library's sampler, in the worker's order
    # of operations: frame b is not reset (the frame before it was greedy), frame b2 is reset with frame b's parameters
    sm = hb.Sampler(CFG["NV"])
    def replay(n):
        ids = list(PROMPT); got = []
        lg = om.prefill(np.array(ids, np.int32))
        for step in range(n):
            t = sm.next(lg); sm.count(t); got.append(t); ids.append(t)
            lg = om.decode(t, len(ids) - 1)
        return got
    sm.configure(**SAMPLING)
    assert done[1]["gen_ids"] == replay(10)
    sm.reset(PROMPT, **SAMPLING); sm.configure(**SAMPLING2)
    got2 = replay(10)
    assert done[2]["gen_ids"] == got2 and got2 != done[1]["gen_ids"]
    om.close(); sm.close()
    toks = [e for e in ours if e["_ev"] == "token"][:8]
    assert [t["context_len"] for t in toks] == list(range(8, 16)) and all(t["string"] == "" for t in toks)


def test_same_stream_as_the_reference_worker(ours, model_file, tmp_path):
    if not have_worker():
        pytest.skip("oracle/_ref/gpt2_infer or oracle/_ref/kovc/model14.ptx not built")
    env = {k: v for k, v in os.environ.items() if not k.startswith("HX_")}
    env.pop("LD_LIBRARY_PATH", None)
    env.update({k: os.path.join(KOVC, v + ".ptx") for k, v in SIDE.items()})
    env.update(HX_KV="1")
    stdin = "".join(json.dumps(f) + "\n" for f in FRAMES)
    p = subprocess.run([ol.REF_INFER, os.path.join(KOVC, "model14.ptx"), model_file, "--serve", "--max-ctx", str(MAX_CTX)], input=stdin,
                       capture_output=True, text=True, timeout=600, env=env, cwd=str(tmp_path))
    assert "GPT2_SERVE_READY" in p.stderr, p.stderr[-3000:]
    ref = events(p.stdout)
    assert [e["_ev"] for e in ref] == [e["_ev"] for e in ours]
    assert [e["seq"] for e in ref] == [e["seq"] for e in ours]
    worst = 0.0
    for r, o in zip(ref, ours):
        ev = r["_ev"]
        if ev == "hello":
            for k in ("schema_version", "n_layer", "n_head", "d_model", "d_ff", "n_vocab", "mode"):
                assert r[k] == o[k], k
        elif ev == "tokenize":
            assert (r["ids"], r["strings"], r["n_prompt"], r["s_pad"]) == (o["ids"], o["strings"], o["n_prompt"], o["s_pad"])
        elif ev == "forward_begin":
            assert {k: r[k] for k in ("step", "context_len", "s_pad", "n_layers")} == {k: o[k] for k in ("step", "context_len", "s_pad", "n_layers")}
        elif ev == "token":
            assert (r["step"], r["id"], r["string"], r["context_len"]) == (o["step"], o["id"], o["string"], o["context_len"])
            worst = max(worst, abs(r["logit"] - o["logit"]))
        elif ev == "done":
            for k in ("n_prompt", "n_gen", "n_total", "text", "gen_ids", "nonfinite"):
                assert r[k] == o[k], k
        elif ev == "error":
            assert (r["where"], r["message"], r["fatal"]) == (o["where"], o["message"], o["fatal"])
    print(f"serve: {len(ref)} events equal; chosen-token logits differ by at most {worst:.3g}")
    assert worst < 2e-4


# ---- with a tokenizer: "prompt" frames, decoded pieces in the events, stop strings, control tokens ------------------
import tok_fixture as tf   # noqa: E402

TEXT_FRAMES = [
    {"prompt": "hello world, the quick brown fox", "n_gen": 6, "request_id": "t1", "detail": "token"},
    {"prompt": "<|im_start|>user\nit's 42<|im_end|>\n", "n_gen": 5, "request_id": "t2", "detail": "token"},
    {"prompt": "naïve café 日本語", "n_gen": 12, "request_id": "t3", "detail": "token", "stop": ["\n", "fox"]},
    {"ids": [5, 6, 7], "n_gen": 3, "request_id": "t4", "detail": "token"},
    {"cmd": "quit"},
]


@pytest.fixture(scope="module")
def text_setup(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("serve_text"))
    vpath, mpath, nv = tf.write_files(d)
    cfg = dict(CFG, NV=((nv + 63) // 64) * 64)                      # the reference's GEMMs want widths in multiples of 64
    path = d + "/m.weights"
    ol.write_v3(path, cfg, ol.synth_tensors(cfg, seed=43))
    return d, vpath, mpath, path, cfg


def run_text(cmd, env, cwd):
    stdin = "".join(json.dumps(f) + "\n" for f in TEXT_FRAMES)
    # pieces of a byte-level vocabulary need not be valid UTF-8: the stream is read as bytes, one byte per character
    p = subprocess.run(cmd, input=stdin.encode(), capture_output=True, timeout=600, env=env, cwd=cwd)
    assert b"GPT2_SERVE_READY" in p.stderr, p.stderr[-3000:]
    return events(p.stdout.decode("latin-1"))


def test_text_frames(text_setup):
    d, vpath, mpath, path, cfg = text_setup
    env = dict(os.environ, HX_SPECIALS="1")
    ours = run_text([hb.worker_path(), path, "--serve", "--max-ctx", str(MAX_CTX), "--vocab", vpath, "--merges", mpath], env, d)
    tk = hb.Tokenizer(vpath, mpath)
    toks = [e for e in ours if e["_ev"] == "tokenize"]
    assert toks[0]["ids"] == list(tk.encode(TEXT_FRAMES[0]["prompt"]))
    assert "".join(toks[0]["strings"]).encode("latin-1") == TEXT_FRAMES[0]["prompt"].encode()
    assert toks[1]["ids"] == list(tk.encode(TEXT_FRAMES[1]["prompt"], with_specials=True)) and toks[1]["strings"][0] == "<|im_start|>"
    done = [e for e in ours if e["_ev"] == "done"]
    for dn in done:
        assert dn["text"].encode("latin-1") == tk.decode(dn["gen_ids"])
    # the stop strings end request t3 at the first piece that completes one of them, and never later than n_gen
    gen3 = done[2]["gen_ids"]
    text3 = tk.decode(gen3)
    assert len(gen3) <= 12 and (len(gen3) == 12 or text3.endswith(b"\n") or text3.endswith(b"fox"))
    tk.close()
    if not (have_worker() and os.path.exists(ol.REF_INFER_SERVE)):
        pytest.skip("the reference serve worker with its tokenizer is not built")
    renv = {k: v for k, v in os.environ.items() if not k.startswith("HX_")}
    renv.pop("LD_LIBRARY_PATH", None)
    renv.update({k: os.path.join(KOVC, v + ".ptx") for k, v in SIDE.items()})
    renv.update(HX_KV="1", HX_SPECIALS="1")
    ref = run_text([ol.REF_INFER_SERVE, os.path.join(KOVC, "model14.ptx"), path, "--serve", "--max-ctx", str(MAX_CTX), "--vocab", vpath,
                    "--merges", mpath], renv, d)
    assert [e["_ev"] for e in ref] == [e["_ev"] for e in ours]
    for r, o in zip(ref, ours):
        ev = r["_ev"]
        if ev == "tokenize":
            assert (r["ids"], r["strings"], r["n_prompt"], r["s_pad"]) == (o["ids"], o["strings"], o["n_prompt"], o["s_pad"])
        elif ev == "token":
            assert (r["step"], r["id"], r["string"], r["context_len"]) == (o["step"], o["id"], o["string"], o["context_len"])
            assert abs(r["logit"] - o["logit"]) < 2e-4
        elif ev == "done":
            for k in ("n_prompt", "n_gen", "n_total", "text", "gen_ids", "nonfinite"):
                assert r[k] == o[k], k
    print(f"serve with tokenizer: {len(ref)} events equal to the reference worker's")
