"""Writes tests/golden/tok_golden.json: the ids the reference's tokenizer (helixc/runtime/gpt2_tok.c compiled as
oracle/_ref/gpt2_tok by `make -C oracle ref`) gives for the texts of tests/tok_fixture.py over that fixture's
vocabulary.  Run from the repository root: python tests/golden/make_tok_golden.py"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol          # noqa: E402
import tok_fixture as tf         # noqa: E402


def main():
    d = tempfile.mkdtemp()
    vpath, mpath, nv = tf.write_files(d)
    out = {"vocab_size": nv, "cases": []}
    for t in tf.texts():
        data = t.encode("utf-8")
        p = subprocess.run([ol.REF_TOK, vpath, mpath, "encode"], input=data, capture_output=True)
        assert p.returncode == 0, p.stderr
        ids = [int(x) for x in p.stdout.split()]
        q = subprocess.run([ol.REF_TOK, vpath, mpath, "decode"] + [str(i) for i in ids], capture_output=True)
        assert q.stdout == data, (t, q.stdout)
        out["cases"].append({"utf8_hex": data.hex(), "ids": ids})
    json.dump(out, open(os.path.join(HERE, "tok_golden.json"), "w"))
    print("wrote", len(out["cases"]), "cases")


if __name__ == "__main__":
    main()
