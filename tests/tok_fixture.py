"""A small byte-level BPE vocabulary in the GPT-2 file formats, built from a seeded corpus: 256 byte tokens, the
merges a plain BPE trainer learns, and two control tokens.  Used by the tokenizer tests and by the script that writes
their golden file."""
import collections
import json

import numpy as np

SPECIALS = ["<|im_start|>", "<|im_end|>"]
WORDS = ["the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "hello", "world", "it's", "we'll", "they've", "I'm", "don't",
         "you're", "he'd", "2024", "3.14159", "42", "naïve", "café", "über", "日本語", "テスト", "данные", "x=y+1;", "(a,b)", "foo_bar", "***",
         "->", "e-mail", "tokens", "tokenizer", "byte", "level"]


def byte_to_unicode():
    """GPT-2's printable stand-ins for bytes: printable Latin-1 bytes stand for themselves, the rest for 256, 257, ..."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, k = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + k); k += 1
    return table


def corpus(seed=5, n=600):
    rng = np.random.default_rng(seed)
    seps = [" ", " ", " ", "  ", "\n", ", ", ". ", "\t", " \n ", "   "]
    out = []
    for _ in range(n):
        out.append(WORDS[int(rng.integers(0, len(WORDS)))])
        out.append(seps[int(rng.integers(0, len(seps)))])
    return "".join(out)


def train(text, n_merges=180):
    """Plain BPE over space-prefixed words (enough to get realistic merge rules; not the pre-tokenizer under test)."""
    words = collections.Counter()
    for w in text.replace("\n", " ").replace("\t", " ").split(" "):
        if w:
            words[tuple(bytes([b]) for b in (" " + w).encode("utf-8"))] += 1
    merges = []
    for _ in range(n_merges):
        pairs = collections.Counter()
        for w, c in words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += c
        if not pairs:
            break
        (a, b), _ = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
        merges.append((a, b))
        new = collections.Counter()
        for w, c in words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b); i += 2
                else:
                    out.append(w[i]); i += 1
            new[tuple(out)] += c
        words = new
    return merges


def write_files(d, seed=5):
    b2u = byte_to_unicode()
    enc = lambda bs: "".join(b2u[b] for b in bs)
    merges = train(corpus(seed))
    vocab = {}
    for b in range(256):
        vocab[enc(bytes([b]))] = len(vocab)
    for a, b in merges:
        vocab.setdefault(enc(a + b), len(vocab))
    for s in SPECIALS:
        vocab[s] = len(vocab)
    vpath, mpath = d + "/vocab.json", d + "/merges.txt"
    json.dump(vocab, open(vpath, "w"))                      # ensure_ascii: the stand-ins above 0x7F become \\uXXXX escapes
    with open(mpath, "w", encoding="utf-8") as f:
        f.write("#version: 0.2\n")
        for a, b in merges:
            f.write(enc(a) + " " + enc(b) + "\n")
    return vpath, mpath, len(vocab)


def texts(seed=9):
    rng = np.random.default_rng(seed)
    fixed = ["", " ", "  ", "hello world", "Hello  world  ", " the quick brown fox", "it's we'll they've I'm don't you're he'd 'x 'll",
             "line one\nline two\n\n  indented\ttab", "3.14159 + 42 = 45.14159?!", "naïve café über", "日本語のテスト、データ。", "данные и tokens",
             "trailing spaces   ", "\n\n\n", "a b c　d", "x=y+1; (a,b) -> foo_bar *** e-mail", "'''", "''s't",
             "<|im_start|>user\nhello<|im_end|>\n<|im_start|>assistant\n", "emoji \U0001F600 ok", bytes([0xff, 0xfe, 0x41, 0x80]).decode("latin-1")]
    for _ in range(40):
        n = int(rng.integers(1, 60))
        alphabet = list(" \n\tabcdefghijklmnopqrstuvwxyzABC0123456789'.,;:!?-_()é日本дан")
        fixed.append("".join(alphabet[int(rng.integers(0, len(alphabet)))] for _ in range(n)))
    return fixed
