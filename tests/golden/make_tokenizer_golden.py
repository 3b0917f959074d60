"""Records golden vectors of the reference's tokenizer (tokenizer.h: build_tokenizer / encode / decode / safe_printf).

Run in the build container, where the reference sources are present and `make -C oracle REF=<reference dir>` has built
oracle/_ref/libref_tok.so from them:

    python tests/golden/make_tokenizer_golden.py

Writes tests/golden/tiny_tokenizer.bin (a small synthetic vocabulary in the tokenizer.bin format: the three specials,
the 256 byte pieces, single characters and a few hundred scored merges) and tests/golden/tokenizer_golden.json (for
each test string the ids the reference's encode() returns and the text its decode() + safe_printf() would print).
"""
import ctypes as C
import json
import os
import struct

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_tok.so")

TEXTS = [
    "", " ", "a", "hello", "hello world", "Hello, World!", "  two  spaces", "the theme of the thesis", "tab\tand\nnewline",
    "café naïve", "你好 世界", "emoji \U0001F600 end", "mixed é你\U0001F600", "aaaaaaaaaaaaaaaa", "ththththth",
    "Write a poem on GPUs", "1234567890", "trailing space ", "\x7f\x01 control", "stray \x80\x80\x80\x80\x80 bytes",
]


def build_vocab(rng):
    pieces = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
    scores = [0.0, 0.0, 0.0] + [0.0] * 256
    singles = [" "] + [chr(c) for c in range(33, 127)] + ["é", "你", "好", "\t"]   # no "\n", no other CJK: byte fallback
    for s in singles:
        pieces.append(s)
        scores.append(-1000.0 - len(pieces))
    words = ["th", "he", "the", " t", " th", " the", "in", "er", "an", "re", "on", "at", "en", "nd", "ll", "lo", "hel", "hell", "hello",
             " w", "wo", "or", "wor", "world", " world", "aa", "aaaa", "es", "is", "si", "sis", "me", "eme", "of", " of", "  ", "   ",
             "GP", "GPU", "GPUs", "po", "poem", " a", "Wr", "ite", "12", "34", "1234", "ce", "pa", "space", " space", "你好", "ing"]
    for w in words:
        if w not in pieces:
            pieces.append(w)
            scores.append(float(-rng.integers(1, 400)) - 0.001 * len(pieces))   # distinct scores: no ties to break
    return pieces, scores


def main():
    rng = np.random.default_rng(0)
    pieces, scores = build_vocab(rng)
    path = os.path.join(HERE, "tiny_tokenizer.bin")
    with open(path, "wb") as f:
        f.write(struct.pack("<I", max(len(p.encode()) for p in pieces)))
        for p, s in zip(pieces, scores):
            b = p.encode()
            f.write(struct.pack("<fi", s, len(b)) + b)
    L = C.CDLL(REF_LIB)
    L.ref_tok_open.restype = C.c_void_p
    L.ref_tok_open.argtypes = [C.c_char_p, C.c_int]
    L.ref_tok_encode.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_int)]
    L.ref_tok_decode.restype = C.c_char_p
    L.ref_tok_decode.argtypes = [C.c_void_p, C.c_int, C.c_int]
    t = L.ref_tok_open(path.encode(), len(pieces))
    cases = []
    for text in TEXTS:
        raw = text.encode("utf-8", "surrogateescape") if "\x80" not in text else text.encode("latin-1")
        for bos, eos in ((1, 0), (0, 0), (1, 1)):
            buf = (C.c_int * (len(raw) + 8))()
            n = L.ref_tok_encode(t, raw, bos, eos, buf)
            ids = [int(buf[i]) for i in range(n)]
            shown, prev = [], 1
            for tok in ids:
                shown.append(L.ref_tok_decode(t, prev, tok).decode("latin-1"))
                prev = tok
            cases.append({"text_latin1": raw.decode("latin-1"), "bos": bos, "eos": eos, "ids": ids, "printed_latin1": shown})
    with open(os.path.join(HERE, "tokenizer_golden.json"), "w") as f:
        json.dump({"vocab_size": len(pieces), "cases": cases}, f, indent=0)
    print(f"{len(cases)} cases, vocabulary of {len(pieces)} pieces")


if __name__ == "__main__":
    main()
