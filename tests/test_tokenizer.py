"""q4_tokenizer_* (host code of the library) against golden vectors recorded from the reference's own tokenizer
(tests/golden/make_tokenizer_golden.py) and, where the reference project is present beside this repository, live
against the reference's tokenizer.bin with the README prompt."""
import ctypes as C
import json
import os

import pytest

from conftest import GOLDEN, ROOT
from llama_cu_awq_b200 import _lib


def _open(path, vocab_size):
    L = _lib.lib()
    t = C.c_void_p()
    assert L.q4_tokenizer_load(C.byref(t), path.encode(), vocab_size) == 0
    return L, t


def _encode(L, t, raw, bos, eos):
    buf = (C.c_int * (len(raw) + 8))()
    n = C.c_int()
    assert L.q4_tokenizer_encode(t, raw, bos, eos, buf, len(raw) + 8, C.byref(n)) == 0
    return [int(buf[i]) for i in range(n.value)]


def test_tokenizer_matches_reference_golden_vectors():
    g = json.load(open(os.path.join(GOLDEN, "tokenizer_golden.json")))
    L, t = _open(os.path.join(GOLDEN, "tiny_tokenizer.bin"), g["vocab_size"])
    for case in g["cases"]:
        raw = case["text_latin1"].encode("latin-1")
        ids = _encode(L, t, raw, case["bos"], case["eos"])
        assert ids == case["ids"], case["text_latin1"]
        prev = 1
        for tok, want in zip(ids, case["printed_latin1"]):
            assert L.q4_tokenizer_decode(t, prev, tok).decode("latin-1") == want
            prev = tok
    L.q4_tokenizer_free(t)


def test_tokenizer_errors():
    L = _lib.lib()
    t = C.c_void_p()
    assert L.q4_tokenizer_load(C.byref(t), b"/nonexistent/tokenizer.bin", 100) == _lib.Q4_ERR_IO
    g = json.load(open(os.path.join(GOLDEN, "tokenizer_golden.json")))
    assert L.q4_tokenizer_load(C.byref(t), os.path.join(GOLDEN, "tiny_tokenizer.bin").encode(), g["vocab_size"] + 50) == _lib.Q4_ERR_IO  # short file
    L, t = _open(os.path.join(GOLDEN, "tiny_tokenizer.bin"), g["vocab_size"])
    buf = (C.c_int * 2)()
    n = C.c_int()
    assert L.q4_tokenizer_encode(t, b"hello world", 1, 0, buf, 2, C.byref(n)) == _lib.Q4_ERR_LIMIT and n.value > 2
    assert L.q4_tokenizer_decode(t, 1, 10**6) == b""
    L.q4_tokenizer_free(t)


def _reference_dir():
    ref = os.environ.get("REF") or os.path.join(os.path.dirname(ROOT), "reference")
    return ref if os.path.exists(os.path.join(ref, "tokenizer.bin")) else None


@pytest.mark.skipif(_reference_dir() is None or not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libref_tok.so")),
                    reason="reference project (tokenizer.bin) or its built tokenizer not present")
def test_tokenizer_live_against_reference_vocabulary():
    """The reference's 32000-piece tokenizer.bin: README prompt and a few more strings, encode and decode, both sides."""
    path = os.path.join(_reference_dir(), "tokenizer.bin")
    R = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_tok.so"))
    R.ref_tok_open.restype = C.c_void_p
    R.ref_tok_open.argtypes = [C.c_char_p, C.c_int]
    R.ref_tok_encode.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_int)]
    R.ref_tok_decode.restype = C.c_char_p
    R.ref_tok_decode.argtypes = [C.c_void_p, C.c_int, C.c_int]
    rt = R.ref_tok_open(path.encode(), 32000)
    L, t = _open(path, 32000)
    texts = ["Write a poem on GPUs", "", "Hello, World! 1234", "tensor parallel decode à 8 GPUs — 你好", "line one\nline two\ttabbed",
             "The quick brown fox jumps over the lazy dog. " * 4]
    for text in texts:
        raw = text.encode()
        buf = (C.c_int * (len(raw) + 8))()
        n = R.ref_tok_encode(rt, raw, 1, 0, buf)
        want = [int(buf[i]) for i in range(n)]
        assert _encode(L, t, raw, 1, 0) == want, text
        prev = 1
        for tok in want:
            assert L.q4_tokenizer_decode(t, prev, tok) == R.ref_tok_decode(rt, prev, tok)
            prev = tok
    for tok in range(0, 32000, 7):   # decode of a sweep of ids, byte pieces included
        assert L.q4_tokenizer_decode(t, 5, tok) == R.ref_tok_decode(rt, 5, tok), tok
    L.q4_tokenizer_free(t)
    R.ref_tok_close(rt)
