"""ctypes loader of the CPU oracle (oracle/q4_oracle.c). Test infrastructure only: imported by tests/,
by __graft_entry__.smoke() and by bench.py's cpu_baseline / reference legs, never by the package."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libq4oracle.so")
_lib = None


def build():
    subprocess.run(["make", "-C", HERE, "-s"], check=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = C.CDLL(LIB_PATH)
        L.q4o_h2f.restype = C.c_float
        L.q4o_h2f.argtypes = [C.c_uint16]
        L.q4o_f2h.restype = C.c_uint16
        L.q4o_f2h.argtypes = [C.c_float]
        L.q4o_model_open.restype = C.c_void_p
        L.q4o_model_open.argtypes = [C.c_void_p, C.c_size_t]
        L.q4o_model_close.argtypes = [C.c_void_p]
        L.q4o_model_forward.restype = C.c_int
        L.q4o_model_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
        L.q4o_model_logits.restype = C.c_void_p
        L.q4o_model_logits.argtypes = [C.c_void_p]
        L.q4o_model_x.restype = C.c_void_p
        L.q4o_model_x.argtypes = [C.c_void_p]
        L.q4o_num_threads.restype = C.c_int
        L.q4o_sample_topp.restype = C.c_int
        L.q4o_sample_topp.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float]
        L.q4o_random_f32.restype = C.c_float
        L.q4o_random_f32.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


def _qw(q):
    return _c(q["weight"], np.uint32), _c(q["zeros"], np.uint32), _c(q["scales"], np.float16)


def unpack(q, K, N):
    w, z, _ = _qw(q)
    G = (K + 127) // 128
    qo = np.empty((N, K), np.uint8)
    zo = np.empty((N, G), np.uint8)
    lib().q4o_unpack(_ptr(qo), _ptr(zo), _ptr(w), _ptr(z), K, N)
    return qo, zo


def dequant(q, K, N):
    w, z, s = _qw(q)
    out = np.empty((N, K), np.float32)
    lib().q4o_dequant(_ptr(out), _ptr(w), _ptr(z), _ptr(s), K, N)
    return out


def matvec(x, q, K, N, y_old=None, gpu_count=1, order=0):
    w, z, s = _qw(q)
    x = _c(x, np.float16)
    y = np.zeros(N, np.float16) if y_old is None else _c(y_old, np.float16).copy()
    lib().q4o_matvec(_ptr(y), _ptr(x), _ptr(w), _ptr(z), _ptr(s), K, N, int(y_old is not None), gpu_count, order)
    return y


def matvec_f32(x, q, K, N):
    w, z, s = _qw(q)
    x = _c(x, np.float16)
    y = np.zeros(N, np.float32)
    lib().q4o_matvec_f32(_ptr(y), _ptr(x), _ptr(w), _ptr(z), _ptr(s), K, N)
    return y


def ffn_silu(x, gate, up, K, N, order=0):
    gw, gz, gs = _qw(gate)
    uw, uz, us = _qw(up)
    x = _c(x, np.float16)
    h = np.zeros(N, np.float16)
    lib().q4o_ffn_silu(_ptr(h), _ptr(x), _ptr(gw), _ptr(gz), _ptr(gs), _ptr(uw), _ptr(uz), _ptr(us), K, N, order)
    return h


def matvec_f16(x, W, K, N, alpha=1.0, order=0):
    x = _c(x, np.float16)
    W = _c(W, np.float16)
    y = np.zeros(N, np.float16)
    lib().q4o_matvec_f16(_ptr(y), _ptr(x), _ptr(W), K, N, C.c_float(alpha), order)
    return y


def rmsnorm(x, w):
    x = _c(x, np.float16)
    w = _c(w, np.float16)
    o = np.zeros_like(x)
    lib().q4o_rmsnorm(_ptr(o), _ptr(x), _ptr(w), x.size)
    return o


def rope(q, k_row, n_heads, n_kv_heads, head_size, pos, theta):
    q = _c(q, np.float16).copy()
    k = _c(k_row, np.float16).copy()
    lib().q4o_rope(_ptr(q), _ptr(k), n_heads, n_kv_heads, head_size, pos, C.c_float(theta))
    return q, k


def attention(q, kcache, vcache, n_heads, head_size, kv_mul, pos):
    """kcache / vcache: fp16 [T>=pos+1][kv_stride]."""
    q = _c(q, np.float16)
    kc = _c(kcache, np.float16)
    vc = _c(vcache, np.float16)
    out = np.zeros(n_heads * head_size, np.float16)
    lib().q4o_attention(_ptr(out), _ptr(q), _ptr(kc), _ptr(vc), n_heads, head_size, kv_mul, kc.shape[1], pos)
    return out


def argmax(logits):
    logits = _c(logits, np.float16)
    return lib().q4o_argmax(_ptr(logits), logits.size)


def sample_topp(logits, temperature, topp, coin):
    """(token, probabilities): the non-greedy branch of the reference's sample(); `logits` is not modified."""
    p = _c(logits, np.float16).copy()
    tok = lib().q4o_sample_topp(_ptr(p), p.size, C.c_float(temperature), C.c_float(topp), C.c_float(coin))
    return tok, p


class Rng:
    """The reference's xorshift* state (sampler.h:66-75)."""

    def __init__(self, seed):
        self.state = C.c_ulonglong(seed)

    def f32(self):
        return float(lib().q4o_random_f32(C.byref(self.state)))


def allreduce_ref_order(parts, rank):
    parts = _c(parts, np.float16)
    g, n = parts.shape
    out = np.zeros(n, np.float16)
    lib().q4o_allreduce_ref_order(_ptr(out), _ptr(parts), g, rank, n)
    return out


class Model:
    """Whole-model oracle on a packed file image (single-GPU math)."""

    def __init__(self, image):
        self.image = np.ascontiguousarray(np.frombuffer(image, dtype=np.uint8))
        self.h = lib().q4o_model_open(_ptr(self.image), self.image.size)
        if not self.h:
            raise ValueError("bad model image")
        hdr = np.frombuffer(self.image[:28].tobytes(), np.int32)
        self.dim, self.hidden_dim, self.n_layers, self.n_heads, self.n_kv_heads, self.vocab_size, self.seq_len = [int(v) for v in hdr]

    def forward(self, token, pos, order=0):
        return lib().q4o_model_forward(self.h, int(token), int(pos), order)

    def logits(self):
        p = lib().q4o_model_logits(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), (self.vocab_size,)).view(np.float16).copy()

    def x(self):
        p = lib().q4o_model_x(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), (self.dim,)).view(np.float16).copy()

    def close(self):
        if self.h:
            lib().q4o_model_close(self.h)
            self.h = None

    def __del__(self):
        self.close()


def num_threads():
    return lib().q4o_num_threads()
