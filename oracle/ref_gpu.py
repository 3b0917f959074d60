"""ctypes loader of oracle/_ref/libref_q4.so: the reference's own CUDA kernels, wrappers and generation loop
compiled for sm_100a from the reference sources (oracle/Makefile, oracle/ref_harness.cu). Needs a GPU.
Test / baseline infrastructure only."""
import ctypes as C
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_ref", "libref_q4.so")
_lib = None


def available():
    return os.path.exists(LIB_PATH) and torch.cuda.is_available()


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(LIB_PATH)
        L.ref_stream.restype = C.c_void_p
        assert L.ref_init() == 0
        _lib = L
    return _lib


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _q(q):
    return dev(q["weight"].view(np.int32)), dev(q["zeros"].view(np.int32)), dev(q["scales"])


def matmul_q4(x, q, K, N, y_old=None, gpu_count=1):
    w, z, s = _q(q)
    y = torch.zeros(N, dtype=torch.float16, device="cuda") if y_old is None else dev(y_old)
    torch.cuda.synchronize()
    xd = dev(x)  # keep every device tensor referenced until the kernel has run
    lib().ref_matmul_q4(_p(y), _p(xd), _p(w), _p(z), _p(s), K, N, int(y_old is not None), gpu_count, -1, None)
    lib().ref_sync()
    return y.cpu().numpy()


def ffn_matvec_silu(x, gate, up, K, N):
    gw, gz, gs = _q(gate)
    uw, uz, us = _q(up)
    h = torch.zeros(N, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    xd = dev(x)
    lib().ref_ffn_matvec_silu(_p(h), _p(xd), _p(gw), _p(gz), _p(gs), _p(uw), _p(uz), _p(us), K, N)
    lib().ref_sync()
    return h.cpu().numpy()


def rmsnorm(x, w):
    o = torch.zeros(x.size, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    xd, wd = dev(x), dev(w)
    lib().ref_rmsnorm(_p(o), _p(xd), _p(wd), x.size)
    lib().ref_sync()
    return o.cpu().numpy()


def rope(q, kcache, n_heads, n_kv_heads, head_size, pos, loff, theta):
    qd, kd = dev(q), dev(kcache)
    pd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    lib().ref_rope(_p(qd), _p(kd), n_heads, n_kv_heads, head_size, _p(pd), loff, C.c_float(theta))
    lib().ref_sync()
    return qd.cpu().numpy(), kd.cpu().numpy()


def mha(q, kc, vc, n_heads, head_size, kv_mul, pos):
    out = torch.zeros(n_heads * head_size, dtype=torch.float16, device="cuda")
    att = torch.zeros(n_heads * (pos + 8), dtype=torch.float16, device="cuda")
    pd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    qd, kd, vd = dev(q), dev(kc), dev(vc)
    lib().ref_mha(_p(out), _p(qd), _p(kd), _p(vd), _p(att), n_heads, head_size, kv_mul, pos + 1, _p(pd))
    lib().ref_sync()
    return out.cpu().numpy()


def matmul_f16(x, W, n, d):
    y = torch.zeros(d, dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    xd, Wd = dev(x), dev(W)
    lib().ref_matmul_f16(_p(y), _p(xd), _p(Wd), n, d)
    lib().ref_sync()
    return y.cpu().numpy()


def generate(path, prompt_tokens, steps, vocab_size, gpu_count=1):
    """The reference program's own loader and generation loop; gpu_count > 1 = its hybrid tensor parallelism, one host
    thread per GPU (devices 0 .. gpu_count-1 of this process)."""
    prompt = np.ascontiguousarray(prompt_tokens, dtype=np.int32)
    out = np.zeros(steps + 2, np.int32)
    logits = np.zeros(vocab_size, np.float16)
    toks, timed, secs = C.c_double(), C.c_int(), C.c_double()
    L = lib()
    rc = L.ref_generate(path.encode(), prompt.ctypes.data_as(C.c_void_p), prompt.size, steps, int(gpu_count), out.ctypes.data_as(C.c_void_p),
                        logits.ctypes.data_as(C.c_void_p), C.byref(toks), C.byref(timed), C.byref(secs))
    assert rc == 0, rc
    return out[:steps + 1], logits, toks.value, timed.value, secs.value


def sample(logits16, temperature, topp, seed):
    """The reference's sample() on fp16 logits: (token, coin)."""
    a = np.ascontiguousarray(logits16, dtype=np.float16)
    tok, coin = C.c_int(), C.c_float()
    rc = lib().ref_sample(a.ctypes.data_as(C.c_void_p), a.size, C.c_float(temperature), C.c_float(topp), C.c_ulonglong(seed), C.byref(tok), C.byref(coin))
    assert rc == 0, rc
    return tok.value, coin.value


def time_q4(kind, K, N, nmat=32, reps=20, seed=0):
    """Microseconds per launch of the reference's W4 wrapper (0 matmul, 1 qkv_matvec, 2 ffn_matvec_silu) over `nmat`
    distinct random matrices of one shape (weights from HBM, not L2)."""
    per = {0: 1, 1: 3, 2: 2}[kind]
    nmat = max(per, nmat // per * per)
    g = torch.Generator(device="cuda").manual_seed(seed)
    pw, pz, gg = ((K + 31) // 32) * 4, ((K + 127) // 128 + 7) // 8, (K + 127) // 128
    ws = [torch.randint(-2**31, 2**31 - 1, (N, pw), dtype=torch.int32, device="cuda", generator=g) for _ in range(nmat)]
    zs = [torch.randint(-2**31, 2**31 - 1, (N, pz), dtype=torch.int32, device="cuda", generator=g) for _ in range(nmat)]
    ss = [(torch.rand((N, gg), device="cuda", generator=g) * 0.018 + 0.002).half() for _ in range(nmat)]
    x = torch.randn(K, device="cuda", generator=g).half()
    ys = [torch.zeros(max(N, 8) * 4, dtype=torch.float16, device="cuda") for _ in range(3)]
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    arr = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])  # noqa: E731
    us = C.c_double()
    torch.cuda.synchronize()
    rc = lib().ref_time_q4(kind, _p(ys[0]), _p(ys[1]), _p(ys[2]), _p(x), arr(ws), arr(zs), arr(ss), nmat, K, N, reps, _p(pos), C.byref(us))
    assert rc == 0, rc
    return us.value


def time_allreduce(gpu_count, count, reps=200):
    """Microseconds per call of the reference's cudaAllReduce of `count` halfs on gpu_count GPUs (thread per GPU)."""
    us = C.c_double()
    rc = lib().ref_time_allreduce(gpu_count, count, reps, C.byref(us))
    assert rc == 0, rc
    return us.value
