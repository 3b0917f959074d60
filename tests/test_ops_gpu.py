"""GPU parity of RMSNorm, RoPE, attention, the fp16 classifier GEMV, embedding gather and the greedy hand-off."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import assert_close
from llama_cu_awq_b200 import _lib, ops
from oracle import q4_oracle as O

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n", [8, 128, 1000, 4096, 5120, 8192])
def test_rmsnorm(n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 3).astype(np.float16)
    w = rng.uniform(0.5, 1.5, n).astype(np.float16)
    o = torch.empty(n, dtype=torch.float16, device="cuda")
    ops.rmsnorm(o, dev(x), dev(w), n)
    ref = O.rmsnorm(x, w)
    got = o.cpu().numpy()
    assert_close(got, ref, "rmsnorm", max_rel=2e-3)
    def key(a):
        u = a.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    assert np.abs(key(got) - key(ref)).max() <= 1  # at most 1 fp16 step
    xd = dev(x)
    ops.rmsnorm(xd, xd, dev(w), n)  # in place, as the final norm does (llama2_q4.cu:528)
    assert (xd.cpu().numpy().view(np.uint16) == got.view(np.uint16)).all()


@pytest.mark.parametrize("heads,kv_heads,hs,pos", [(2, 2, 64, 0), (32, 32, 128, 17), (8, 1, 128, 4095), (4, 2, 128, 300)])
def test_rope(heads, kv_heads, hs, pos):
    rng = np.random.default_rng(pos + heads)
    q = rng.standard_normal(heads * hs).astype(np.float16)
    seq, layers = pos + 2, 2
    kv_dim = kv_heads * hs
    kc = rng.standard_normal(layers * seq * kv_dim).astype(np.float16)
    loff = 1 * seq * kv_dim
    qd, kd = dev(q), dev(kc)
    ops.RoPERotation(qd, kd, heads, kv_heads, hs, torch.tensor([pos], dtype=torch.int32, device="cuda"), loff, 10000.0)
    row = slice(loff + pos * kv_dim, loff + (pos + 1) * kv_dim)
    qr, kr = O.rope(q, kc[row], heads, kv_heads, hs, pos, 10000.0)
    # sin/cos of large arguments differ by a few ulp of fp32 between libm and CUDA; outputs are fp16
    assert_close(qd.cpu().numpy(), qr, "rope q", max_rel=2e-3)
    k_out = kd.cpu().numpy()
    assert_close(k_out[row], kr, "rope k", max_rel=2e-3)
    k_out[row] = kc[row]
    assert (k_out.view(np.uint16) == kc.view(np.uint16)).all(), "touched other cache rows"


@pytest.mark.parametrize("heads,kv_mul,hs,pos", [(2, 1, 64, 0), (4, 1, 128, 5), (32, 1, 128, 15), (32, 1, 128, 271), (8, 8, 128, 1000),
                                               (64, 8, 128, 33), (40, 1, 128, 2047), (2, 2, 256, 77)])
def test_attention(heads, kv_mul, hs, pos):
    rng = np.random.default_rng(pos * 3 + heads)
    kv_stride = heads * hs // kv_mul
    seq = pos + 3
    q = rng.standard_normal(heads * hs).astype(np.float16)
    kc = (rng.standard_normal((seq, kv_stride)) * 0.5).astype(np.float16)
    vc = rng.standard_normal((seq, kv_stride)).astype(np.float16)
    kc[pos + 1:] = np.float16(100.0)  # rows beyond pos must not be read
    vc[pos + 1:] = np.float16(-1000.0)
    out = torch.full((heads * hs,), float("nan"), dtype=torch.float16, device="cuda")
    scratch = ops.attention_scratch(heads, hs)
    ops.MultiHeadAttention(out, dev(q), dev(kc), dev(vc), scratch, heads, hs, kv_mul, seq, torch.tensor([pos], dtype=torch.int32, device="cuda"))
    ref = O.attention(q, kc, vc, heads, hs, kv_mul, pos)
    # the reference rounds probabilities to fp16 before the V product; the split softmax here stays in fp32
    assert_close(out.cpu().numpy(), ref, f"attention pos={pos}", max_rel=5e-3)


@pytest.mark.parametrize("n,d", [(8, 8), (256, 40), (4096, 1000), (5120, 4000), (4096, 32000)])
def test_classifier_matvec_f16(n, d):
    rng = np.random.default_rng(n + d)
    W = (rng.standard_normal((d, n)) * 0.02).astype(np.float16)
    x = rng.standard_normal(n).astype(np.float16)
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    ops.matmul(y, dev(x), dev(W), n, d)
    assert_close(y.cpu().numpy(), O.matvec_f16(x, W, n, d, order=1), "classifier", max_rel=2e-3)


def _pinned_mailbox():
    t = torch.zeros(4 + 64, dtype=torch.int32).pin_memory()
    return t  # [0] = pos, [4:] = tokens (layout is private to this test)


def test_embed_and_argmax_handoff():
    rng = np.random.default_rng(0)
    V, dim = 1000, 256
    table = rng.standard_normal((V, dim)).astype(np.float16)
    mb = _pinned_mailbox()
    mb[4 + 3] = 777
    pos_dev = torch.tensor([3], dtype=torch.int32, device="cuda")
    mb[0] = 3
    x = torch.empty(dim, dtype=torch.float16, device="cuda")
    tokens_ptr = mb.data_ptr() + 16
    ops.copy_embedding(x, dev(table), dim, tokens_ptr, pos_dev)
    torch.cuda.synchronize()
    assert (x.cpu().numpy().view(np.uint16) == table[777].view(np.uint16)).all()

    logits = rng.standard_normal(V).astype(np.float16)
    logits[[123, 600]] = np.float16(9.0)  # tie: lowest index wins
    ops.sample_greedy(dev(logits), V, tokens_ptr, mb.data_ptr(), pos_dev, True)
    torch.cuda.synchronize()
    assert int(mb[0]) == 4 and int(pos_dev.item()) == 4 and int(mb[4 + 4]) == 123 == O.argmax(logits)
    ops.sample_greedy(dev(logits), V, tokens_ptr, mb.data_ptr(), pos_dev, False)  # prompt phase: position only
    torch.cuda.synchronize()
    assert int(mb[0]) == 5 and int(mb[4 + 5]) == 0


@pytest.mark.parametrize("size", [8, 1000, 32000])
def test_argmax_matches_oracle(size):
    rng = np.random.default_rng(size)
    for trial in range(3):
        logits = (rng.standard_normal(size) * 2).astype(np.float16)  # fp16 values collide often at 32000
        mb = _pinned_mailbox()
        pos_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.sample_greedy(dev(logits), size, mb.data_ptr() + 16, mb.data_ptr(), pos_dev, True)
        torch.cuda.synchronize()
        assert int(mb[4 + 1]) == O.argmax(logits)
