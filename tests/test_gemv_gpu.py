"""GPU parity of the W4 g128 dequant + GEMV kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from llama_cu_awq_b200 import _lib, ops, synth
from oracle import q4_oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [(128, 8), (256, 16), (384, 8), (96, 8), (40, 16), (1024, 24), (2048, 40), (4096, 64), (640, 5120 // 8 * 0 + 64), (3584, 32),
          (11008, 32), (13824, 16), (4096, 4096)]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def mk(K, N, seed=0):
    rng = np.random.default_rng(seed)
    q = synth.synth_qweight(rng, K, N)
    x = rng.standard_normal(K).astype(np.float16)
    return q, x, rng


@pytest.mark.parametrize("K,N", [(128, 8), (384, 16), (4096, 64), (11008, 8), (96, 8)])
def test_unpack_and_dequant_bit_exact(K, N):
    q, _, _ = mk(K, N, seed=K)
    W = ops.QWeight.from_numpy(q)
    qd, zd = ops.unpack_nibbles(W, K, N)
    qo, zo = O.unpack(q, K, N)
    assert (qd.cpu().numpy() == qo).all() and (zd.cpu().numpy() == zo).all()
    w = ops.dequant(W, K, N).cpu().numpy()
    assert (w.view(np.uint32) == O.dequant(q, K, N).view(np.uint32)).all()


@pytest.mark.parametrize("K,N", SHAPES)
def test_matvec_parity(K, N):
    q, x, _ = mk(K, N, seed=K * 7 + N)
    W = ops.QWeight.from_numpy(q)
    y = torch.full((N,), float("nan"), dtype=torch.float16, device="cuda")
    ops.matmul(y, dev(x), W, K, N)
    torch.cuda.synchronize()
    ref = O.matvec(x, q, K, N, order=1)
    r, _ = assert_close(y.cpu().numpy(), ref, f"matvec {K}x{N}")
    assert r < 4e-3  # well inside the tolerance; also compared with the unrounded sum:
    assert_close(y.cpu().numpy(), O.matvec_f32(x, q, K, N), f"matvec {K}x{N} vs f64", max_rel=4e-3)


def test_config0_single_layer():
    """The single-layer configuration of the metric: fp16 [1,4096] ~ N(0,1), 4096x4096 W4 g128, scales U[0.002,0.02], seed 0."""
    q, x, _ = mk(4096, 4096, seed=0)
    W = ops.QWeight.from_numpy(q)
    y = torch.empty(4096, dtype=torch.float16, device="cuda")
    ops.matmul(y, dev(x), W, 4096, 4096)
    r, c = assert_close(y.cpu().numpy(), O.matvec(x, q, 4096, 4096, order=1), "cfg0")
    assert r < 3e-3 and c > 0.99999


@pytest.mark.parametrize("g", [1, 2, 8])
def test_matvec_accum_residual(g):
    K, N = 1024, 256
    q, x, rng = mk(K, N, seed=g)
    W = ops.QWeight.from_numpy(q)
    y0 = (rng.standard_normal(N) * 5).astype(np.float16)
    y = dev(y0.copy())
    ops.matmul(y, dev(x), W, K, N, accum=True, gpu_count=g)
    assert_close(y.cpu().numpy(), O.matvec(x, q, K, N, y_old=y0, gpu_count=g, order=1), "accum", max_rel=4e-3)


def test_matvec_kv_cache_offset():
    K, N, seq, layers = 512, 64, 8, 3
    q, x, _ = mk(K, N, seed=5)
    W = ops.QWeight.from_numpy(q)
    cache = torch.zeros(layers * seq * N, dtype=torch.float16, device="cuda")
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    loff = 2 * seq * N
    ops.matmul(cache, dev(x), W, K, N, loff=loff, pPos=pos)
    c = cache.cpu().numpy()
    ref = O.matvec(x, q, K, N, order=1)
    assert_close(c[loff + 5 * N: loff + 6 * N], ref, "kv row", max_rel=4e-3)
    c[loff + 5 * N: loff + 6 * N] = 0
    assert not c.any(), "wrote outside the cache row"


@pytest.mark.parametrize("K,Nq,Nkv", [(256, 256, 256), (512, 512, 128), (4096, 4096, 4096), (8192, 1024, 128)])
def test_qkv_matvec(K, Nq, Nkv):
    rng = np.random.default_rng(K + Nkv)
    qs = [synth.synth_qweight(rng, K, n) for n in (Nq, Nkv, Nkv)]
    x = rng.standard_normal(K).astype(np.float16)
    Ws = [ops.QWeight.from_numpy(q) for q in qs]
    seq, l = 6, 1
    qo = torch.empty(Nq, dtype=torch.float16, device="cuda")
    kc = torch.zeros(2 * seq * Nkv, dtype=torch.float16, device="cuda")
    vc = torch.zeros(2 * seq * Nkv, dtype=torch.float16, device="cuda")
    pos = torch.tensor([3], dtype=torch.int32, device="cuda")
    loff = l * seq * Nkv
    ops.qkv_matvec(qo, kc, vc, dev(x), *Ws, K, Nq, loff, pos, kvSize=Nkv)
    row = slice(loff + 3 * Nkv, loff + 4 * Nkv)
    assert_close(qo.cpu().numpy(), O.matvec(x, qs[0], K, Nq, order=1), "q", max_rel=4e-3)
    assert_close(kc.cpu().numpy()[row], O.matvec(x, qs[1], K, Nkv, order=1), "k", max_rel=4e-3)
    assert_close(vc.cpu().numpy()[row], O.matvec(x, qs[2], K, Nkv, order=1), "v", max_rel=4e-3)
    assert int((kc != 0).sum()) <= Nkv and int((vc != 0).sum()) <= Nkv


@pytest.mark.parametrize("K,N", [(256, 8), (512, 1376), (4096, 11008), (5120, 1728)])
def test_ffn_matvec_silu(K, N):
    rng = np.random.default_rng(K + N)
    gate, up = synth.synth_qweight(rng, K, N), synth.synth_qweight(rng, K, N)
    x = (rng.standard_normal(K) * 0.25).astype(np.float16)
    h = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.ffn_matvec_silu(h, dev(x), ops.QWeight.from_numpy(gate), ops.QWeight.from_numpy(up), K, N)
    assert_close(h.cpu().numpy(), O.ffn_silu(x, gate, up, K, N, order=1), "ffn")


def test_linearity_full_size():
    """Size-independent property at the 7B down-projection size: W(a*x1 + x2) == a*W(x1) + W(x2)."""
    K, N = 11008, 4096
    q, x1, rng = mk(K, N, seed=11)
    x2 = rng.standard_normal(K).astype(np.float16)
    W = ops.QWeight.from_numpy(q)
    xs = 2.0 * x1.astype(np.float32) + x2.astype(np.float32)
    outs = []
    for x in (x1, x2, xs.astype(np.float16)):
        y = torch.empty(N, dtype=torch.float16, device="cuda")
        ops.matmul(y, dev(x), W, K, N)
        outs.append(y.float().cpu().numpy())
    assert_close(outs[2], 2.0 * outs[0] + outs[1], "linearity", max_rel=5e-3)


def test_zero_padding_nibbles_are_never_read():
    """Unused nibbles of the last zeros word may hold garbage (the reference packer leaves it there)."""
    K, N = 384, 16  # 3 groups -> 5 unused nibbles per zeros word
    q, x, _ = mk(K, N, seed=2)
    a = dict(q)
    b = dict(q)
    b["zeros"] = (q["zeros"] & np.uint32(0x00000FFF)) | np.uint32(0xABCDE000)
    ys = []
    for w in (a, b):
        y = torch.empty(N, dtype=torch.float16, device="cuda")
        ops.matmul(y, dev(x), ops.QWeight.from_numpy(w), K, N)
        ys.append(y.cpu().numpy())
    assert (ys[0].view(np.uint16) == ys[1].view(np.uint16)).all()


def test_unsupported_sizes_return_status():
    q, x, _ = mk(128, 8)
    W = ops.QWeight.from_numpy(q)
    y = torch.empty(16, dtype=torch.float16, device="cuda")
    for K, N in [(124, 8), (128, 12), (0, 8)]:
        with pytest.raises(ops.Q4Error) as e:
            ops.matmul(y, dev(x), W, K, N)
        assert e.value.status == _lib.Q4_ERR_UNSUPPORTED_SIZE
    with pytest.raises(ops.Q4Error) as e:
        ops.matmul(y, dev(x), dev(x), 12, 8)
    assert e.value.status == _lib.Q4_ERR_UNSUPPORTED_SIZE
