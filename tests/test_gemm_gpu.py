"""The batched / prefill W4 dequant-GEMM on tcgen05 (q4_matmul_q4_batched) against the oracle: every row of Y is the
reference's matmul(QWeight) of that row of X (gpu_kernels.h:179-248), within the fp16 tolerance."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from llama_cu_awq_b200 import ops, synth
from oracle import q4_oracle as O

pytestmark = pytest.mark.gpu


def _case(M, K, N, seed, interleave):
    rng = np.random.default_rng(seed)
    q = synth.synth_qweight(rng, K, N)
    x = rng.standard_normal((M, K)).astype(np.float16)
    W = ops.QWeight.from_numpy(q)
    mm = ops.BatchedMatmul(W, K, N, M, interleave=interleave)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    mm(y, xd, M)
    assert mm.status() == 0
    return q, x, y.cpu().numpy(), mm, xd


@pytest.mark.parametrize("interleave", [True, False])
@pytest.mark.parametrize("M,K,N", [(16, 256, 128), (16, 128, 128), (1, 384, 136), (5, 1024, 8), (17, 640, 264), (64, 2048, 384), (100, 896, 520),
                                    (300, 512, 128)])
def test_small_shapes_against_the_oracle_rows(M, K, N, interleave):
    """Tails everywhere: rows that do not fill a batch tile, features that do not fill a 128-row tile, a last chunk of
    128 inputs, one to several K splits. Each row against the oracle's GEMV in the reference's summation order."""
    q, x, y, _, _ = _case(M, K, N, seed=M * 7 + K + N, interleave=interleave)
    for m in sorted({0, M // 2, M - 1}):
        assert_close(y[m], O.matvec(x[m], q, K, N, order=1), f"row {m} of {M}x{K}x{N}", max_rel=4e-3)
    w = O.dequant(q, K, N).astype(np.float64)     # [N][K], bit-exact dequantised weights
    assert_close(y, x.astype(np.float64) @ w.T, f"{M}x{K}x{N} vs f64", max_rel=4e-3)


@pytest.mark.parametrize("M", [16, 64, 512])
@pytest.mark.parametrize("K,N", [(4096, 12288), (4096, 22016), (11008, 4096), (4096, 4096)])
def test_7b_projection_shapes(M, K, N):
    """The four Llama-2-7B projection shapes (fused QKV, fused gate/up, down, O) at the three batch sizes: a few rows
    against the oracle's GEMV, the whole result against an fp32 product of the bit-exact dequantised weights."""
    q, x, y, mm, xd = _case(M, K, N, seed=K + N + M, interleave=True)
    for m in (0, M - 1):
        assert_close(y[m], O.matvec(x[m], q, K, N, order=0), f"row {m} of {M}x{K}x{N}", max_rel=4e-3)
    torch.backends.cuda.matmul.allow_tf32 = False
    w = torch.from_numpy(O.dequant(q, K, N)).cuda()
    ref = (xd.float() @ w.t()).cpu().numpy()
    assert_close(y, ref, f"{M}x{K}x{N} vs fp32 product", max_rel=4e-3)
    # a second call on the same workspace (tile counters back at zero) and bit-equal results (fixed summation order)
    y2 = torch.empty_like(torch.from_numpy(y)).cuda()
    mm(y2, xd, M)
    assert mm.status() == 0
    assert (y2.cpu().numpy().view(np.uint16) == y.view(np.uint16)).all()


def test_back_to_back_launches_are_bit_reproducible():
    """Forty launches queued back to back on one workspace (their prologues overlap the previous launch's tail through
    programmatic dependent launch): every result equals the first, bit for bit."""
    M, K, N = 512, 4096, 11008
    q, x, y, mm, xd = _case(M, K, N, seed=3, interleave=True)
    first = torch.from_numpy(y).cuda()
    outs = [torch.zeros_like(first) for _ in range(8)]
    for _ in range(5):
        for o in outs:
            mm(o, xd, M)
        torch.cuda.synchronize()
        for o in outs:
            assert torch.equal(o, first)
    assert mm.status() == 0


def test_rejects_unsupported_arguments():
    from llama_cu_awq_b200 import _lib
    rng = np.random.default_rng(0)
    q = synth.synth_qweight(rng, 96, 8)
    W = ops.QWeight.from_numpy(q)
    x = torch.zeros((4, 96), dtype=torch.float16, device="cuda")
    y = torch.zeros((4, 8), dtype=torch.float16, device="cuda")
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    L = _lib.lib()
    s = ops._stream()
    assert L.q4_matmul_q4_batched(s, ops._p(y), ops._p(x), W.ref, None, 4, 96, 8, ops._p(ws), 4096) == _lib.Q4_ERR_UNSUPPORTED_SIZE   # K % 128
    q = synth.synth_qweight(rng, 128, 8)
    W = ops.QWeight.from_numpy(q)
    x = torch.zeros((4, 128), dtype=torch.float16, device="cuda")
    assert L.q4_matmul_q4_batched(s, ops._p(y), ops._p(x), W.ref, None, 4, 128, 8, ops._p(ws), 16) == _lib.Q4_ERR_LIMIT   # workspace too small
    assert L.q4_matmul_q4_batched(s, ops._p(y), ops._p(x), W.ref, None, 0, 128, 8, ops._p(ws), 4096) == _lib.Q4_ERR_INVALID
