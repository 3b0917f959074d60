"""The W4 products for a handful of rows (q4_matmul_q4_rows, q4_qkv_matmul_rows, q4_ffn_silu_rows: the projections of
batched decode) against the oracle: every row is what the reference's batch-1 kernels compute for that row of x
(gpu_kernels.h:179-283), within the fp16 tolerance; results are bit-reproducible."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from llama_cu_awq_b200 import _lib, ops, synth
from oracle import q4_oracle as O

pytestmark = pytest.mark.gpu


def _x(rng, M, K):
    return rng.standard_normal((M, K)).astype(np.float16)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("K,N", [(128, 16), (384, 48), (1024, 1024), (2816, 1024), (4096, 4096), (11008, 4096), (4096, 11008)])
def test_matmul_rows(M, K, N):
    """One group to 86 groups (fewer groups than warps, uneven slices), one to many 16-feature tiles, both tile pairings."""
    rng = np.random.default_rng(M + K + N)
    q = synth.synth_qweight(rng, K, N)
    x = _x(rng, M, K)
    W = ops.QWeight.from_numpy(q)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    ops.matmul_rows(y, xd, W, M, K, N)
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    for m in sorted({0, M // 2, M - 1}):
        assert_close(got[m], O.matvec(x[m], q, K, N, order=1), f"row {m} of {M}x{K}x{N}", max_rel=2e-3)
    w = O.dequant(q, K, N).astype(np.float64)
    assert_close(got, x.astype(np.float64) @ w.T, f"{M}x{K}x{N} vs f64", max_rel=2e-3)
    y2 = torch.empty_like(y)
    ops.matmul_rows(y2, xd, W, M, K, N)
    torch.cuda.synchronize()
    assert (y2.cpu().numpy().view(np.uint16) == got.view(np.uint16)).all()


@pytest.mark.parametrize("M", [2, 8, 13])
@pytest.mark.parametrize("gpu_count", [1, 4])
def test_matmul_rows_residual_in_place(M, gpu_count):
    """The accum form (gpu_kernels.h:237-238): y = product + y / gpu_count, written over the residual."""
    K, N = 1408, 1024
    rng = np.random.default_rng(M)
    q = synth.synth_qweight(rng, K, N)
    x = _x(rng, M, K)
    res = rng.standard_normal((M, N)).astype(np.float16)
    W = ops.QWeight.from_numpy(q)
    y = torch.from_numpy(res.copy()).cuda()
    ops.matmul_rows(y, torch.from_numpy(x).cuda(), W, M, K, N, residual=y, residual_scale=1.0 / gpu_count)
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    for m in range(M):
        assert_close(got[m], O.matvec(x[m], q, K, N, y_old=res[m], gpu_count=gpu_count, order=1), f"row {m}", max_rel=2e-3)


@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("K,NQ,NKV", [(1024, 1024, 256), (4096, 4096, 4096), (8192, 1024, 128)])
def test_qkv_rows(M, K, NQ, NKV):
    rng = np.random.default_rng(M + K + NQ)
    qs = [synth.synth_qweight(rng, K, n) for n in (NQ, NKV, NKV)]
    Ws = [ops.QWeight.from_numpy(q) for q in qs]
    x = _x(rng, M, K)
    outs = [torch.full((M, n), float("nan"), dtype=torch.float16, device="cuda") for n in (NQ, NKV, NKV)]
    ops.qkv_matmul_rows(*outs, torch.from_numpy(x).cuda(), *Ws, M, K, NQ, NKV)
    torch.cuda.synchronize()
    for o, q, n, name in zip(outs, qs, (NQ, NKV, NKV), "qkv"):
        got = o.cpu().numpy()
        for m in sorted({0, M - 1}):
            assert_close(got[m], O.matvec(x[m], q, K, n, order=1), f"{name} row {m}", max_rel=2e-3)
        assert_close(got, x.astype(np.float64) @ O.dequant(q, K, n).astype(np.float64).T, f"{name} vs f64", max_rel=2e-3)


@pytest.mark.parametrize("M", [1, 8, 16])
@pytest.mark.parametrize("K,N", [(1024, 2816), (4096, 11008)])
def test_ffn_silu_rows(M, K, N):
    rng = np.random.default_rng(M + K + N)
    gate, up = synth.synth_qweight(rng, K, N), synth.synth_qweight(rng, K, N)
    x = _x(rng, M, K)
    h = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    ops.ffn_silu_rows(h, torch.from_numpy(x).cuda(), ops.QWeight.from_numpy(gate), ops.QWeight.from_numpy(up), M, K, N)
    torch.cuda.synchronize()
    got = h.cpu().numpy()
    for m in sorted({0, M // 2, M - 1}):
        assert_close(got[m], O.ffn_silu(x[m], gate, up, K, N, order=1), f"row {m}", max_rel=2e-3)


def test_rejects_unsupported_arguments():
    rng = np.random.default_rng(0)
    q = synth.synth_qweight(rng, 128, 16)
    W = ops.QWeight.from_numpy(q)
    x = torch.zeros((17, 128), dtype=torch.float16, device="cuda")
    y = torch.zeros((17, 16), dtype=torch.float16, device="cuda")
    L, s = _lib.lib(), ops._stream()
    assert L.q4_matmul_q4_rows(s, ops._p(y), ops._p(x), W.ref, 17, 128, 16, None, 0.0) == _lib.Q4_ERR_INVALID            # more than 16 rows
    assert L.q4_matmul_q4_rows(s, ops._p(y), ops._p(x), W.ref, 0, 128, 16, None, 0.0) == _lib.Q4_ERR_INVALID
    assert L.q4_matmul_q4_rows(s, ops._p(y), ops._p(x), W.ref, 4, 96, 16, None, 0.0) == _lib.Q4_ERR_UNSUPPORTED_SIZE     # K % 128
    assert L.q4_matmul_q4_rows(s, ops._p(y), ops._p(x), W.ref, 4, 128, 8, None, 0.0) == _lib.Q4_ERR_UNSUPPORTED_SIZE     # N % 16
    assert L.q4_qkv_matmul_rows(s, ops._p(y), ops._p(y), ops._p(y), ops._p(x), W.ref, W.ref, W.ref, 4, 128, 16, 16) == _lib.Q4_ERR_UNSUPPORTED_SIZE
