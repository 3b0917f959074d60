"""On a GPU box: the reference's own CUDA kernels (built from the reference sources into oracle/_ref/) against
the CPU oracle (bit for bit in its warp order) and against this library (tolerance)."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from llama_cu_awq_b200 import ops, synth
from oracle import q4_oracle as O
from oracle import ref_gpu as R

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not R.available(), reason="oracle/_ref/libref_q4.so not built")]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("K,N", [(256, 16), (384, 8), (4096, 64), (11008, 16), (4096, 4096)])
def test_reference_matvec_vs_oracle_and_library(K, N):
    rng = np.random.default_rng(K + N)
    q = synth.synth_qweight(rng, K, N)
    x = rng.standard_normal(K).astype(np.float16)
    ref = R.matmul_q4(x, q, K, N)
    orc = O.matvec(x, q, K, N, order=1)
    assert (ref.view(np.uint16) == orc.view(np.uint16)).all(), "oracle (warp order) is not bit-identical to mat_vec_kernel_int4"
    y = torch.empty(N, dtype=torch.float16, device="cuda")
    ops.matmul(y, dev(x), ops.QWeight.from_numpy(q), K, N)
    assert_close(y.cpu().numpy(), ref, "library vs reference kernel", max_rel=4e-3)


def test_reference_ffn_and_accum_vs_oracle():
    rng = np.random.default_rng(7)
    K, N = 512, 64
    g, u = synth.synth_qweight(rng, K, N), synth.synth_qweight(rng, K, N)
    x = (rng.standard_normal(K) * 0.25).astype(np.float16)
    ref = R.ffn_matvec_silu(x, g, u, K, N)
    orc = O.ffn_silu(x, g, u, K, N, order=1)
    assert_close(orc, ref, "ffn oracle vs reference", max_rel=1e-3)  # expf differs by an ulp between libm and CUDA
    y0 = rng.standard_normal(N).astype(np.float16)
    ref = R.matmul_q4(x, g, K, N, y_old=y0, gpu_count=2)
    orc = O.matvec(x, g, K, N, y_old=y0, gpu_count=2, order=1)
    assert (ref.view(np.uint16) == orc.view(np.uint16)).all()


def test_reference_model_generation_vs_library(tmp_path):
    path = str(tmp_path / "tiny.bin")
    synth.write_model_file(path, "tiny", seed=0)
    prompt = [1, 17, 300, 45]
    steps = 16
    toks, logits, *_ = R.generate(path, prompt, steps, 512)
    from llama_cu_awq_b200.model import Transformer
    t = Transformer(path)
    # teacher-force the reference's sequence and compare the final logits
    t.reset(toks, 0)
    for pos in range(steps):
        t.forward(gen_token=False, path=1)
    t.synchronize()
    assert_close(t.logits(), logits, "final logits vs reference program")
    t.close()


@pytest.mark.parametrize("topp", [0.9, 0.5, 0.0])
def test_sampler_pick_matches_the_reference_away_from_boundaries(topp):
    """q4_sample_topp against the reference's own sample() (sampler.h:77-115: softmax kernel, radix sort, fp16 prefix
    sum, threshold search) on the same logits, temperature, top-p and seed. The reference accumulates its prefix sum
    in fp16 in an order the library leaves open, so only cases are compared where the threshold lies clear of the
    picked element's boundaries (in exact arithmetic); those must agree, and they must be the large majority."""
    from test_oracle_sampler import select_float64
    from test_sampler_gpu import Mailbox
    n = 32000
    compared = agreed = 0
    for seed in range(1, 25):
        rng = np.random.default_rng(seed)
        logits = rng.standard_normal(n)
        logits[rng.choice(n, 12, replace=False)] += rng.uniform(8.0, 12.0, 12)   # a dozen dominant tokens hold most of the mass
        logits = logits.astype(np.float16)
        temperature = (0.7, 1.0, 1.3)[seed % 3]
        ref_tok, coin = R.sample(logits, temperature, topp, seed)
        tok, p = Mailbox().run(logits, temperature, topp, coin)
        assert tok == select_float64(p, topp, coin)
        # distance of the threshold from the nearest prefix-sum boundary of the picked element, in exact arithmetic
        pf = p.astype(np.float64)
        order = np.argsort(-pf, kind="stable") if 0.0 < topp < 1.0 else np.arange(n)
        cum = np.cumsum(pf[order])
        thr = coin * topp if 0.0 < topp < 1.0 else coin
        k = int(np.nonzero(order == tok)[0][0])
        margin = min(cum[k] - thr, thr - (cum[k - 1] if k > 0 else 0.0))
        if margin < 6e-3:      # fp16 running sums near 0.5-1.0 carry steps of 5e-4-1e-3: too close to call
            continue
        compared += 1
        agreed += int(tok == ref_tok)
    assert compared >= 8
    assert agreed == compared, (agreed, compared)
