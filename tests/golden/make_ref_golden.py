"""Runs the reference's own CUDA kernels (oracle/_ref/libref_q4.so, built from the reference sources by
oracle/Makefile) on seeded inputs on a GPU box and stores their outputs:

    python tests/golden/make_ref_golden.py <out.npz>

The committed copy, tests/golden/ref_kernels_sm100.npz, pins the CPU oracle to the reference's arithmetic:
tests/test_oracle_ref_golden.py regenerates the same inputs from the seeds (cases() below) and compares.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from llama_cu_awq_b200 import synth  # noqa: E402

MATVEC = [(256, 16, 0), (384, 8, 1), (1024, 24, 2), (4096, 64, 3), (11008, 8, 4), (640, 16, 5)]
FFN = [(256, 8, 10), (4096, 32, 11)]
RMS = [(256, 20), (4096, 21), (5120, 22)]
ROPE = [(4, 2, 128, 37, 30), (8, 8, 64, 500, 31)]
MHA = [(4, 1, 128, 37, 40), (8, 4, 128, 300, 41), (2, 1, 64, 0, 42)]
F16 = [(256, 40, 50), (4096, 104, 51)]
MODEL = ("tiny", 0, [1, 17, 300, 45], 16)  # config, seed, prompt, steps


def matvec_inputs(K, N, seed):
    rng = np.random.default_rng(seed)
    return synth.synth_qweight(rng, K, N), rng.standard_normal(K).astype(np.float16), (rng.standard_normal(N) * 4).astype(np.float16)


def ffn_inputs(K, N, seed):
    rng = np.random.default_rng(seed)
    return synth.synth_qweight(rng, K, N), synth.synth_qweight(rng, K, N), (rng.standard_normal(K) * 0.25).astype(np.float16)


def rms_inputs(n, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(n) * 3).astype(np.float16), rng.uniform(0.5, 1.5, n).astype(np.float16)


def rope_inputs(heads, kv_heads, hs, pos, seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal(heads * hs).astype(np.float16), rng.standard_normal((pos + 1) * kv_heads * hs).astype(np.float16)


def mha_inputs(heads, kv_mul, hs, pos, seed):
    rng = np.random.default_rng(seed)
    stride = heads * hs // kv_mul
    return (rng.standard_normal(heads * hs).astype(np.float16), (rng.standard_normal((pos + 1, stride)) * 0.5).astype(np.float16),
            rng.standard_normal((pos + 1, stride)).astype(np.float16))


def f16_inputs(n, d, seed):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((d, n)) * 0.02).astype(np.float16), rng.standard_normal(n).astype(np.float16)


def main(out_path):
    from oracle import ref_gpu as R
    out = {}
    for K, N, seed in MATVEC:
        q, x, y0 = matvec_inputs(K, N, seed)
        out[f"matvec_{K}_{N}"] = R.matmul_q4(x, q, K, N)
        out[f"matvec_accum4_{K}_{N}"] = R.matmul_q4(x, q, K, N, y_old=y0, gpu_count=4)
        out[f"in_x_{K}_{N}"] = x  # guards against a different random stream when the test regenerates inputs
    for K, N, seed in FFN:
        g, u, x = ffn_inputs(K, N, seed)
        out[f"ffn_{K}_{N}"] = R.ffn_matvec_silu(x, g, u, K, N)
    for n, seed in RMS:
        x, w = rms_inputs(n, seed)
        out[f"rms_{n}"] = R.rmsnorm(x, w)
    for heads, kvh, hs, pos, seed in ROPE:
        q, kc = rope_inputs(heads, kvh, hs, pos, seed)
        qo, ko = R.rope(q, kc, heads, kvh, hs, pos, 0, 10000.0)
        row = slice(pos * kvh * hs, (pos + 1) * kvh * hs)
        out[f"rope_q_{heads}_{hs}_{pos}"] = qo
        out[f"rope_k_{heads}_{hs}_{pos}"] = ko[row]  # the rotated cache row; every other row must be untouched
        out[f"rope_k_untouched_{heads}_{hs}_{pos}"] = np.array((ko[: row.start].view(np.uint16) == kc[: row.start].view(np.uint16)).all())
    for heads, kv_mul, hs, pos, seed in MHA:
        q, kc, vc = mha_inputs(heads, kv_mul, hs, pos, seed)
        out[f"mha_{heads}_{kv_mul}_{hs}_{pos}"] = R.mha(q, kc, vc, heads, hs, kv_mul, pos)
    for n, d, seed in F16:
        W, x = f16_inputs(n, d, seed)
        out[f"f16_{n}_{d}"] = R.matmul_f16(x, W, n, d)
    cfg, seed, prompt, steps = MODEL
    path = "/tmp/ref_golden_model.bin"
    synth.write_model_file(path, cfg, seed=seed)
    toks, logits, *_ = R.generate(path, prompt, steps, synth.CONFIGS[cfg][5])
    out["model_tokens"] = toks
    out["model_last_logits"] = logits
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1])
