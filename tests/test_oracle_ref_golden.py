"""CPU test: the oracle against outputs of the reference's own CUDA kernels, recorded on a B200
(tests/golden/ref_kernels_sm100.npz, made by tests/golden/make_ref_golden.py)."""
import importlib.util
import os

import numpy as np
import pytest

from conftest import GOLDEN, assert_close
from llama_cu_awq_b200 import synth
from oracle import q4_oracle as O

PATH = os.path.join(GOLDEN, "ref_kernels_sm100.npz")
pytestmark = pytest.mark.skipif(not os.path.exists(PATH), reason="reference-kernel fixture not recorded yet")

spec = importlib.util.spec_from_file_location("make_ref_golden", os.path.join(GOLDEN, "make_ref_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)


@pytest.fixture(scope="module")
def gold():
    return np.load(PATH)


def bits(a):
    return np.asarray(a).view(np.uint16)


def ulp_distance(a, b):
    """Distance in fp16 steps (sign-magnitude bits mapped onto a monotonic integer line)."""
    def key(x):
        u = bits(x).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u)
    return np.abs(key(a) - key(b)).max()


def test_matvec_bit_exact(gold):
    for K, N, seed in G.MATVEC:
        q, x, y0 = G.matvec_inputs(K, N, seed)
        assert (bits(x) == bits(gold[f"in_x_{K}_{N}"])).all(), "random stream differs from the one the fixture was made with"
        assert (bits(O.matvec(x, q, K, N, order=1)) == bits(gold[f"matvec_{K}_{N}"])).all(), (K, N)
        assert (bits(O.matvec(x, q, K, N, y_old=y0, gpu_count=4, order=1)) == bits(gold[f"matvec_accum4_{K}_{N}"])).all(), (K, N)
        assert_close(O.matvec(x, q, K, N, order=0), gold[f"matvec_{K}_{N}"], "fast order", max_rel=1e-3)


def test_ffn_rms_rope_mha_f16(gold):
    for K, N, seed in G.FFN:
        g, u, x = G.ffn_inputs(K, N, seed)
        assert_close(O.ffn_silu(x, g, u, K, N, order=1), gold[f"ffn_{K}_{N}"], "ffn", max_rel=1e-3)
    for n, seed in G.RMS:
        x, w = G.rms_inputs(n, seed)
        o = O.rmsnorm(x, w)
        assert ulp_distance(o, gold[f"rms_{n}"]) <= 1
    for heads, kvh, hs, pos, seed in G.ROPE:
        q, kc = G.rope_inputs(heads, kvh, hs, pos, seed)
        row = slice(pos * kvh * hs, (pos + 1) * kvh * hs)
        qo, ko = O.rope(q, kc[row], heads, kvh, hs, pos, 10000.0)
        assert_close(qo, gold[f"rope_q_{heads}_{hs}_{pos}"], "rope q", max_rel=2e-3)
        assert_close(ko, gold[f"rope_k_{heads}_{hs}_{pos}"], "rope k", max_rel=2e-3)
        assert bool(gold[f"rope_k_untouched_{heads}_{hs}_{pos}"])
    for heads, kv_mul, hs, pos, seed in G.MHA:
        q, kc, vc = G.mha_inputs(heads, kv_mul, hs, pos, seed)
        assert_close(O.attention(q, kc, vc, heads, hs, kv_mul, pos), gold[f"mha_{heads}_{kv_mul}_{hs}_{pos}"], "mha", max_rel=2e-3)
    for n, d, seed in G.F16:
        W, x = G.f16_inputs(n, d, seed)
        assert (bits(O.matvec_f16(x, W, n, d, order=1)) == bits(gold[f"f16_{n}_{d}"])).all()


def test_model_tokens_and_logits(gold, tmp_path):
    cfg, seed, prompt, steps = G.MODEL
    path = str(tmp_path / "m.bin")
    synth.write_model_file(path, cfg, seed=seed)
    m = O.Model(open(path, "rb").read())
    toks = [int(t) for t in gold["model_tokens"]]
    assert toks[: len(prompt)] == prompt
    for pos in range(steps):
        nxt = m.forward(toks[pos], pos, order=1)
        if pos + 1 >= len(prompt) and nxt != toks[pos + 1]:
            lg = np.sort(m.logits().astype(np.float32))
            assert lg[-1] - lg[-2] < 5e-2, f"token mismatch at {pos} with a clear margin"
    assert_close(m.logits(), gold["model_last_logits"], "last logits vs reference program", max_rel=5e-3)
