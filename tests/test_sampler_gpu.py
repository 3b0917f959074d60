"""Temperature / top-p sampling kernel (q4_sample_topp) against the oracle, and through the model."""
import ctypes as C

import numpy as np
import pytest
import torch

from llama_cu_awq_b200 import ops, synth
from llama_cu_awq_b200.model import Transformer
from oracle import q4_oracle as O
from test_oracle_sampler import select_float64

pytestmark = pytest.mark.gpu


class Mailbox:
    """Pinned host token mailbox + device position, as the sampling kernels expect them (common.h:57-60)."""

    def __init__(self, pos=5):
        self.host = torch.zeros(64, dtype=torch.int32).pin_memory()
        self.host[0] = pos
        self.pos_dev = torch.tensor([pos], dtype=torch.int32, device="cuda")
        self.pos = pos

    def run(self, logits16, temperature, topp, coin):
        d = torch.from_numpy(logits16.view(np.int16).copy()).cuda()
        base = self.host.data_ptr()
        ops.sample_topp(d, logits16.size, temperature, topp, coin, base + 4, base, self.pos_dev)
        torch.cuda.synchronize()
        self.pos += 1
        assert int(self.host[0]) == self.pos and int(self.pos_dev.item()) == self.pos
        return int(self.host[1 + self.pos]), d.cpu().numpy().view(np.float16)


@pytest.mark.parametrize("n", [32000, 1000, 37, 131072])
@pytest.mark.parametrize("topp", [0.9, 0.3, 0.0, 1.0])
def test_sample_topp_kernel(n, topp):
    rng = np.random.default_rng(n + int(topp * 10))
    logits = (rng.standard_normal(n) * 2.5).astype(np.float16)
    same = total = 0
    for temperature in (0.5, 1.0, 2.0):
        for coin in (0.0, 1e-7, 0.25, 0.6180339, 0.99, 0.99999994):
            mb = Mailbox()
            tok, p = mb.run(logits, temperature, topp, coin)
            # bit-exact: the selection rule applied to the probabilities the kernel itself produced
            assert tok == select_float64(p, topp, coin), (temperature, coin)
            ref_tok, ref_p = O.sample_topp(logits, temperature, topp, coin)
            # the probabilities: device expf and the host's differ by an ulp now and then, hence one fp16 step at most
            d = np.abs(p.view(np.int16).astype(np.int32) - ref_p.view(np.int16).astype(np.int32))
            assert d.max() <= 1
            total += 1
            if d.max() == 0:
                assert tok == ref_tok
                same += 1
    assert same >= total // 2   # identical probabilities (and then the identical token) in most cases


def test_sample_topp_threshold_never_reached():
    logits = np.zeros(4096, np.float16)
    logits[7] = np.float16(-20.0)
    for topp in (0.999, 0.0):
        tok, p = Mailbox().run(logits, 1.0, topp, 0.99999994)
        assert tok == select_float64(p, topp, 0.99999994)


@pytest.mark.parametrize("fwd_path", [0, 1, 2])
def test_model_sampling(fwd_path, tmp_path):
    """Through the model: the prompt phase stays greedy hand-off, generated positions are sampled with one coin per
    forward call from the reference's generator, and the mailbox receives the token the selection rule gives for the
    probabilities left in the logits buffer."""
    path = str(tmp_path / "mid.bin")
    synth.write_model_file(path, "mid", seed=11)
    t = Transformer(path)
    if fwd_path == 2:
        assert t.best_path() == 2
    prompt = np.array([1, 99, 1500], np.int32)
    seed, temperature, topp = 42, 0.9, 0.8
    runs = []
    for rep in range(2):
        t.set_sampler(temperature, topp, seed)
        t.reset(prompt, 0)
        coins = O.Rng(seed)
        toks = []
        for pos in range(12):
            gen = pos >= len(prompt) - 1
            t.forward(gen_token=gen, path=fwd_path)
            t.synchronize()
            coin = coins.f32()
            tok = int(t.shared().tokens[pos + 1])
            if gen:
                p = t.logits()
                assert abs(float(p.astype(np.float64).sum()) - 1.0) < 2e-3
                assert tok == select_float64(p, topp, coin), pos
            else:
                assert tok == prompt[pos + 1]
            toks.append(tok)
        runs.append(toks)
    assert runs[0] == runs[1]            # same seed, same tokens
    t.set_sampler(0.0, topp, seed)       # temperature 0: greedy again
    t.reset(prompt, 0)
    for pos in range(6):
        t.forward(gen_token=pos >= 2, path=fwd_path)
        t.synchronize()
        if pos >= 2:
            assert int(t.shared().tokens[pos + 1]) == O.argmax(t.logits())
    assert t.status() == 0
    t.close()
