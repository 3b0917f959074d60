"""The llama2_q4 command line (reference flags plus -k token-id file, -g path) on one GPU and, where the box has them,
on all GPUs with -x hybrid (one host thread per GPU, peer pointers exchanged in-process)."""
import os
import re
import subprocess

import numpy as np
import pytest
import torch

from conftest import ROOT
from llama_cu_awq_b200 import synth
from llama_cu_awq_b200.model import Transformer

pytestmark = pytest.mark.gpu
CLI = os.path.join(ROOT, "llama_cu_awq_b200", "llama2_q4")


def run_cli(model, tokens_file, extra, env=None):
    cmd = [CLI, model, "-k", tokens_file, "-n", "24", "-t", "0"] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    return r.stdout


def generated_ids(out):
    """The ids rank 0 streams (the text of a run without a vocabulary file): the line before the blank line and the
    tok/s summary."""
    body = out.split("[GPU:")[0]
    line = [l for l in body.splitlines() if re.fullmatch(r"( \d+)+", l)]
    assert line, out[-800:]
    return [int(v) for v in line[-1].split()]


@pytest.fixture(scope="module")
def model_and_prompt(tmp_path_factory):
    d = tmp_path_factory.mktemp("cli")
    path = str(d / "mid.bin")
    synth.write_model_file(path, "mid", seed=13)
    prompt = np.array([1, 700, 45, 1999], np.int32)
    tf = str(d / "prompt.txt")
    with open(tf, "w") as f:
        f.write(" ".join(str(int(v)) for v in prompt))
    return path, tf, prompt


@pytest.mark.parametrize("fwd_path", [1, 2])
def test_cli_single_gpu_matches_generate(model_and_prompt, fwd_path):
    path, tf, prompt = model_and_prompt
    out = run_cli(path, tf, ["-x", "none", "-g", str(fwd_path)])
    assert "Loading Weights... done!" in out and "Model params:-" in out
    assert re.search(r"\[GPU: 0\] achieved tok/s: [0-9.]+\. Tokens: \d+, seconds: [0-9.e+-]+", out)
    ids = generated_ids(out)
    t = Transformer(path)
    toks, timed, _ = t.generate(prompt, 24, path=fwd_path)
    t.close()
    # the CLI streams tokens[1..]: prompt echo first, then the generated ids (until EOS or -n)
    assert ids == [int(v) for v in toks[1:1 + len(ids)]]
    assert abs(len(ids) - timed) <= 1   # an EOS id is printed but not counted


def test_cli_sampling_is_seeded(model_and_prompt):
    path, tf, _ = model_and_prompt
    a = generated_ids(run_cli(path, tf, ["-x", "none", "-t", "0.9", "-p", "0.8", "-s", "7"]))
    b = generated_ids(run_cli(path, tf, ["-x", "none", "-t", "0.9", "-p", "0.8", "-s", "7"]))
    c = generated_ids(run_cli(path, tf, ["-x", "none", "-t", "0.9", "-p", "0.8", "-s", "8"]))
    assert a == b and a != c


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_cli_column_mode(model_and_prompt):
    """-x column: same arithmetic per output column as one GPU; -g 2 falls back to the CUDA-graph path."""
    path, tf, _ = model_and_prompt
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="0,1")
    out = run_cli(path, tf, ["-x", "column"], env=env)
    assert "[GPU: 0] achieved tok/s" in out and "[GPU: 1] achieved tok/s" in out
    ids = generated_ids(out)
    single = generated_ids(run_cli(path, tf, ["-x", "none", "-g", "1"]))
    assert ids[:4] == single[:4]
    assert sum(int(x == y) for x, y in zip(ids, single)) >= len(single) // 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fwd_path", [1, 2])
def test_cli_hybrid_all_gpus(model_and_prompt, fwd_path):
    """-x hybrid over two GPUs (thread per GPU): every rank reports, and the ids agree with the single-GPU run up to
    fp16 re-association of the sharded sums (TP(g) == TP(1) only up to rounding, so a late id may differ)."""
    path, tf, _ = model_and_prompt
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="0,1")
    out = run_cli(path, tf, ["-x", "hybrid", "-g", str(fwd_path)], env=env)
    assert "[GPU: 0] achieved tok/s" in out and "[GPU: 1] achieved tok/s" in out
    ids = generated_ids(out)
    single = generated_ids(run_cli(path, tf, ["-x", "none", "-g", str(fwd_path)]))
    same = sum(int(x == y) for x, y in zip(ids, single))
    assert same >= len(single) // 2, (ids, single)
    assert ids[:4] == single[:4]


def test_cli_prompt_in_one_pass(model_and_prompt):
    """-b 1: the prompt but its last position through q4_model_prefill; same ids as q4_generate with the same option."""
    path, tf, prompt = model_and_prompt
    out = run_cli(path, tf, ["-x", "none", "-g", "2", "-b", "1"])
    ids = generated_ids(out)
    t = Transformer(path)
    toks, timed, _ = t.generate(prompt, 24, path=2, prompt_one_pass=True)
    t.close()
    assert ids == [int(v) for v in toks[1:1 + len(ids)]]
    assert abs(len(ids) - timed) <= 1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_cli_prompt_in_one_pass_hybrid(model_and_prompt):
    """-b 1 with -x hybrid (thread per GPU): the prompt rows' all-reduce goes through the peer-push kernels; the echoed prompt
    and the first generated ids agree with the single-GPU run of the same option."""
    path, tf, _ = model_and_prompt
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="0,1")
    out = run_cli(path, tf, ["-x", "hybrid", "-g", "2", "-b", "1"], env=env)
    assert "[GPU: 0] achieved tok/s" in out and "[GPU: 1] achieved tok/s" in out
    ids = generated_ids(out)
    single = generated_ids(run_cli(path, tf, ["-x", "none", "-g", "2", "-b", "1"]))
    assert ids[:4] == single[:4]
    assert sum(int(x == y) for x, y in zip(ids, single)) >= len(single) // 2, (ids, single)
