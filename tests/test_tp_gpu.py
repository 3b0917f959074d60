"""Tensor-parallel decode on 2 (or more) GPUs of one box: one process per GPU over torchrun, peer-memory
all-reduce. Skipped on boxes with a single GPU."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import ROOT
from llama_cu_awq_b200 import synth

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _run_tp(cfg, fwd_path, n, tmp_path, mode="hybrid", extra=""):
    path = str(tmp_path / f"{cfg}.bin")
    if extra == "synthetic":
        synth.write_counter_model_file(path, cfg, seed=7)
    else:
        synth.write_model_file(path, cfg, seed=7)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + fwd_path + (10 if cfg == "mid" else 20) + 40 * (n - 2) + (5 if mode == "column" else 0) + {"": 0, "synthetic": 100, "nccl": 200, "prefill": 300, "prefill-p2p": 350, "batch": 400, "collectives": 450}[extra]),
           os.path.join(ROOT, "tests", "tp_worker.py"), cfg, path, str(fwd_path), mode, extra]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ranks identical: True" in r.stdout


@pytest.mark.parametrize("cfg", ["mid", "mid-gqa"])
@pytest.mark.parametrize("fwd_path", [0, 1, 2])
def test_tp2_logits_match_single_gpu_oracle(cfg, fwd_path, tmp_path):
    _run_tp(cfg, fwd_path, 2, tmp_path)


@pytest.mark.parametrize("cfg", ["mid", "mid-gqa"])
@pytest.mark.parametrize("fwd_path", [0, 1])
def test_tp2_column_mode(cfg, fwd_path, tmp_path):
    """-x column (llama2_q4.cu:479-493, 510-524): all matrices split by output columns, four all-gathers per layer."""
    _run_tp(cfg, fwd_path, 2, tmp_path, mode="column")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("fwd_path", [1, 2])
def test_tp4_logits_match_single_gpu_oracle(fwd_path, tmp_path):
    """Uneven row split: the 22 groups of the down projection fall 6, 6, 5, 5 on the four ranks."""
    _run_tp("mid", fwd_path, 4, tmp_path)


def test_tp2_device_generated_shards(tmp_path):
    """Shards generated on the device by each rank (q4_model_create_synthetic) form the same model as the packed file
    of the same generator: TP2 logits against the single-GPU oracle run on that file."""
    _run_tp("mid", 2, 2, tmp_path, extra="synthetic")


@pytest.mark.parametrize("mode", ["hybrid", "column"])
def test_tp2_nccl_backend(mode, tmp_path):
    """The per-op paths with their collectives routed through NCCL (the reference's -DENABLE_NCCL build)."""
    _run_tp("mid", 0, 2, tmp_path, mode=mode, extra="nccl")


@pytest.mark.parametrize("extra", ["prefill", "prefill-p2p"])
def test_tp2_prefill(extra, tmp_path):
    """Prompt prefill on two ranks: the [rows x dim] all-reduces go through NCCL (backend AUTO picks it for large messages)
    or, without NCCL attached, through the peer push in pieces; decoding then goes on through the fused path."""
    _run_tp("mid-gqa", 2, 2, tmp_path, extra=extra)


def test_tp2_batched_decode(tmp_path):
    """Three sequences decoded together on two ranks (skinny W4 kernels + peer-push all-reduce inside the step graph)."""
    _run_tp("mid-gqa", 2, 2, tmp_path, extra="batch")


def test_tp2_collectives_short_and_long_vectors(tmp_path):
    """The peer-push all-reduce on 16-byte to 256 KB vectors (one CTA / several CTAs, interleaved) and the all-gather."""
    _run_tp("mid", 0, 2, tmp_path, extra="collectives")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp4_collectives_short_and_long_vectors(tmp_path):
    _run_tp("mid", 0, 4, tmp_path, extra="collectives")
