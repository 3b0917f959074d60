"""The fused decode kernel (forward path 2) beyond plain logits parity: run-to-run bit reproducibility, parity on the
7B layer shapes, the block-fixed-point activation staging on hostile inputs, expiry of a bounded device-side wait,
and recovery from a failed set-up. The last three use the test build of the library (libq4b200_test.so)."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import assert_close
from llama_cu_awq_b200 import _lib, ops, synth
from llama_cu_awq_b200.model import Transformer
from oracle import q4_oracle as O

pytestmark = pytest.mark.gpu


class _DevView:
    """A device pointer as something torch.as_tensor accepts (CUDA array interface)."""

    def __init__(self, ptr, n, typestr="<f2"):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (int(ptr), False), "version": 2}


@pytest.fixture(scope="module")
def model_4l(tmp_path_factory):
    p = tmp_path_factory.mktemp("models") / "llama2-7b-4l.bin"
    synth.write_model_file(str(p), "llama2-7b-4l", seed=0)
    return str(p)


def _run(t, tokens, queued):
    """Teacher-forced logits at every position. queued: all launches and stream-ordered logits copies are enqueued
    without any host synchronisation in between; else the host waits for every token."""
    vocab, n = t.config.vocab_size, len(tokens)
    src = torch.as_tensor(_DevView(t.logits_device_ptr(), vocab), device="cuda")
    keep = torch.empty((n, vocab), dtype=torch.float16, device="cuda")
    t.reset(tokens, 0)
    with torch.cuda.stream(t.stream):
        for pos in range(n):
            t.forward(gen_token=False, path=2)
            keep[pos].copy_(src, non_blocking=True)
            if not queued:
                t.synchronize()
    t.synchronize()
    assert t.status() == 0
    return keep.cpu().numpy()


def test_fused_path_is_bit_reproducible(model_4l):
    """The same 64 positions through path 2, once queued back to back and once with a host wait per token, and a third
    time in a fresh model object: every logit of every position must come out with identical bits (no sum may depend on
    the order in which other CTAs' results happen to arrive)."""
    tokens = np.random.default_rng(3).integers(3, 32000, size=64, dtype=np.int32)
    t = Transformer(model_4l)
    assert t.best_path() == 2
    a = _run(t, tokens, queued=True)
    b = _run(t, tokens, queued=False)
    c = _run(t, tokens, queued=True)
    t.close()
    t2 = Transformer(model_4l)
    d = _run(t2, tokens, queued=False)
    t2.close()
    for name, other in (("queued vs synchronised", b), ("queued, second run", c), ("fresh model", d)):
        diff = np.nonzero((a.view(np.uint16) != other.view(np.uint16)).any(axis=1))[0]
        assert diff.size == 0, f"{name}: logits differ first at position {diff[0]}"


def test_fused_path_parity_on_7b_layer_shapes(model_4l):
    """Four layers with the 7B matrix shapes and the 32000-row classifier against the oracle, 8 teacher-forced positions."""
    tokens = np.random.default_rng(5).integers(3, 32000, size=8, dtype=np.int32)
    t = Transformer(model_4l)
    assert t.best_path() == 2
    got = _run(t, tokens, queued=False)
    t.close()
    m = O.Model(open(model_4l, "rb").read())
    for pos, tok in enumerate(tokens):
        m.forward(int(tok), pos, order=0)
        assert_close(got[pos], m.logits(), f"7B-shaped 4-layer model, pos {pos}")
    m.close()


def _hostile(kind, K, rng):
    x = rng.standard_normal(K).astype(np.float32)
    G = (K + 127) // 128
    if kind == "outlier100" or kind == "outlier1000":
        f = 100.0 if kind == "outlier100" else 1000.0
        for g in range(G):   # one outlier per group of 128: its 127 neighbours share its block scale
            x[g * 128 + int(rng.integers(0, min(128, K - g * 128)))] *= f
        if kind == "outlier1000":
            x *= 0.05        # keep the dot products inside fp16
    elif kind == "zero_groups":
        for g in range(0, G, 3):
            x[g * 128:(g + 1) * 128] = 0.0
    elif kind == "subnormal":
        x *= 2.0 ** -20      # most elements are fp16 subnormals
        x[::128] = 1.0
    elif kind == "fp16_max":
        x *= 1e-3
        x[5::256] = 65504.0
        x[133::256] = -65504.0
    return x.astype(np.float16)


@pytest.mark.parametrize("K,N", [(4096, 64), (11008, 32)])
@pytest.mark.parametrize("kind", ["normal", "outlier100", "outlier1000", "zero_groups", "subnormal", "fp16_max"])
def test_block_fixed_point_activations(kind, K, N):
    """gemv_slot replaces the reference's fp16 x fp32 FMA (gpu_kernels.h:203-208) by an integer dot product over a
    per-group 15-bit fixed-point copy of x. Hostile activation vectors must stay inside the fp16 tolerance."""
    L = _lib.test_lib()
    rng = np.random.default_rng(K + len(kind))
    q = synth.synth_qweight(rng, K, N)
    if kind == "fp16_max":
        q["scales"] = (q["scales"].astype(np.float32) * 0.01).astype(np.float16)   # keep |y| below 65504
    x = _hostile(kind, K, rng)
    W = ops.QWeight.from_numpy(q)
    xd = torch.from_numpy(x).cuda()
    y = torch.full((N,), float("nan"), dtype=torch.float16, device="cuda")
    st = L.q4_test_fused_gemv(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(y.data_ptr()), C.c_void_p(xd.data_ptr()), W.ref, K, N)
    assert st == 0
    ref = O.matvec(x, q, K, N, order=1)
    assert np.isfinite(ref.astype(np.float32)).all()
    assert_close(y.cpu().numpy(), ref, f"{kind} {K}x{N}")
    # and against the unrounded sum: the fixed-point step must not cost more than the reference's own fp16 output rounding
    assert_close(y.cpu().numpy(), O.matvec_f32(x, q, K, N), f"{kind} {K}x{N} vs f64", max_rel=4e-3)


def test_fused_attention_splits(tmp_path):
    """Heads split over several CTAs (long contexts): forced here with a tiny split length (test build)."""
    L = _lib.test_lib()
    path = str(tmp_path / "mid_gqa.bin")
    synth.write_model_file(path, "mid-gqa", seed=3)
    tokens = np.random.default_rng(9).integers(3, 2048, size=60, dtype=np.int32)
    L.q4_test_set_split_len(8)
    try:
        t = Transformer(path, lib=L)
        assert t.best_path() == 2
        got = _run(t, tokens, queued=False)
        t.close()
    finally:
        L.q4_test_set_split_len(0)
    m = O.Model(open(path, "rb").read())
    for pos, tok in enumerate(tokens):
        m.forward(int(tok), pos, order=1)
        if pos in (0, 7, 8, 9, 23, 24, 25, 40, 59):
            assert_close(got[pos], m.logits(), f"split attention, pos {pos}")


def test_fused_wait_runs_out_and_the_path_recovers(tmp_path):
    """A rank of a 2-rank tensor-parallel group whose peer never runs: the peer's exchange area is a second local
    allocation that nobody writes. The kernel's wait for the peer's partial sums ends after the (shortened) limit with
    Q4_ERR_TIMEOUT, the context stays usable, q4_model_reset re-arms the path, and with the exchange kept local (test
    switch) the same rank then reproduces, bit for bit, the logits it produced before the time-out."""
    L = _lib.test_lib()
    path = str(tmp_path / "mid.bin")
    synth.write_model_file(path, "mid", seed=2)
    a, b = C.c_void_p(), C.c_void_p()
    assert L.q4_comm_create_local(C.byref(a), 2, 0) == 0 and L.q4_comm_create_local(C.byref(b), 2, 1) == 0
    assert L.q4_test_comm_set_peer(a, 1, b) == 0
    tokens = np.random.default_rng(1).integers(3, 2048, size=4, dtype=np.int32)
    t = Transformer(path, rank=0, gpu_count=2, tp_mode=_lib.Q4_TP_HYBRID, comm=a, lib=L)
    assert t.best_path() == 2
    t.set_wait_limit_ns(20_000_000)   # 20 ms instead of 2 s
    try:
        L.q4_test_set_fused_debug(16)          # exchange kept local: this rank alone, zeros as the peer's partials
        before = _run(t, tokens, queued=False)
        L.q4_test_set_fused_debug(0)           # now the kernel waits for rank 1, which does not exist
        t.reset(tokens, 0)
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(t.stream):
            t0.record(t.stream)
            t.forward(gen_token=False, path=2)
            t1.record(t.stream)
        t.synchronize()
        assert t.status() == _lib.Q4_ERR_TIMEOUT
        assert t0.elapsed_time(t1) < 1000.0    # gave up after the limit (a few waits of 20-40 ms), not after seconds
        L.q4_test_set_fused_debug(16)
        after = _run(t, tokens, queued=False)  # reset re-arms; status is clean again (asserted inside)
        assert (before.view(np.uint16) == after.view(np.uint16)).all()
    finally:
        L.q4_test_set_fused_debug(0)
        t.close()
        L.q4_comm_destroy(a)
        L.q4_comm_destroy(b)


def test_all_reduce_wait_runs_out():
    """q4_all_reduce on a 2-rank communicator whose second rank never calls: the kernel stores into the (valid, local)
    stand-in inbox, waits for the missing flag until the limit, records Q4_ERR_TIMEOUT and returns; after q4_comm_reset
    the status is clean."""
    L = _lib.test_lib()
    a, b = C.c_void_p(), C.c_void_p()
    assert L.q4_comm_create_local(C.byref(a), 2, 0) == 0 and L.q4_comm_create_local(C.byref(b), 2, 1) == 0
    assert L.q4_test_comm_set_peer(a, 1, b) == 0
    assert L.q4_comm_set_wait_limit_ns(a, 20_000_000) == 0
    buf = torch.ones(4096, dtype=torch.float16, device="cuda")
    s = torch.cuda.current_stream()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record(s)
    assert L.q4_all_reduce(a, C.c_void_p(s.cuda_stream), C.c_void_p(buf.data_ptr()), 4096) == 0
    e1.record(s)
    torch.cuda.synchronize()
    assert L.q4_comm_status(a) == _lib.Q4_ERR_TIMEOUT
    assert 15.0 < e0.elapsed_time(e1) < 500.0
    assert L.q4_comm_reset(a) == 0 and L.q4_comm_status(a) == 0
    L.q4_comm_destroy(a)
    L.q4_comm_destroy(b)


def test_failed_prepare_leaves_no_half_built_state(tmp_path):
    """An allocation that fails in the middle of q4_model_prepare (injected on the host) must not leave a state that a
    later call takes for ready: the call reports the error, the next call builds from scratch and the model works."""
    L = _lib.test_lib()
    path = str(tmp_path / "tiny_gqa.bin")
    synth.write_model_file(path, "tiny-gqa", seed=1)
    tokens = np.random.default_rng(2).integers(3, 512, size=6, dtype=np.int32)
    ref = Transformer(path, lib=L)
    assert ref.best_path() == 2
    want = _run(ref, tokens, queued=False)
    ref.close()
    for fail_at in (0, 3, 9, 20):
        t = Transformer(path, lib=L)
        L.q4_test_fail_fused_alloc(fail_at)
        assert L.q4_model_prepare(t.h, 2) == _lib.Q4_ERR_CUDA
        assert L.q4_model_prepare(t.h, 2) == 0          # the injector fires once; this call starts over
        got = _run(t, tokens, queued=False)
        assert (got.view(np.uint16) == want.view(np.uint16)).all()
        t.close()
    L.q4_test_fail_fused_alloc(-1)


def test_model_api_rejects_out_of_range_ids_and_positions(tmp_path):
    L = _lib.lib()
    path = str(tmp_path / "tiny.bin")
    synth.write_model_file(path, "tiny", seed=0)
    t = Transformer(path)
    bad = np.array([1, 512, 3], np.int32)            # vocabulary is 512
    assert L.q4_model_reset(t.h, bad.ctypes.data_as(C.POINTER(C.c_int)), 3, 0) == _lib.Q4_ERR_INVALID
    neg = np.array([1, -7], np.int32)
    assert L.q4_model_reset(t.h, neg.ctypes.data_as(C.POINTER(C.c_int)), 2, 0) == _lib.Q4_ERR_INVALID
    seq = synth.CONFIGS["tiny"][6]
    ok = np.ones(seq, np.int32)
    t.reset(ok, 0)
    for _ in range(seq):
        t.forward(gen_token=False, path=1)
    t.synchronize()
    # the cache is full: one more call would write row seq_len
    assert L.q4_model_forward(t.h, C.c_void_p(t.stream.cuda_stream), 0, 1) == _lib.Q4_ERR_LIMIT
    t.close()
