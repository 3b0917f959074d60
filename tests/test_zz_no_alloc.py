"""q4_attention_static: the attention entry point for callers that cannot allocate device memory (hosts with all
device memory handed out at start-up, plugins that only receive the owning runtime's pointers). Its scratch is a
fixed array inside the library. Checked against q4_attention, which takes a caller-owned scratch buffer, on two
calls in a row (the array keeps the previous call's contents, which must not matter)."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import assert_close
from llama_cu_awq_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_both(heads, kv_mul, hs, pos, seed):
    rng = np.random.default_rng(seed)
    stride = heads * hs // kv_mul
    q = dev(rng.standard_normal(heads * hs).astype(np.float16))
    kc = dev((rng.standard_normal((pos + 1, stride)) * 0.5).astype(np.float16))
    vc = dev(rng.standard_normal((pos + 1, stride)).astype(np.float16))
    pd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    ref = torch.empty(heads * hs, dtype=torch.float16, device="cuda")
    ops.MultiHeadAttention(ref, q, kc, vc, ops.attention_scratch(heads, hs), heads, hs, kv_mul, pos + 1, pd)
    out = torch.full((heads * hs,), float("nan"), dtype=torch.float16, device="cuda")
    L = _lib.lib()
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = L.q4_attention_static(s, C.c_void_p(out.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(kc.data_ptr()), C.c_void_p(vc.data_ptr()),
                               heads, hs, kv_mul, pos + 1, C.c_void_p(pd.data_ptr()))
    assert st == _lib.Q4_OK
    torch.cuda.synchronize()
    return out.cpu().numpy(), ref.cpu().numpy()


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    # two different problems back to back: the second call finds the first call's partials in the array
    for heads, kv_mul, hs, pos, seed in [(32, 1, 128, 300, 1), (8, 4, 128, 37, 2)]:
        out, ref = run_both(heads, kv_mul, hs, pos, seed)
        assert_close(out, ref, f"static vs caller scratch ({heads} heads, pos {pos})")
        assert (out.view(np.uint16) == ref.view(np.uint16)).all()  # same kernels, same arithmetic


def test_static_call_allocates_and_frees_nothing():
    """The advertised property: after the first call on a device (which looks the array's address up once), a call leaves
    the device's free memory exactly where it was - nothing is allocated, nothing is freed. head_size 64 rides along."""
    out, ref = run_both(16, 2, 64, 90, 3)     # first use of this shape; also the head_size 64 case
    assert (out.view(np.uint16) == ref.view(np.uint16)).all()
    rng = np.random.default_rng(5)
    heads, kv_mul, hs, pos = 32, 1, 128, 200
    q = dev(rng.standard_normal(heads * hs).astype(np.float16))
    kc = dev((rng.standard_normal((pos + 1, heads * hs)) * 0.5).astype(np.float16))
    vc = dev(rng.standard_normal((pos + 1, heads * hs)).astype(np.float16))
    pd = torch.tensor([pos], dtype=torch.int32, device="cuda")
    out = torch.empty(heads * hs, dtype=torch.float16, device="cuda")
    L = _lib.lib()
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = (s, C.c_void_p(out.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(kc.data_ptr()), C.c_void_p(vc.data_ptr()), heads, hs, kv_mul, pos + 1,
            C.c_void_p(pd.data_ptr()))
    assert L.q4_attention_static(*args) == _lib.Q4_OK
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert L.q4_attention_static(*args) == _lib.Q4_OK
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before


def test_static_scratch_rejects_oversized_shapes():
    L = _lib.lib()
    heads, hs = 1024, 256
    assert L.q4_attention_scratch_bytes(heads, hs) > 256 * 1024
    x = torch.zeros(8, dtype=torch.float16, device="cuda")
    pd = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = C.c_void_p(x.data_ptr())
    st = L.q4_attention_static(C.c_void_p(torch.cuda.current_stream().cuda_stream), p, p, p, p, heads, hs, 1, 8, C.c_void_p(pd.data_ptr()))
    assert st == _lib.Q4_ERR_LIMIT
