"""Host-side mirror of the reference's op wrappers (llama2_q4.cu:347-427, sampler.h:77-84) over the C ABI.

Same names, argument meaning and order as the reference's free functions, minus the leading `rank`
(the reference uses it only to pick `streams[rank].stream`; here the stream is torch's current stream
unless one is passed). Arguments are torch CUDA tensors (fp16 activations, int32 packed weights); torch
only provides the device memory and the stream. Where the reference prints "Unsupported matmul size.
Exiting" and exits, these raise Q4Error with status Q4_ERR_UNSUPPORTED_SIZE.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import Q4Error, check, q4_qweight  # noqa: F401


def _stream(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


class QWeight:
    """One quantized K x N matrix on the device (common.h:26-30): weight int32[N][4*ceil(K/32)],
    zeros int32[N][ceil(ceil(K/128)/8)], scales fp16[N][ceil(K/128)]."""

    def __init__(self, weight, zeros, scales):
        assert weight.dtype == torch.int32 and zeros.dtype == torch.int32 and scales.dtype == torch.float16
        assert weight.is_cuda and weight.is_contiguous() and zeros.is_contiguous() and scales.is_contiguous()
        self.weight, self.zeros, self.scales = weight, zeros, scales
        self.c = q4_qweight(weight.data_ptr(), zeros.data_ptr(), scales.data_ptr())

    @classmethod
    def from_numpy(cls, d, device="cuda"):
        return cls(torch.from_numpy(d["weight"].view("int32")).to(device), torch.from_numpy(d["zeros"].view("int32")).to(device),
                   torch.from_numpy(d["scales"]).to(device))

    @property
    def ref(self):
        return C.byref(self.c)


def rmsnorm(o, x, weight, size, stream=None):
    check(_lib.lib().q4_rmsnorm(_stream(stream), _p(o), _p(x), _p(weight), size), "rmsnorm")


def matmul(xout, x, w, inpSize, opSize, accum=False, gpu_count=1, loff=-1, pPos=None, alpha=1.0, stream=None):
    """matmul(): quantized form when `w` is a QWeight (llama2_q4.cu:367), fp16 form otherwise (:357)."""
    if isinstance(w, QWeight):
        check(_lib.lib().q4_matmul_q4(_stream(stream), _p(xout), _p(x), w.ref, inpSize, opSize, int(bool(accum)), gpu_count, loff, _p(pPos)),
              "matmul")
    else:
        check(_lib.lib().q4_matmul_f16(_stream(stream), _p(xout), _p(x), _p(w), inpSize, opSize, alpha), "matmul")


def qkv_matvec(q, key_cache, value_cache, x, qw, kw, vw, inpSize, opSize, loff, pPos, kvSize=None, stream=None):
    check(_lib.lib().q4_qkv_matvec(_stream(stream), _p(q), _p(key_cache), _p(value_cache), _p(x), qw.ref, kw.ref, vw.ref, inpSize, opSize,
                                   opSize if kvSize is None else kvSize, loff, _p(pPos)), "qkv_matvec")


def ffn_matvec_silu(xout, x, gate_w, up_w, inpSize, opSize, stream=None):
    check(_lib.lib().q4_ffn_matvec_silu(_stream(stream), _p(xout), _p(x), gate_w.ref, up_w.ref, inpSize, opSize), "ffn_matvec_silu")


def RoPERotation(q, k, num_heads, num_kv_heads, head_size, pPos, loff, rope_theta, stream=None):
    check(_lib.lib().q4_rope(_stream(stream), _p(q), _p(k), num_heads, num_kv_heads, head_size, _p(pPos), loff, rope_theta), "RoPERotation")


def attention_scratch(num_heads, head_size, device="cuda"):
    n = _lib.lib().q4_attention_scratch_bytes(num_heads, head_size)
    return torch.empty(n, dtype=torch.uint8, device=device)


def MultiHeadAttention(output, q, key_cache, value_cache, att, num_heads, head_size, kv_mul, max_seq_len, pPos, stream=None):
    """`att` is the scratch buffer from attention_scratch() (the reference passes its score buffer there)."""
    check(_lib.lib().q4_attention(_stream(stream), _p(output), _p(q), _p(key_cache), _p(value_cache), _p(att), num_heads, head_size, kv_mul,
                                  max_seq_len, _p(pPos)), "MultiHeadAttention")


def copy_embedding(x, table, dim, tokens_ptr, pPos, stream=None):
    check(_lib.lib().q4_embed(_stream(stream), _p(x), _p(table), dim, C.c_void_p(tokens_ptr), _p(pPos)), "copy_embedding")


def sample_greedy(logits, size, tokens_ptr, pos_pinned_ptr, pos_dev, gen_token, stream=None):
    """Greedy branch of sample() (sampler.h:77-84): tokens/pos pointers are pinned host addresses."""
    check(_lib.lib().q4_argmax(_stream(stream), _p(logits), size, C.c_void_p(tokens_ptr), C.c_void_p(pos_pinned_ptr), _p(pos_dev),
                               int(bool(gen_token))), "sample")


def sample_topp(logits, size, temperature, topp, coin, tokens_ptr, pos_pinned_ptr, pos_dev, stream=None):
    """Non-greedy branch of sample() (sampler.h:85-115): logits become probabilities, the token goes to the mailbox."""
    check(_lib.lib().q4_sample_topp(_stream(stream), _p(logits), size, temperature, topp, coin, C.c_void_p(tokens_ptr),
                                    C.c_void_p(pos_pinned_ptr), _p(pos_dev)), "sample")


def dequant(w, K, N, stream=None):
    out = torch.empty((N, K), dtype=torch.float32, device=w.weight.device)
    check(_lib.lib().q4_dequant(_stream(stream), _p(out), w.ref, K, N), "dequant")
    return out


def unpack_nibbles(w, K, N, stream=None):
    G = (K + 127) // 128
    q = torch.empty((N, K), dtype=torch.uint8, device=w.weight.device)
    z = torch.empty((N, G), dtype=torch.uint8, device=w.weight.device)
    check(_lib.lib().q4_unpack_nibbles(_stream(stream), _p(q), _p(z), w.ref, K, N), "unpack_nibbles")
    return q, z


class BatchedMatmul:
    """matmul(QWeight) for M rows at once (q4_matmul_q4_batched): the tcgen05 dequant-GEMM. Holds the workspace and,
    with interleave=True, the re-ordered copy of the packed weights."""

    def __init__(self, w, inpSize, opSize, max_rows, interleave=True):
        L = _lib.lib()
        self.w, self.K, self.N, self.max_rows = w, inpSize, opSize, max_rows
        self.ws_bytes = max(L.q4_matmul_q4_batched_workspace_bytes(m, inpSize, opSize) for m in {1, 16, 17, 64, 65, max_rows})
        self.ws = torch.zeros(self.ws_bytes, dtype=torch.uint8, device="cuda")
        self.wi = None
        if interleave:
            self.wi = torch.empty_like(w.weight)
            check(L.q4_gemm_interleave_weights(_stream(), _p(self.wi), _p(w.weight), inpSize, opSize), "interleave_weights")

    def __call__(self, y, x, rows, stream=None):
        assert rows <= self.max_rows
        check(_lib.lib().q4_matmul_q4_batched(_stream(stream), _p(y), _p(x), self.w.ref, _p(self.wi), rows, self.K, self.N, _p(self.ws), self.ws_bytes),
              "matmul_batched")

    def status(self, stream=None):
        return _lib.lib().q4_matmul_q4_batched_status(_stream(stream), _p(self.ws))


def matmul_rows(y, x, w, rows, inpSize, opSize, residual=None, residual_scale=1.0, stream=None):
    """matmul(QWeight) for 1..16 rows (q4_matmul_q4_rows): y[m] = x[m] * deq(w) [+ residual[m] * residual_scale]."""
    check(_lib.lib().q4_matmul_q4_rows(_stream(stream), _p(y), _p(x), w.ref, rows, inpSize, opSize, _p(residual), residual_scale), "matmul_rows")


def qkv_matmul_rows(q, k, v, x, qw, kw, vw, rows, inpSize, opSize, kvSize, stream=None):
    """qkv_matvec for 1..16 rows (q4_qkv_matmul_rows); K and V rows land in plain [rows][kvSize] buffers."""
    check(_lib.lib().q4_qkv_matmul_rows(_stream(stream), _p(q), _p(k), _p(v), _p(x), qw.ref, kw.ref, vw.ref, rows, inpSize, opSize, kvSize),
          "qkv_matmul_rows")


def ffn_silu_rows(h, x, gate_w, up_w, rows, inpSize, opSize, stream=None):
    """ffn_matvec_silu for 1..16 rows (q4_ffn_silu_rows)."""
    check(_lib.lib().q4_ffn_silu_rows(_stream(stream), _p(h), _p(x), gate_w.ref, up_w.ref, rows, inpSize, opSize), "ffn_silu_rows")
