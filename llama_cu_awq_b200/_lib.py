"""ctypes binding of libq4b200.so (the C ABI declared in include/q4b200.h).

The library is the product; there is no Python or CPU fallback. Loading fails loudly when the shared
object has not been built (python -m llama_cu_awq_b200.build).
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libq4b200.so")
# The same sources built with -DQ4_TEST_BUILD: adds measurement switches and host-side fault injectors (tests only).
TEST_LIB_PATH = os.path.join(HERE, "libq4b200_test.so")

Q4_OK = 0
Q4_ERR_UNSUPPORTED_SIZE = 1
Q4_ERR_CUDA = 2
Q4_ERR_IO = 3
Q4_ERR_BAD_MODEL = 4
Q4_ERR_INVALID = 5
Q4_ERR_TIMEOUT = 6
Q4_ERR_LIMIT = 7
Q4_PATH_PROMPT_ONE_PASS = 0x100
Q4_MAX_SEQ_LEN = 128 * 1024
Q4_TP_NONE, Q4_TP_COLUMN, Q4_TP_HYBRID = 0, 1, 2
Q4_COMM_BACKEND_P2P, Q4_COMM_BACKEND_NCCL, Q4_COMM_BACKEND_AUTO = 0, 1, 2


class Q4Error(RuntimeError):
    def __init__(self, status, what):
        self.status = status
        super().__init__(f"{what}: {status_string(status)} (status {status})")


class q4_config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "vocab_size", "seq_len")] + [
        ("rope_theta", C.c_float)
    ]


class q4_qweight(C.Structure):
    _fields_ = [("weight", C.c_void_p), ("zeros", C.c_void_p), ("scales", C.c_void_p)]


class q4_shared_data(C.Structure):
    _fields_ = [("pos", C.c_int32), ("tokens", C.c_int32 * Q4_MAX_SEQ_LEN)]


_P = C.c_void_p
_I = C.c_int
_QW = C.POINTER(q4_qweight)

# name -> (restype, argtypes); every symbol include/q4b200.h declares
SIGNATURES = {
    "q4_status_string": (C.c_char_p, [_I]),
    "q4_abi_version": (_I, []),
    "q4_build_arch": (C.c_char_p, []),
    "q4_rmsnorm": (_I, [_P, _P, _P, _P, _I]),
    "q4_matmul_q4": (_I, [_P, _P, _P, _QW, _I, _I, _I, _I, _I, _P]),
    "q4_matmul_q4_batched_workspace_bytes": (C.c_size_t, [_I, _I, _I]),
    "q4_gemm_interleave_weights": (_I, [_P, _P, _P, _I, _I]),
    "q4_matmul_q4_batched": (_I, [_P, _P, _P, _QW, _P, _I, _I, _I, _P, C.c_size_t]),
    "q4_matmul_q4_batched_residual": (_I, [_P, _P, _P, _QW, _P, _I, _I, _I, _P, C.c_float, _P, C.c_size_t]),
    "q4_matmul_q4_batched_status": (_I, [_P, _P]),
    "q4_matmul_q4_rows": (_I, [_P, _P, _P, _QW, _I, _I, _I, _P, C.c_float]),
    "q4_qkv_matmul_rows": (_I, [_P, _P, _P, _P, _P, _QW, _QW, _QW, _I, _I, _I, _I]),
    "q4_ffn_silu_rows": (_I, [_P, _P, _P, _QW, _QW, _I, _I, _I]),
    "q4_time_matmul_q4_batched": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, C.c_size_t, _I, C.POINTER(C.c_double)]),
    "q4_qkv_matvec": (_I, [_P, _P, _P, _P, _P, _QW, _QW, _QW, _I, _I, _I, _I, _P]),
    "q4_ffn_matvec_silu": (_I, [_P, _P, _P, _QW, _QW, _I, _I]),
    "q4_rope": (_I, [_P, _P, _P, _I, _I, _I, _P, _I, C.c_float]),
    "q4_attention_scratch_bytes": (C.c_size_t, [_I, _I]),
    "q4_attention": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "q4_attention_static": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "q4_matmul_f16": (_I, [_P, _P, _P, _P, _I, _I, C.c_float]),
    "q4_embed": (_I, [_P, _P, _P, _I, _P, _P]),
    "q4_argmax": (_I, [_P, _P, _I, _P, _P, _P, _I]),
    "q4_sample_topp": (_I, [_P, _P, _I, C.c_float, C.c_float, C.c_float, _P, _P, _P]),
    "q4_random_u32": (C.c_uint, [_P]),
    "q4_random_f32": (C.c_float, [_P]),
    "q4_dequant": (_I, [_P, _P, _QW, _I, _I]),
    "q4_unpack_nibbles": (_I, [_P, _P, _P, _QW, _I, _I]),
    "q4_comm_id_create": (_I, [C.POINTER(_P), _I]),
    "q4_comm_id_destroy": (_I, [_P]),
    "q4_comm_init_rank": (_I, [C.POINTER(_P), _I, _P, _I]),
    "q4_comm_create_local": (_I, [C.POINTER(_P), _I, _I]),
    "q4_comm_export": (_I, [_P, C.c_char_p]),
    "q4_comm_import": (_I, [_P, _I, C.c_char_p]),
    "q4_all_reduce": (_I, [_P, _P, _P, _I]),
    "q4_all_gather": (_I, [_P, _P, _P, _P, _I]),
    "q4_comm_status": (_I, [_P]),
    "q4_comm_set_wait_limit_ns": (_I, [_P, C.c_ulonglong]),
    "q4_comm_reset": (_I, [_P]),
    "q4_comm_nccl_available": (_I, []),
    "q4_comm_nccl_unique_id": (_I, [_P]),
    "q4_comm_nccl_init": (_I, [_P, _P]),
    "q4_comm_set_backend": (_I, [_P, _I]),
    "q4_comm_destroy": (_I, [_P]),
    "q4_model_load": (_I, [C.POINTER(_P), C.c_char_p, _I, _I, _I, _P]),
    "q4_model_create_synthetic": (_I, [C.POINTER(_P), C.POINTER(q4_config), C.c_ulonglong, _I, _I, _I, _P]),
    "q4_model_free": (_I, [_P]),
    "q4_model_config": (_I, [_P, C.POINTER(q4_config)]),
    "q4_model_shared": (C.POINTER(q4_shared_data), [_P]),
    "q4_model_logits": (_P, [_P]),
    "q4_model_x": (_P, [_P]),
    "q4_model_read": (_I, [_P, _I, _P]),
    "q4_model_reset": (_I, [_P, C.POINTER(C.c_int), _I, _I]),
    "q4_model_forward": (_I, [_P, _P, _I, _I]),
    "q4_model_prepare": (_I, [_P, _I]),
    "q4_model_prefill": (_I, [_P, _P, _I, _I]),
    "q4_batch_create": (_I, [C.POINTER(_P), _P, _I]),
    "q4_batch_reset": (_I, [_P, C.POINTER(_I), _I]),
    "q4_batch_forward": (_I, [_P, _P]),
    "q4_batch_logits": (_P, [_P]),
    "q4_batch_read_tokens": (_I, [_P, C.POINTER(_I), _I]),
    "q4_batch_free": (_I, [_P]),
    "q4_model_set_sampler": (_I, [_P, C.c_float, C.c_float, C.c_ulonglong]),
    "q4_model_status": (_I, [_P]),
    "q4_model_set_wait_limit_ns": (_I, [_P, C.c_ulonglong]),
    "q4_generate": (_I, [_P, C.POINTER(C.c_int), _I, _I, _I, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_double)]),
    "q4_model_token_bytes": (C.c_double, [_P, _I]),
    "q4_model_time_ffn": (_I, [_P, _P, _I, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "q4_time_q4_op": (_I, [_P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "q4_time_q4_rows_op": (_I, [_P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "q4_time_all_reduce": (_I, [_P, _P, _P, _I, _I, C.POINTER(C.c_double)]),
    "q4_model_trace": (_I, [_P, _P, _P, _I]),
    "q4_tokenizer_load": (_I, [C.POINTER(_P), C.c_char_p, _I]),
    "q4_tokenizer_free": (None, [_P]),
    "q4_tokenizer_encode": (_I, [_P, C.c_char_p, _I, _I, C.POINTER(_I), _I, C.POINTER(_I)]),
    "q4_tokenizer_decode": (C.c_char_p, [_P, _I, _I]),
    "q4_row_split_range": (None, [_I, _I, _I, C.POINTER(_I), C.POINTER(_I)]),
    "q4_shard_columns_host": (_I, [_QW, _I, _I, _I, _I, _P, _P, _P]),
    "q4_shard_rows_host": (_I, [_QW, _I, _I, _I, _I, _P, _P, _P]),
}

# exported by the test build only
TEST_SIGNATURES = {
    "q4_test_set_fused_debug": (None, [_I]),
    "q4_test_set_split_len": (None, [_I]),
    "q4_test_set_ring_entries": (None, [_I]),
    "q4_test_fail_fused_alloc": (None, [_I]),
    "q4_test_comm_set_peer": (_I, [_P, _I, _P]),
    "q4_test_fused_gemv": (_I, [_P, _P, _P, _QW, _I, _I]),
    "q4_test_model_slot_trace": (_I, [_P, _P]),
}

_lib = None
_test_lib = None


def _load(path, signatures):
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: build it with `python -m llama_cu_awq_b200.build`; there is no fallback path")
    L = C.CDLL(path)
    for name, (res, args) in signatures.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


def lib():
    """The loaded shared library; raises if it is missing (no fallback of any kind)."""
    global _lib
    if _lib is None:
        _lib = _load(LIB_PATH, SIGNATURES)
    return _lib


def test_lib():
    """The test build of the library (its own copy of all state; objects of one build must not be passed to the other)."""
    global _test_lib
    if _test_lib is None:
        _test_lib = _load(TEST_LIB_PATH, {**SIGNATURES, **TEST_SIGNATURES})
    return _test_lib


def status_string(status):
    return lib().q4_status_string(int(status)).decode()


def check(status, what):
    if status != Q4_OK:
        raise Q4Error(status, what)
