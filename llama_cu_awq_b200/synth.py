"""Seeded synthetic tensors and model files in the packed-q4 layout (the layout weight_packer.cpp:256-291
writes and llama2_q4.cu:220-246 reads). Stand-ins for real AWQ checkpoints, which need a network to fetch.

Value distributions: packed weight words uniform uint32 (nibbles uniform on 0..15), zero nibbles uniform on
0..15 (padding nibbles of the last zeros word are left random on purpose: they must never be read), scales
fp16 of U[0.002, 0.02], embeddings / classifier fp16 of N(0, 0.02), RMSNorm weights 1.0.
"""
import struct

import numpy as np

CONFIGS = {
    # name: dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len, rope_theta
    "tiny": (256, 512, 2, 2, 2, 512, 64, 10000.0),
    "tiny-gqa": (512, 768, 2, 4, 2, 512, 64, 10000.0),
    "mid": (1024, 2816, 2, 8, 8, 2048, 128, 10000.0),      # 22 groups in the down projection: a full and a partial k-tile
    "mid-gqa": (1024, 2816, 2, 8, 2, 2048, 128, 10000.0),
    "mid-long": (1024, 2816, 2, 8, 2, 2048, 2048, 10000.0),         # long context on a small model (attention over > 1000 positions)
    "llama2-13b-1l": (5120, 13824, 1, 40, 40, 4096, 128, 10000.0),   # 13B / 70B layer shapes, one layer, small vocabulary:
    "llama2-70b-1l": (8192, 28672, 1, 64, 8, 4096, 128, 10000.0),    # shape coverage (3, 4, 7 and 14 k-tiles, 8 query heads per KV head)
    "llama2-7b-4l": (4096, 11008, 4, 32, 32, 32000, 2048, 10000.0),  # 7B layer shapes, 4 layers: profiling-sized
    "llama2-7b": (4096, 11008, 32, 32, 32, 32000, 2048, 10000.0),
    "llama2-13b": (5120, 13824, 40, 40, 40, 32000, 2048, 10000.0),
    "llama2-70b": (8192, 28672, 80, 64, 8, 32000, 4096, 10000.0),
}


def div_up(a, b):
    return (a - 1) // b + 1


def packed_dims(K):
    return div_up(K, 32) * 4, div_up(div_up(K, 128), 8), div_up(K, 128)


def qweight_bytes(K, N):
    pw, pz, g = packed_dims(K)
    return N * (pw * 4 + pz * 4 + g * 2)


def synth_qweight(rng, K, N):
    pw, pz, g = packed_dims(K)
    weight = rng.integers(0, 2**32, size=(N, pw), dtype=np.uint32)
    zeros = rng.integers(0, 2**32, size=(N, pz), dtype=np.uint32)
    scales = rng.uniform(0.002, 0.02, size=(N, g)).astype(np.float16)
    return {"weight": weight, "zeros": zeros, "scales": scales, "K": K, "N": N}


def header(cfg):
    return struct.pack("<7if", *cfg[:7], cfg[7])


def file_bytes(cfg):
    dim, hid, L, H, KV, V, _, _ = cfg
    kvd = dim * KV // H
    per_layer = 2 * qweight_bytes(dim, dim) + 2 * qweight_bytes(dim, kvd) + 2 * qweight_bytes(dim, hid) + qweight_bytes(hid, dim) + 4 * dim
    return 32 + 4 * V * dim + 2 * dim + per_layer * L


def write_model_file(path, cfg, seed=0):
    """Writes a whole synthetic model file, tensor by tensor. Returns the byte count."""
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    dim, hid, L, H, KV, V, _, _ = cfg
    kvd = dim * KV // H
    rng = np.random.default_rng(seed)
    n = 0
    with open(path, "wb") as f:
        def put(a):
            nonlocal n
            b = a.tobytes() if hasattr(a, "tobytes") else a
            f.write(b)
            n += len(b)

        def putq(K, N):
            q = synth_qweight(rng, K, N)
            put(q["weight"]); put(q["zeros"]); put(q["scales"])

        put(header(cfg))
        for _ in range(2):  # token_embedding_table, wcls
            chunk = 4096
            for v0 in range(0, V, chunk):
                rows = min(chunk, V - v0)
                put((rng.standard_normal((rows, dim), dtype=np.float32) * 0.02).astype(np.float16))
        put(np.ones(dim, np.float16))
        for _ in range(L):
            putq(dim, dim); putq(dim, kvd); putq(dim, kvd); putq(dim, dim)
            putq(dim, hid); putq(dim, hid)  # up, then gate
            putq(hid, dim)
            put(np.ones(dim, np.float16)); put(np.ones(dim, np.float16))
    assert n == file_bytes(cfg), (n, file_bytes(cfg))
    return n


def synth_prompt(n=16, vocab=32000, seed=0):
    return np.random.default_rng(seed).integers(3, vocab, size=n, dtype=np.int32)
