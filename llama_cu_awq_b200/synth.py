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


# ---------------------------------------------------------------------------------------------------------
# Counter-based generator: the host twin of csrc/q4_synth.cu. Every element is a function of (seed, tensor id,
# logical element index); q4_model_create_synthetic builds the same model on the device without a file.
# ---------------------------------------------------------------------------------------------------------
_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def counter_hash(seed, tid, idx):
    """64-bit mix of (seed, tensor id, element index); idx is an array of uint64."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + np.uint64(tid) * np.uint64(0x9E3779B97F4A7C15) + idx.astype(np.uint64) * np.uint64(0xD1B54A32D192ED03)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def counter_qweight(seed, tid, K, N):
    """One quantized matrix of the counter-based model (tensor ids tid, tid + 1, tid + 2: weights, zero points, scales)."""
    pw, pz, g = packed_dims(K)
    n = np.arange(N, dtype=np.uint64)[:, None]
    jw = np.arange(pw, dtype=np.uint64)[None, :]
    weight = (counter_hash(seed, tid, n * np.uint64(pw) + jw) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    weight[:, div_up(K, 8):] = 0
    gi = np.arange(g, dtype=np.uint64)[None, :]
    nib = (counter_hash(seed, tid + 1, n * np.uint64(g) + gi) & np.uint64(15)).astype(np.uint32)
    zeros = np.zeros((N, pz), np.uint32)
    for k in range(g):
        zeros[:, k // 8] |= nib[:, k] << np.uint32(4 * (k % 8))
    u = (counter_hash(seed, tid + 2, n * np.uint64(g) + gi) >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    scales = (np.float32(0.002) + np.float32(0.018) * u).astype(np.float16)
    return {"weight": weight, "zeros": zeros, "scales": scales, "K": K, "N": N}


def counter_normal(seed, tid, idx0, count):
    """fp16 of 0.02 * (sum of twelve 16-bit uniforms - 6): elements idx0 .. idx0 + count of tensor tid."""
    i = (np.arange(count, dtype=np.uint64) + np.uint64(idx0)) * np.uint64(4)
    s = np.zeros(count, np.int64)
    for k in range(3):
        h = counter_hash(seed, tid, i + np.uint64(k))
        for sh in (0, 16, 32, 48):
            s += ((h >> np.uint64(sh)) & np.uint64(0xFFFF)).astype(np.int64)
    return ((s - 393210).astype(np.float32) * (np.float32(0.02) / np.float32(65536.0))).astype(np.float16)


def write_counter_model_file(path, cfg, seed=0):
    """The counter-based model as a packed file (same bits as q4_model_create_synthetic generates on the device)."""
    if isinstance(cfg, str):
        cfg = CONFIGS[cfg]
    dim, hid, L, H, KV, V, _, _ = cfg
    kvd = dim * KV // H
    n = 0
    with open(path, "wb") as f:
        def put(a):
            nonlocal n
            b = a.tobytes() if hasattr(a, "tobytes") else a
            f.write(b)
            n += len(b)

        def putq(tid, K, N):
            q = counter_qweight(seed, tid, K, N)
            put(q["weight"]); put(q["zeros"]); put(q["scales"])

        put(header(cfg))
        for tid in (1, 2):  # token_embedding_table, wcls
            rows = 1024
            for v0 in range(0, V, rows):
                r = min(rows, V - v0)
                put(counter_normal(seed, tid, v0 * dim, r * dim))
        put(np.ones(dim, np.float16))
        for l in range(L):
            t = lambda m: 16 + (l * 8 + m) * 4  # noqa: E731
            putq(t(0), dim, dim); putq(t(1), dim, kvd); putq(t(2), dim, kvd); putq(t(3), dim, dim)
            putq(t(4), dim, hid); putq(t(5), dim, hid)  # up, then gate
            putq(t(6), hid, dim)
            put(np.ones(dim, np.float16)); put(np.ones(dim, np.float16))
    assert n == file_bytes(cfg), (n, file_bytes(cfg))
    return n


def synth_prompt(n=16, vocab=32000, seed=0):
    return np.random.default_rng(seed).integers(3, vocab, size=n, dtype=np.int32)
