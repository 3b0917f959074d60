"""Generates the packed-format golden fixture with the reference's own weight_packer.

Run in the build container (needs the reference sources, built by `make -C oracle` into oracle/_ref/):

    python tests/golden/make_golden.py

Writes, next to this script:
  tiny_logical.npz   the logical tensors of a tiny 2-layer GQA model (seeded): per matrix the nibbles
                     q[K,N], zero points z[G,N] (uint8) and scales s[G,N] (fp16), plus fp16 vectors
  tiny_packed_fmt1.bin  what weight_packer wrote when fed those tensors in the old AWQ layout
                     (order-mapped, N-packed; weight_packer.cpp:94-144) - i.e. through its repacking path
The same model fed in the new AWQ layout (weight_packer.cpp:166-170,201-212) is packed too and must equal
the numpy restatement of the layout byte for byte (asserted here, not stored).
The tests check the oracle's and the CUDA path's accessors against these bytes.
"""
import json
import os
import shutil
import subprocess
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PACKER = os.path.join(ROOT, "oracle", "_ref", "weight_packer")

DIM, HID, L, H, KV, V, SEQ, THETA = 128, 384, 2, 2, 1, 32, 32, 10000.0
ORDER = [0, 2, 4, 6, 1, 3, 5, 7]  # AWQ's nibble order inside a word (weight_packer.cpp:96)


def div_up(a, b):
    return (a - 1) // b + 1


def pack_le(a):
    """[rows, cols] nibbles -> [rows, ceil(cols/8)] uint32, nibble i of a word = element 8j+i."""
    r, c = a.shape
    c8 = div_up(c, 8) * 8
    p = np.zeros((r, c8), np.uint32)
    p[:, :c] = a
    p = p.reshape(r, c8 // 8, 8)
    out = np.zeros((r, c8 // 8), np.uint32)
    for i in range(8):
        out |= p[:, :, i] << np.uint32(4 * i)
    return out


def pack_awq_old(a):
    """[rows, cols] nibbles -> [rows, cols/8] uint32 with AWQ's order map: nibble i holds element ORDER[i]."""
    r, c = a.shape
    p = a.reshape(r, c // 8, 8).astype(np.uint32)
    out = np.zeros((r, c // 8), np.uint32)
    for i in range(8):
        out |= p[:, :, ORDER[i]] << np.uint32(4 * i)
    return out


def matrices():
    kvd = DIM * KV // H
    return [("self_attn.q_proj", DIM, DIM), ("self_attn.k_proj", DIM, kvd), ("self_attn.v_proj", DIM, kvd), ("self_attn.o_proj", DIM, DIM),
            ("mlp.up_proj", DIM, HID), ("mlp.gate_proj", DIM, HID), ("mlp.down_proj", HID, DIM)]


def main():
    assert os.path.exists(PACKER), "build the reference packer first: make -C oracle"
    rng = np.random.default_rng(20240611)
    logical = {}
    logical["embed"] = (rng.standard_normal((V, DIM)) * 0.02).astype(np.float16)
    logical["lm_head"] = (rng.standard_normal((V, DIM)) * 0.02).astype(np.float16)
    logical["norm"] = rng.uniform(0.5, 1.5, DIM).astype(np.float16)
    for l in range(L):
        for nm, K, N in matrices():
            G = div_up(K, 128)
            logical[f"{l}.{nm}.q"] = rng.integers(0, 16, (K, N)).astype(np.uint8)
            logical[f"{l}.{nm}.z"] = rng.integers(0, 16, (G, N)).astype(np.uint8)
            logical[f"{l}.{nm}.s"] = rng.uniform(0.002, 0.02, (G, N)).astype(np.float16)
        logical[f"{l}.input_layernorm"] = rng.uniform(0.5, 1.5, DIM).astype(np.float16)
        logical[f"{l}.post_attention_layernorm"] = rng.uniform(0.5, 1.5, DIM).astype(np.float16)
    np.savez_compressed(os.path.join(HERE, "tiny_logical.npz"), **logical)

    for fmt in (1, 0):
        d = tempfile.mkdtemp()
        try:
            json.dump({"hidden_size": DIM, "intermediate_size": HID, "num_hidden_layers": L, "num_attention_heads": H,
                       "num_key_value_heads": KV, "vocab_size": V, "max_position_embeddings": SEQ, "rope_theta": THETA},
                      open(os.path.join(d, "config.json"), "w"))
            logical["embed"].tofile(os.path.join(d, "model.embed_tokens.weight.bin"))
            logical["lm_head"].tofile(os.path.join(d, "lm_head.weight.bin"))
            logical["norm"].tofile(os.path.join(d, "model.norm.weight.bin"))
            for l in range(L):
                for nm, K, N in matrices():
                    G = div_up(K, 128)
                    q, z, s = logical[f"{l}.{nm}.q"], logical[f"{l}.{nm}.z"], logical[f"{l}.{nm}.s"]
                    base = os.path.join(d, f"model.layers.{l}.{nm}")
                    if fmt == 1:  # qweight [K, N/8], qzeros [G, N/8] order-mapped, scales [G, N]
                        pack_awq_old(q).tofile(base + ".qweight.bin")
                        pack_awq_old(z).tofile(base + ".qzeros.bin")
                        s.tofile(base + ".scales.bin")
                    else:  # qweight [N, K/8], qzeros [N, ceil(G/8)], scales [N, 8*ceil(G/8)] (padded)
                        pack_le(q.T).tofile(base + ".qweight.bin")
                        pack_le(z.T).tofile(base + ".qzeros.bin")
                        sp = np.zeros((N, div_up(G, 8) * 8), np.float16)
                        sp[:, :G] = s.T
                        sp.tofile(base + ".scales.bin")
                logical[f"{l}.input_layernorm"].tofile(os.path.join(d, f"model.layers.{l}.input_layernorm.weight.bin"))
                logical[f"{l}.post_attention_layernorm"].tofile(os.path.join(d, f"model.layers.{l}.post_attention_layernorm.weight.bin"))
            out = os.path.join(HERE, f"tiny_packed_fmt{fmt}.bin")
            subprocess.run([PACKER, os.path.join(d, "config.json"), d, out, str(fmt)], check=True, stdout=subprocess.DEVNULL)
            print(out, os.path.getsize(out))
            if fmt == 0:
                exp = [np.array([DIM, HID, L, H, KV, V, SEQ], np.int32).tobytes(), np.float32(THETA).tobytes(),
                       logical["embed"].tobytes(), logical["lm_head"].tobytes(), logical["norm"].tobytes()]
                for l in range(L):
                    for nm, K, N in matrices():
                        exp += [pack_le(logical[f"{l}.{nm}.q"].T).tobytes(), pack_le(logical[f"{l}.{nm}.z"].T).tobytes(),
                                np.ascontiguousarray(logical[f"{l}.{nm}.s"].T).tobytes()]
                    exp += [logical[f"{l}.input_layernorm"].tobytes(), logical[f"{l}.post_attention_layernorm"].tobytes()]
                assert open(out, "rb").read() == b"".join(exp), "new-format packer output differs from the layout restatement"
                os.remove(out)
                print("fmt 0 output identical to the numpy layout model (not stored)")
        finally:
            shutil.rmtree(d)


if __name__ == "__main__":
    main()
