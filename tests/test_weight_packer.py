"""The offline weight_packer tool (csrc/weight_packer.cpp) against the golden file the reference's own packer wrote
(tests/golden/tiny_packed_fmt1.bin, made by tests/golden/make_golden.py from tests/golden/tiny_logical.npz): both AWQ
input layouts must give the reference's bytes, except the zero-point nibbles past a row's last group, which the
reference leaves undefined and this tool writes as 0."""
import json
import os
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN, ROOT

PACKER = os.path.join(ROOT, "llama_cu_awq_b200", "weight_packer")
DIM, HID, L, H, KV, V, SEQ, THETA = 128, 384, 2, 2, 1, 32, 32, 10000.0
ORDER = [0, 2, 4, 6, 1, 3, 5, 7]


def div_up(a, b):
    return (a - 1) // b + 1


def pack_le(a):
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


def write_inputs(d, logical, fmt):
    json.dump({"hidden_size": DIM, "intermediate_size": HID, "num_hidden_layers": L, "num_attention_heads": H, "num_key_value_heads": KV,
               "vocab_size": V, "max_position_embeddings": SEQ, "rope_theta": THETA}, open(os.path.join(d, "config.json"), "w"))
    logical["embed"].tofile(os.path.join(d, "model.embed_tokens.weight.bin"))
    logical["lm_head"].tofile(os.path.join(d, "lm_head.weight.bin"))
    logical["norm"].tofile(os.path.join(d, "model.norm.weight.bin"))
    for l in range(L):
        for nm, K, N in matrices():
            G = div_up(K, 128)
            q, z, s = logical[f"{l}.{nm}.q"], logical[f"{l}.{nm}.z"], logical[f"{l}.{nm}.s"]
            base = os.path.join(d, f"model.layers.{l}.{nm}")
            if fmt == 1:
                pack_awq_old(q).tofile(base + ".qweight.bin")
                pack_awq_old(z).tofile(base + ".qzeros.bin")
                s.tofile(base + ".scales.bin")
            else:
                pack_le(q.T).tofile(base + ".qweight.bin")
                pack_le(z.T).tofile(base + ".qzeros.bin")
                sp = np.zeros((N, div_up(G, 8) * 8), np.float16)
                sp[:, :G] = s.T
                sp.tofile(base + ".scales.bin")
        logical[f"{l}.input_layernorm"].tofile(os.path.join(d, f"model.layers.{l}.input_layernorm.weight.bin"))
        logical[f"{l}.post_attention_layernorm"].tofile(os.path.join(d, f"model.layers.{l}.post_attention_layernorm.weight.bin"))


def used_mask():
    """Byte mask of the packed file: False on the zero-point nibbles past a row's last group (undefined in the reference)."""
    parts = [np.ones(32 + 2 * 2 * V * DIM + 2 * DIM, bool)]
    for _ in range(L):
        for _, K, N in matrices():
            G, PW, PZ = div_up(K, 128), div_up(K, 8), div_up(div_up(K, 128), 8)
            parts.append(np.ones(N * PW * 4, bool))
            z = np.zeros((N, PZ * 8), bool)      # per nibble
            z[:, :G] = True
            zb = (z[:, 0::2] & z[:, 1::2])       # a byte holds two nibbles; compare whole bytes only where both are used
            parts.append(zb.reshape(-1))
            parts.append(np.ones(N * G * 2, bool))
        parts.append(np.ones(4 * DIM, bool))
    return np.concatenate(parts)


@pytest.mark.parametrize("fmt", [1, 0])
def test_weight_packer_reproduces_the_reference_packers_file(fmt, tmp_path):
    if not os.path.exists(PACKER):
        from llama_cu_awq_b200 import build as b
        b.build()
    logical = dict(np.load(os.path.join(GOLDEN, "tiny_logical.npz")))
    d = str(tmp_path)
    write_inputs(d, logical, fmt)
    out = os.path.join(d, "packed.bin")
    r = subprocess.run([PACKER, os.path.join(d, "config.json"), d, out, str(fmt)], capture_output=True, text=True)
    assert r.returncode == 0 and "Done!" in r.stdout, r.stdout[-500:]
    got = np.frombuffer(open(out, "rb").read(), np.uint8)
    want = np.frombuffer(open(os.path.join(GOLDEN, "tiny_packed_fmt1.bin"), "rb").read(), np.uint8)
    assert got.size == want.size
    m = used_mask()
    assert m.size == got.size
    assert (got[m] == want[m]).all()
    # every used zero-point nibble individually (odd group counts share a byte with an unused nibble)
    off = 32 + 2 * 2 * V * DIM + 2 * DIM
    for l in range(L):
        for nm, K, N in matrices():
            G, PW, PZ = div_up(K, 128), div_up(K, 8), div_up(div_up(K, 128), 8)
            off += N * PW * 4
            zg = np.frombuffer(got[off:off + N * PZ * 4].tobytes(), np.uint32).reshape(N, PZ)
            for g in range(G):
                nib = (zg[:, g // 8] >> np.uint32(4 * (g % 8))) & 0xF
                assert (nib == logical[f"{l}.{nm}.z"][g]).all()
            for g in range(G, PZ * 8):
                assert (((zg[:, g // 8] >> np.uint32(4 * (g % 8))) & 0xF) == 0).all()   # unused nibbles: zero here
            off += N * PZ * 4 + N * G * 2
        off += 4 * DIM


def test_weight_packer_usage_and_errors(tmp_path):
    if not os.path.exists(PACKER):
        from llama_cu_awq_b200 import build as b
        b.build()
    r = subprocess.run([PACKER], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.startswith("usage: weight_packer")
    cfg = tmp_path / "config.json"
    cfg.write_text('{"hidden_size": 128}')
    r = subprocess.run([PACKER, str(cfg), str(tmp_path), str(tmp_path / "o.bin"), "0"], capture_output=True, text=True)
    assert r.returncode == 1 and "intermediate_size not found" in r.stdout
