"""CPU tests: the oracle against the reference packer's golden file, fp16 conversions, shard helpers."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from conftest import GOLDEN
from llama_cu_awq_b200 import _lib, synth
from oracle import q4_oracle as O

DIM, HID, L, H, KV, V, SEQ = 128, 384, 2, 2, 1, 32, 32
MATS = [("self_attn.q_proj", DIM, DIM), ("self_attn.k_proj", DIM, DIM * KV // H), ("self_attn.v_proj", DIM, DIM * KV // H),
        ("self_attn.o_proj", DIM, DIM), ("mlp.up_proj", DIM, HID), ("mlp.gate_proj", DIM, HID), ("mlp.down_proj", HID, DIM)]


def walk_file(image):
    """Splits a packed file image into tensors following the documented order; yields (name, dict)."""
    cfg = struct.unpack("<7if", image[:32])
    dim, hid, nl, nh, nkv, v, _, _ = cfg
    kvd = dim * nkv // nh
    off = 32
    out = {"cfg": cfg}

    def take(n, dt):
        nonlocal off
        a = np.frombuffer(image, dt, n, off)
        off += a.nbytes
        return a

    out["embed"] = take(v * dim, np.float16).reshape(v, dim)
    out["lm_head"] = take(v * dim, np.float16).reshape(v, dim)
    out["norm"] = take(dim, np.float16)
    for l in range(nl):
        for nm, K, N in [("self_attn.q_proj", dim, dim), ("self_attn.k_proj", dim, kvd), ("self_attn.v_proj", dim, kvd),
                         ("self_attn.o_proj", dim, dim), ("mlp.up_proj", dim, hid), ("mlp.gate_proj", dim, hid), ("mlp.down_proj", hid, dim)]:
            pw, pz, g = synth.packed_dims(K)
            out[f"{l}.{nm}"] = {"weight": take(N * pw, np.uint32).reshape(N, pw), "zeros": take(N * pz, np.uint32).reshape(N, pz),
                                "scales": take(N * g, np.float16).reshape(N, g), "K": K, "N": N}
        out[f"{l}.input_layernorm"] = take(dim, np.float16)
        out[f"{l}.post_attention_layernorm"] = take(dim, np.float16)
    assert off == len(image)
    return out


@pytest.fixture(scope="module")
def golden():
    image = open(os.path.join(GOLDEN, "tiny_packed_fmt1.bin"), "rb").read()
    logical = np.load(os.path.join(GOLDEN, "tiny_logical.npz"))
    return image, logical


def test_golden_header_and_length(golden):
    image, _ = golden
    cfg = struct.unpack("<7if", image[:32])
    assert cfg == (DIM, HID, L, H, KV, V, SEQ, 10000.0)
    assert len(image) == synth.file_bytes(cfg)


def test_oracle_accessors_match_reference_packer(golden):
    """Every used nibble, zero point and scale the oracle reads out of the reference packer's file equals the
    logical tensor that went in (bit exact). Padding nibbles of the zeros words are not compared: the packer
    leaves garbage there."""
    image, logical = golden
    t = walk_file(image)
    assert (t["embed"] == logical["embed"]).all() and (t["lm_head"] == logical["lm_head"]).all() and (t["norm"] == logical["norm"]).all()
    garbage = 0
    for l in range(L):
        for nm, K, N in MATS:
            q, z = O.unpack(t[f"{l}.{nm}"], K, N)
            assert (q == logical[f"{l}.{nm}.q"].T).all(), (l, nm)
            assert (z == logical[f"{l}.{nm}.z"].T).all(), (l, nm)
            assert (t[f"{l}.{nm}"]["scales"] == logical[f"{l}.{nm}.s"].T).all(), (l, nm)
            G = synth.div_up(K, 128)
            if G % 8:
                pad_mask = np.uint32((0xFFFFFFFF << (4 * (G % 8))) & 0xFFFFFFFF)
                garbage += int((t[f"{l}.{nm}"]["zeros"][:, -1] & pad_mask != 0).sum())
            # dequantised values, exact in fp32
            w = O.dequant(t[f"{l}.{nm}"], K, N)
            s = logical[f"{l}.{nm}.s"].astype(np.float32)
            exp = (logical[f"{l}.{nm}.q"].astype(np.float32) - np.repeat(logical[f"{l}.{nm}.z"].astype(np.float32), 128, 0)[:K]) * np.repeat(s, 128, 0)[:K]
            assert (w == exp.T).all(), (l, nm)
        assert (t[f"{l}.input_layernorm"] == logical[f"{l}.input_layernorm"]).all()
    assert garbage > 0, "the old-format packer path is expected to leave garbage in unused zero nibbles"


def test_oracle_model_opens_golden_and_runs(golden):
    image, _ = golden
    m = O.Model(image)
    assert (m.dim, m.n_layers, m.n_kv_heads) == (DIM, L, KV)
    toks = []
    tok = 5
    for pos in range(6):
        tok = m.forward(tok, pos)
        toks.append(tok)
        lg = m.logits()
        assert np.isfinite(lg.astype(np.float32)).all() and O.argmax(lg) == tok
    with pytest.raises(ValueError):
        O.Model(image[:-2])


def test_fp16_conversions_match_numpy():
    L_ = O.lib()
    hs = np.arange(0, 65536, 3, dtype=np.uint16)
    for h in hs:
        f = L_.q4o_h2f(int(h))
        g = float(np.uint16(h).view(np.float16).astype(np.float32))
        assert f == g or (np.isnan(f) and np.isnan(g))
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.standard_normal(4000) * np.exp(rng.uniform(-25, 11, 4000)), [0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8,
                           2.9802322e-8, 6.1e-5, 6.0975e-5, np.inf, -np.inf]]).astype(np.float32)
    with np.errstate(over="ignore"):
        exp = vals.astype(np.float16).view(np.uint16)
    for v, e in zip(vals, exp):
        assert L_.q4o_f2h(float(v)) == e, v
    # ties to even on the half grid
    for h in range(0x3C00, 0x3C10):
        a, b = np.uint16(h).view(np.float16).astype(np.float32), np.uint16(h + 1).view(np.float16).astype(np.float32)
        mid = np.float32((a + b) / 2)
        assert L_.q4o_f2h(float(mid)) == (h if h % 2 == 0 else h + 1)


def test_matvec_orders_agree_and_match_float64():
    rng = np.random.default_rng(0)
    for K, N in [(128, 8), (256, 16), (384, 8), (4096, 64), (11008, 16), (5120 // 8, 24)]:
        q = synth.synth_qweight(rng, K, N)
        x = rng.standard_normal(K).astype(np.float16)
        y0, y1, y64 = O.matvec(x, q, K, N, order=0), O.matvec(x, q, K, N, order=1), O.matvec_f32(x, q, K, N)
        w = O.dequant(q, K, N).astype(np.float64)
        assert np.allclose(w @ x.astype(np.float64), y64, rtol=1e-6, atol=1e-6)
        for y in (y0, y1):
            assert np.abs(y.astype(np.float32) - y64).max() <= 2e-3 * np.abs(y64).max()
    # fused residual: y_old / gpu_count is added before rounding (gpu_kernels.h:237-239)
    K, N = 256, 8
    q = synth.synth_qweight(rng, K, N)
    x = rng.standard_normal(K).astype(np.float16)
    yo = rng.standard_normal(N).astype(np.float16)
    y = O.matvec(x, q, K, N, y_old=yo, gpu_count=4)
    exp = (O.matvec_f32(x, q, K, N) + yo.astype(np.float32) / 4).astype(np.float16)
    assert np.abs(y.astype(np.float32) - exp.astype(np.float32)).max() <= 2e-3 * np.abs(exp.astype(np.float32)).max()


def test_argmax_lowest_index_on_ties():
    lg = np.zeros(1000, np.float16)
    lg[[17, 400, 999]] = 3.0
    assert O.argmax(lg) == 17
    lg[:] = -np.inf
    assert O.argmax(lg) == 0


def test_allreduce_reference_order_is_rank_dependent():
    """cuda_comm.h:193-219 adds own-then-peers in fp16; different ranks can disagree in the last bit."""
    rng = np.random.default_rng(3)
    parts = (rng.standard_normal((8, 4096)) * 3).astype(np.float16)
    outs = [O.allreduce_ref_order(parts, r) for r in range(8)]
    exact = parts.astype(np.float64).sum(0)
    assert any((outs[0] != o).any() for o in outs[1:])
    for o in outs:
        assert np.abs(o.astype(np.float64) - exact).max() < 0.05


# ---- host-side shard helpers of the C ABI (no GPU involved) ----

def _qw_struct(q):
    return _lib.q4_qweight(q["weight"].ctypes.data, q["zeros"].ctypes.data, q["scales"].ctypes.data)


def test_row_split_ranges_are_group_aligned_and_cover():
    Lb = _lib.lib()
    for K in (4096, 5120, 8192, 11008, 13824, 28672, 384):
        for g in (1, 2, 4, 8):
            tot, prev_end = 0, 0
            for r in range(g):
                kb, kc = C.c_int(), C.c_int()
                Lb.q4_row_split_range(K, g, r, C.byref(kb), C.byref(kc))
                assert kb.value == prev_end and kb.value % 128 == 0
                assert kc.value % 128 == 0 or kb.value + kc.value == K
                prev_end = kb.value + kc.value
                tot += kc.value
            assert tot == K
    kb, kc = C.c_int(), C.c_int()
    Lb.q4_row_split_range(11008, 8, 7, C.byref(kb), C.byref(kc))
    assert (kb.value, kc.value) == (76 * 128, 10 * 128)   # 86 groups -> 11,11,11,11,11,11,10,10


@pytest.mark.parametrize("K,N,g", [(11008, 64, 8), (11008, 32, 4), (11008, 32, 2), (13824, 16, 8), (5120, 16, 8), (1280, 8, 2), (4096, 16, 1)])
def test_row_shards_sum_to_full_matvec(K, N, g):
    """Partial products over the group-aligned input shards add up to the unsharded result (the property
    the reference's byte-offset row split loses when groups-per-rank is odd or fractional)."""
    Lb = _lib.lib()
    rng = np.random.default_rng(K + N + g)
    q = synth.synth_qweight(rng, K, N)
    x = rng.standard_normal(K).astype(np.float16)
    full = O.matvec_f32(x, q, K, N)
    acc = np.zeros(N, np.float64)
    src = _qw_struct(q)
    for r in range(g):
        kb, kc = C.c_int(), C.c_int()
        Lb.q4_row_split_range(K, g, r, C.byref(kb), C.byref(kc))
        pw, pz, gg = synth.packed_dims(kc.value)
        sh = {"weight": np.zeros((N, pw), np.uint32), "zeros": np.full((N, pz), 0xFFFFFFFF, np.uint32), "scales": np.zeros((N, gg), np.float16)}
        assert Lb.q4_shard_rows_host(C.byref(src), K, N, g, r, sh["weight"].ctypes.data, sh["zeros"].ctypes.data, sh["scales"].ctypes.data) == 0
        qs, zs = O.unpack(sh, kc.value, N)
        qf, zf = O.unpack(q, K, N)
        assert (qs == qf[:, kb.value:kb.value + kc.value]).all()
        assert (zs == zf[:, kb.value // 128: kb.value // 128 + gg]).all()
        acc += O.matvec_f32(x[kb.value:kb.value + kc.value], sh, kc.value, N)
    assert np.abs(acc - full).max() <= 1e-4 * max(1.0, np.abs(full).max())


def test_column_shards_are_slices():
    Lb = _lib.lib()
    rng = np.random.default_rng(9)
    K, N, g = 512, 64, 4
    q = synth.synth_qweight(rng, K, N)
    src = _qw_struct(q)
    for r in range(g):
        pw, pz, gg = synth.packed_dims(K)
        n = N // g
        sh = {"weight": np.zeros((n, pw), np.uint32), "zeros": np.zeros((n, pz), np.uint32), "scales": np.zeros((n, gg), np.float16)}
        assert Lb.q4_shard_columns_host(C.byref(src), K, N, g, r, sh["weight"].ctypes.data, sh["zeros"].ctypes.data, sh["scales"].ctypes.data) == 0
        assert (sh["weight"] == q["weight"][r * n:(r + 1) * n]).all() and (sh["scales"] == q["scales"][r * n:(r + 1) * n]).all()
    assert Lb.q4_shard_columns_host(C.byref(src), K, 60, 8, 0, None, None, None) == _lib.Q4_ERR_INVALID


def test_synth_file_roundtrip(tmp_path):
    p = tmp_path / "tiny.bin"
    n = synth.write_model_file(str(p), "tiny", seed=0)
    image = p.read_bytes()
    assert len(image) == n
    t = walk_file(image)
    assert t["cfg"][:7] == synth.CONFIGS["tiny"][:7]
    m = O.Model(image)
    m.forward(3, 0)
    assert np.isfinite(m.logits().astype(np.float32)).all()
