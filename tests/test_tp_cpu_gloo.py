"""Host-side tensor-parallel logic on CPU ranks (gloo, world size 2): each rank shards the matrices with the
library's host helpers, computes its partial results with the oracle, and the ranks exchange them the way the GPU
path does (sum of row-split partials in rank order, concatenation of column-split slices). The result must equal
the unsharded oracle; the fixed-order fp32 sum must give every rank the same bits."""
import ctypes as C
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llama_cu_awq_b200 import _lib, synth
from oracle import q4_oracle as O

DIM, HID = 256, 1152  # 9 groups in the down projection: uneven split 5 + 4


def qw_struct(q):
    return _lib.q4_qweight(q["weight"].ctypes.data, q["zeros"].ctypes.data, q["scales"].ctypes.data)


def shard_rows(L, q, K, N, g, r):
    kb, kc = C.c_int(), C.c_int()
    L.q4_row_split_range(K, g, r, C.byref(kb), C.byref(kc))
    pw, pz, gg = synth.packed_dims(kc.value)
    sh = {"weight": np.zeros((N, pw), np.uint32), "zeros": np.zeros((N, pz), np.uint32), "scales": np.zeros((N, gg), np.float16)}
    src = qw_struct(q)
    assert L.q4_shard_rows_host(C.byref(src), K, N, g, r, sh["weight"].ctypes.data, sh["zeros"].ctypes.data, sh["scales"].ctypes.data) == 0
    return sh, kb.value, kc.value


def cols(q, n0, n1):
    return {"weight": np.ascontiguousarray(q["weight"][n0:n1]), "zeros": np.ascontiguousarray(q["zeros"][n0:n1]),
            "scales": np.ascontiguousarray(q["scales"][n0:n1])}


def worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L = _lib.lib()
        rng = np.random.default_rng(5)  # same tensors on every rank
        gate, up, down = synth.synth_qweight(rng, DIM, HID), synth.synth_qweight(rng, DIM, HID), synth.synth_qweight(rng, HID, DIM)
        x = (rng.standard_normal(DIM) * 0.3).astype(np.float16)
        resid = rng.standard_normal(DIM).astype(np.float16)
        # this rank's slice of the hidden vector = its input rows of the down projection (group aligned)
        dsh, kb, kc = shard_rows(L, down, HID, DIM, world, rank)
        hb = O.ffn_silu(x, cols(gate, kb, kb + kc), cols(up, kb, kb + kc), DIM, kc, order=1)          # column split, no exchange
        part = O.matvec_f32(hb, dsh, kc, DIM) + resid.astype(np.float32) / world                       # row split partial + residual / g
        # fp16 bit patterns travel as int32 (gloo has no 16-bit integer type)
        part16 = torch.from_numpy(part.astype(np.float16).view(np.uint16).astype(np.int32))
        gathered = [torch.empty_like(part16) for _ in range(world)]
        dist.all_gather(gathered, part16)                                                              # what the inbox holds on every rank
        acc = np.zeros(DIM, np.float32)
        for r in range(world):                                                                         # fixed rank order, fp32
            acc += gathered[r].numpy().astype(np.uint16).view(np.float16).astype(np.float32)
        y = acc.astype(np.float16)
        ys = [torch.empty(DIM, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(ys, torch.from_numpy(y.view(np.uint16).astype(np.int32)))
        if rank == 0:
            same = all(torch.equal(ys[0], t) for t in ys)
            hb_full = O.ffn_silu(x, gate, up, DIM, HID, order=1)
            ref = O.matvec(hb_full, down, HID, DIM, y_old=resid, gpu_count=1, order=1).astype(np.float32)
            err = float(np.abs(y.astype(np.float32) - ref).max() / np.abs(ref).max())
            out.put((same, err, kb, kc))
    finally:
        dist.destroy_process_group()


def test_hybrid_ffn_on_two_cpu_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, 2, 29611, q)) for r in range(2)]
    for p in procs:
        p.start()
    same, err, kb, kc = q.get(timeout=90)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert same, "ranks disagree on the reduced vector"
    assert err < 4e-3, err
    assert (kb, kc) == (0, 5 * 128)
