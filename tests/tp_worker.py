"""Worker of the tensor-parallel GPU test: launched by torchrun, one rank per GPU (see test_tp_gpu.py).
Loads a synthetic model sharded Megatron-style over the ranks, teacher-forces a token sequence and checks the
logits against the single-GPU oracle; all ranks must hold bit-identical logits (fixed-order fp32 all-reduce)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from llama_cu_awq_b200 import _lib, synth  # noqa: E402
from llama_cu_awq_b200.comm import ProcessComm  # noqa: E402
from llama_cu_awq_b200.model import Batch, Transformer  # noqa: E402


def collectives_mode(comm, rank, world):
    """q4_all_reduce / q4_all_gather alone: short vectors (one CTA), long ones (several CTAs with their own flags and
    counters) and the two kinds interleaved, several rounds without any host synchronisation in between; the result must
    be, bit for bit, the fp32 sum in rank order rounded once - on every rank."""
    import ctypes as C
    L = _lib.lib()
    s = torch.cuda.current_stream()
    ok = 1
    counts = [8, 4096, 16384, 16392, 40960, 65536, 131072, 5120, 131072, 8]
    for rnd in range(3):
        bufs, wants = [], []
        for i, n in enumerate(counts):
            parts = [np.random.default_rng(1000 * rnd + 10 * i + r).standard_normal(n).astype(np.float16) for r in range(world)]
            acc = np.zeros(n, np.float32)
            for r in range(world):
                acc += parts[r].astype(np.float32)
            wants.append(acc.astype(np.float16))
            bufs.append(torch.from_numpy(parts[rank].copy()).cuda())
        torch.cuda.synchronize()
        dist.barrier()
        for b, n in zip(bufs, counts):     # queued back to back
            assert L.q4_all_reduce(comm.handle, C.c_void_p(s.cuda_stream), C.c_void_p(b.data_ptr()), n) == 0
        torch.cuda.synchronize()
        for b, w, n in zip(bufs, wants, counts):
            if not (b.cpu().numpy().view(np.uint16) == w.view(np.uint16)).all():
                print(f"rank {rank}: all-reduce of {n} halfs (round {rnd}) differs from the rank-order fp32 sum")
                ok = 0
    n = 4000
    mine = torch.from_numpy(np.random.default_rng(rank).standard_normal(n).astype(np.float16)).cuda()
    out = torch.zeros(world * n, dtype=torch.float16, device="cuda")
    assert L.q4_all_gather(comm.handle, C.c_void_p(s.cuda_stream), C.c_void_p(mine.data_ptr()), C.c_void_p(out.data_ptr()), n) == 0
    torch.cuda.synchronize()
    want = np.concatenate([np.random.default_rng(r).standard_normal(n).astype(np.float16) for r in range(world)])
    if not (out.cpu().numpy().view(np.uint16) == want.view(np.uint16)).all():
        print(f"rank {rank}: all-gather differs")
        ok = 0
    assert L.q4_all_reduce(comm.handle, C.c_void_p(s.cuda_stream), C.c_void_p(out.data_ptr()), 131072 + 8) == _lib.Q4_ERR_LIMIT
    assert comm.status() == 0
    if rank == 0:
        print(f"TP{world} collectives: ranks identical: {bool(ok)}")
    return ok


def batch_mode(t, comm, cfg_name, path, rank, world):
    """Three sequences decoded together on the sharded model (q4_batch_*): eight prompt positions, then four generated ones;
    each sequence's logits against the single-GPU oracle fed the same ids, every rank holding the same bits."""
    vocab = synth.CONFIGS[cfg_name][5]
    prompts = np.random.default_rng(1).integers(3, vocab, size=(3, 8), dtype=np.int32)
    b = Batch(t, 3)
    runs = []
    for _ in range(2):   # twice: the step graph is replayed, and the results must repeat bit for bit
        b.reset(prompts)
        dist.barrier()
        for _ in range(12):
            b.forward()
        t.synchronize()
        runs.append((b.logits().copy(), b.tokens(13).copy()))
    assert t.status() == 0 and comm.status() == 0
    ok = 1
    if not ((runs[0][0].view(np.uint16) == runs[1][0].view(np.uint16)).all() and (runs[0][1] == runs[1][1]).all()):
        print(f"rank {rank}: batched decode differs between two runs")
        ok = 0
    logits, toks = runs[0]
    mine = torch.from_numpy(logits.view(np.int16).astype(np.int32)).cuda()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    if rank == 0:
        from oracle import q4_oracle as O
        ok = ok if all(torch.equal(gathered[0], g) for g in gathered[1:]) else 0
        image = open(path, "rb").read()
        worst = 0.0
        for s in range(3):
            assert (toks[s, :8] == prompts[s]).all()
            m = O.Model(image)
            for pos in range(12):
                m.forward(int(toks[s, pos]), pos, order=1)
            ref, got = m.logits().astype(np.float64), logits[s].astype(np.float64)
            err = np.abs(got - ref).max() / np.abs(ref).max()
            cos = got @ ref / (np.linalg.norm(got) * np.linalg.norm(ref))
            worst = max(worst, err)
            if err > 1e-2 or cos < 0.999:
                print(f"sequence {s}: rel err {err:.3e} cos {cos:.6f}")
                ok = 0
        print(f"TP{world} {cfg_name} batched decode: worst rel err vs single-GPU oracle {worst:.3e}; ranks identical: {bool(ok)}")
    b.close()
    return ok


def main():
    cfg_name, path, fwd_path = sys.argv[1], sys.argv[2], int(sys.argv[3])
    tp_mode = _lib.Q4_TP_COLUMN if len(sys.argv) > 4 and sys.argv[4] == "column" else _lib.Q4_TP_HYBRID
    synthetic = len(sys.argv) > 5 and sys.argv[5] == "synthetic"   # shards generated on the device; `path` holds the same model as a file
    nccl = len(sys.argv) > 5 and sys.argv[5] == "nccl"             # per-op paths: collectives through NCCL instead of the peer push
    prefill = len(sys.argv) > 5 and sys.argv[5] in ("prefill", "prefill-p2p")   # the first 17 positions in one pass (GEMM path), the rest token by token
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = ProcessComm(rank, world, dist)
    if nccl:
        comm.attach_nccl(dist)
        comm.set_backend(_lib.Q4_COMM_BACKEND_NCCL)
    if prefill and sys.argv[5] == "prefill":   # large all-reduces of the prefill through NCCL, the decode steps' small ones stay on the peer push
        comm.attach_nccl(dist)
        comm.set_backend(_lib.Q4_COMM_BACKEND_AUTO)
    if len(sys.argv) > 5 and sys.argv[5] == "collectives":
        ok = collectives_mode(comm, rank, world)
        flag = torch.tensor([ok], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if int(flag.item()) == 1 else 1)
    t = Transformer(path, rank=rank, gpu_count=world, tp_mode=tp_mode, comm=comm.handle,
                    synthetic=(synth.CONFIGS[cfg_name], 7) if synthetic else None)
    vocab = synth.CONFIGS[cfg_name][5]
    tokens = np.random.default_rng(0).integers(3, vocab, size=24, dtype=np.int32)
    t.reset(tokens, 0)
    if fwd_path == 2:
        assert t.best_path() == 2, "the fused path must serve this sharded model"
    dist.barrier()   # the fused path exchanges activations between the ranks' kernels: all ranks prepared before any launches
    torch.cuda.synchronize()
    if len(sys.argv) > 5 and sys.argv[5] == "batch":
        ok = batch_mode(t, comm, cfg_name, path, rank, world)
        flag = torch.tensor([ok], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        t.close()
        comm.close()
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if int(flag.item()) == 1 else 1)

    def run(sync_every_token):
        out = []
        t.reset(tokens, 0)
        dist.barrier()
        first = 0
        if prefill:
            first = 17
            t.prefill(first, gen_token=False)
            t.synchronize()
            out += [None] * (first - 1) + [t.logits()]
        for pos in range(first, len(tokens)):
            t.forward(gen_token=False, path=fwd_path)
            if sync_every_token or pos == len(tokens) - 1:
                t.synchronize()
                out.append(t.logits())
        assert t.status() == 0 and comm.status() == 0
        return out

    logits = run(True)
    # run-to-run reproducibility: a second pass with per-token waits and one queued without any (last position compared)
    again, queued = run(True), run(False)
    same = all((a.view(np.uint16) == b.view(np.uint16)).all() for a, b in zip(logits, again) if a is not None)
    same = same and (queued[-1].view(np.uint16) == logits[-1].view(np.uint16)).all()
    mine = torch.from_numpy(np.stack([l for l in logits if l is not None]).view(np.int16).astype(np.int32)).cuda()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    ok = 1 if same else 0
    if not same:
        print(f"rank {rank}: logits differ between two runs of the same sequence")
    if rank == 0:
        from oracle import q4_oracle as O
        for r in range(1, world):
            if not torch.equal(gathered[0], gathered[r]):
                print(f"rank {r} logits differ from rank 0")
                ok = 0
        m = O.Model(open(path, "rb").read())
        worst = 0.0
        for pos, tok in enumerate(tokens):
            m.forward(int(tok), pos, order=1)
            if logits[pos] is None:
                continue
            ref = m.logits().astype(np.float64)
            got = logits[pos].astype(np.float64)
            err = np.abs(got - ref).max() / np.abs(ref).max()
            cos = got @ ref / (np.linalg.norm(got) * np.linalg.norm(ref))
            worst = max(worst, err)
            if err > 1e-2 or cos < 0.999:
                print(f"pos {pos}: rel err {err:.3e} cos {cos:.6f}")
                ok = 0
        print(f"TP{world} {cfg_name}: worst rel err vs single-GPU oracle {worst:.3e}; ranks identical: {bool(ok)}")
    flag = torch.tensor([ok], device="cuda")
    dist.broadcast(flag, 0)
    t.close()
    comm.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
