"""Decode benchmark of the B200 path: Llama-2 W4 g128, batch 1, 16 synthetic prompt ids + 256 greedy tokens.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--model llama2-7b]

A step is one whole generation (272 positions, the reference's `-n 272`) of the synthetic model. For N > 1 the
script is launched by torchrun, one rank per GPU; the model is sharded Megatron-style across the ranks (strong
scaling: the job is one sequence). Rank 0 prints one JSON line.

  value     tokens/s timed on the device (CUDA events around all positions of the K steps, token loop queued
            without host synchronisation, weights resident in HBM), max over ranks
  e2e       tokens/s of the user-facing call q4_generate(): the reference's generation loop and timing window
            (host synchronisation per token, token ids exchanged through the pinned host mailbox)
  roofline  the dominant kernel against the measured HBM bandwidth
  parity    logits of the first positions of this very model against the CPU oracle, and the token ids of the two
            timed loops against each other; the run FAILS (exit code 1) when either check does not hold
  cpu_baseline  the CPU oracle (OpenMP port of the reference arithmetic) on a bounded sample, rank 0, N = 1
  extra     kernels: every W4 projection shape of the model (and the single 4096x4096 layer) per op, rotated over
            distinct matrices; allreduce (N > 1): peer push vs NCCL per message size; models (N > 1): the larger models
            the metric names for tensor parallelism (13B at TP N; 70B at TP 4 and 8), generated on the device, with the
            share of the step that waits for the exchange
--impl reference runs the reference's own CUDA program (built from the reference sources into oracle/_ref/) on the
same file and prompt, on N GPUs with its own hybrid tensor parallelism; without that build it times the CPU port.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_PROMPT, N_DECODE = 16, 256
STEPS_PER_GEN = N_PROMPT + N_DECODE  # positions per generation (-n 272)
# dram__bytes_read + dram__bytes_write over algorithmic bytes of one fused_token_kernel launch, from the ncu capture
# of this kernel on the 4-layer model of the same layer shapes (traffic grows with the layer count like the bytes do)
FUSED_TRAFFIC_RATIO = 1.023
PARITY_POSITIONS = 4
MAX_REL, MIN_COS = 1e-2, 0.999   # tolerance of the floating-point parity checks


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return json.load(open(p)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.idx)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def model_file(name, rank, dist):
    """Synthetic packed model file shared by all ranks of the node (rank 0 writes it once)."""
    from llama_cu_awq_b200 import synth
    d = os.environ.get("Q4_BENCH_DIR", "/tmp")
    path = os.path.join(d, f"q4b200_{name}_seed0.bin")
    want = synth.file_bytes(synth.CONFIGS[name])
    if rank == 0 and not (os.path.exists(path) and os.path.getsize(path) == want):
        synth.write_model_file(path, name, seed=0)
    if dist is not None:
        dist.barrier()
    return path


def cpu_port(path, prompt, n_tokens, order=0):
    """The CPU oracle on positions 0 .. n_tokens of the same workload (teacher-forced with the prompt): tokens/s over
    positions 1 .. n_tokens (position 0 pages the file in), the thread count, and the logits of every position.
    order 0: plain loops (the timed port); order 1: the reference kernels' own summation order (lane-sequential FMA,
    shuffle tree)."""
    from oracle import q4_oracle as O
    with open(path, "rb") as f:
        m = O.Model(f.read())
    logits = []
    m.forward(int(prompt[0]), 0, order=order)
    logits.append(m.logits().copy())
    t0 = time.perf_counter()
    for pos in range(1, 1 + n_tokens):
        m.forward(int(prompt[pos]), pos, order=order)
        logits.append(m.logits().copy())
    dt = time.perf_counter() - t0
    cores = O.num_threads()
    m.close()
    return n_tokens / dt, cores, logits


def compare(got, ref):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    rel = float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
    cos = float(got @ ref / max(np.linalg.norm(got) * np.linalg.norm(ref), 1e-30))
    return rel, cos


# ---------------------------------------------------------------------------------------------------------------
# reference arm
# ---------------------------------------------------------------------------------------------------------------
REF_CHILD = r"""
import json, sys
sys.path.insert(0, {root!r})
import numpy as np
from oracle import ref_gpu as R
prompt = np.array({prompt!r}, np.int32)
vals = []
for i in range({runs}):
    toks, _, tps, timed, secs = R.generate({path!r}, prompt, {steps}, {vocab}, gpu_count={gpus})
    vals.append((timed, secs))
extra = {{}}
if {kernels}:
    shapes = {shapes!r}
    extra["kernels"] = {{name: {{"us": R.time_q4(kind, K, N, nmat=nmat), "K": K, "N": N}} for name, kind, K, N, nmat in shapes}}
if {gpus} > 1:
    extra["allreduce"] = {{str(2 * c): R.time_allreduce({gpus}, c) for c in (4096, 5120, 8192)}}
print("REFRESULT " + json.dumps({{"vals": vals, "extra": extra}}))
"""


def kernel_shapes(cfg):
    """(name, kind, K, N, distinct matrices) of the W4 ops of one layer, plus the single-layer config of the metric."""
    dim, hid = cfg[0], cfg[1]
    hid8 = hid // 8 * 8
    return [("cfg0_gemv_4096x4096", 0, 4096, 4096, 32), ("o_proj", 0, dim, dim, 32), ("down_proj", 0, hid8, dim, 16),
            ("qkv_matvec", 1, dim, dim, 33), ("ffn_gate_up_silu", 2, dim, hid8, 16)]


def run_reference(args, rank, world):
    from llama_cu_awq_b200 import synth
    if rank != 0:
        return None
    cfg = synth.CONFIGS[args.model]
    prompt = synth.synth_prompt(N_PROMPT, cfg[5], seed=0)
    path = model_file(args.model, 0, None)
    base = {"metric": "decode tok/s @bs1", "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 (int4 weights, fp32 accumulate)",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": f"{args.model} W4 g128, 16 synthetic prompt ids + 256 greedy tokens, batch 1 (-n 272)",
                       "parallelism": f"tp{args.gpus}" if args.gpus > 1 else "none", "l2": "weights per token >> L2"}}
    have_gpu = False
    try:
        import torch
        from oracle import ref_gpu as R
        have_gpu = R.available() and torch.cuda.device_count() >= args.gpus
    except Exception:
        have_gpu = False
    if have_gpu:
        # The reference program itself (llama2_q4.cu): its own loader, kernels, collectives and token loop, -x none on one
        # GPU, -x hybrid with one host thread per GPU on N. It runs in a child process with a time limit: its host-side
        # rendezvous (std::barrier inside every collective, cuda_comm.h:184,223) has no time-out of its own.
        code = REF_CHILD.format(root=ROOT, prompt=[int(v) for v in prompt], runs=args.warmup + args.steps, path=path, steps=STEPS_PER_GEN,
                                vocab=cfg[5], gpus=args.gpus, kernels=args.gpus == 1 and not args.no_extras, shapes=kernel_shapes(cfg))
        sampler = ClockSampler(0)
        sampler.start()
        try:
            r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
            line = [l for l in r.stdout.splitlines() if l.startswith("REFRESULT ")]
            res = json.loads(line[-1][len("REFRESULT "):]) if r.returncode == 0 and line else None
            why = None if res else f"reference program exited with code {r.returncode}: {(r.stderr or r.stdout)[-300:]}"
        except subprocess.TimeoutExpired:
            res, why = None, "reference program did not finish within 600 s on this GPU count (killed)"
        clocks = sampler.stop()
        if res is None:
            return {"impl": "reference", "unavailable": why.replace("\n", " ")}
        vals = res["vals"][args.warmup:]
        tot_t = sum(v[0] for v in vals)
        tot_s = sum(v[1] for v in vals)
        v = tot_t / tot_s
        base.update({"value": v, "ms_per_step": 1e3 * tot_s / len(vals), "clocks": clocks, "gpu_launches": 0,
                     "cpu_baseline": {"value": v, "unit": "tok/s", "cores": 0, "kind": "reference",
                                      "sample": f"the reference's own CUDA program compiled for sm_100a (oracle/_ref), {args.gpus} GPU(s), whole "
                                                "272-position run; the reference has no CPU implementation of this path"},
                     "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                     "extra": res["extra"]})
        if args.gpus > 1:
            base["config"]["note"] = ("the reference's row-split loader misplaces zero points and scales when groups-per-rank is odd or "
                                      "fractional (7B down projection at every N > 1): its outputs differ there, its timing is valid")
    else:
        n = 3
        vals = []
        for i in range(min(args.warmup, 1) + args.steps):
            v, cores, _ = cpu_port(path, prompt, n)
            vals.append(v)
        vals = vals[-args.steps:]
        v = sum(vals) / len(vals)
        base.update({"value": v, "ms_per_step": 1e3 * n / v, "gpu_launches": 0,
                     "cpu_baseline": {"value": v, "unit": "tok/s", "cores": cores, "kind": "port", "sample": f"{n} positions of the same model per step, OpenMP"},
                     "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    return base


# ---------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------
def time_generations(t, prompt, fwd_path, steps, warmup, barrier, torch, dist, on_timed_start=None, prompt_one_pass=False):
    """Device-timed tokens/s over `steps` generations (max over ranks), and the token ids of the last one. With
    prompt_one_pass the prompt positions but the last go through q4_model_prefill (what q4_generate does with
    Q4_PATH_PROMPT_ONE_PASS); the positions counted are the same."""
    def run():
        first = 0
        if prompt_one_pass and N_PROMPT > 1:
            t.prefill(N_PROMPT - 1, gen_token=False)
            first = N_PROMPT - 1
        for pos in range(first, STEPS_PER_GEN - 1):  # the reference counts pos-1 = 271 timed positions per run
            t.forward(gen_token=pos >= N_PROMPT - 1, path=fwd_path)

    def one():
        t.reset(prompt, 0)
        run()

    barrier()   # ranks start together: a rank that comes late (rank 0 runs the CPU oracle) must not leave its peers' kernels waiting
    for _ in range(warmup):
        one()
    t.synchronize()
    barrier()
    if on_timed_start:
        on_timed_start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms = 0.0
    for _ in range(steps):
        t.reset(prompt, 0)  # synchronous; outside the timed region
        barrier()
        with torch.cuda.stream(t.stream):
            e0.record(t.stream)
            run()
            e1.record(t.stream)
        t.synchronize()
        total_ms += e0.elapsed_time(e1)
    barrier()
    tokens = np.array(t.shared().tokens[:STEPS_PER_GEN])
    ms_t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    total_ms = float(ms_t.item())
    return (STEPS_PER_GEN - 1) * steps / (total_ms / 1e3), total_ms, tokens


def op_kernels(cfg, torch, rows=0):
    """Every W4 op of one layer (and the single 4096 x 4096 layer) timed alone over distinct matrices: the batch-1 kernels
    (rows = 0) or their few-rows forms for batched decode with `rows` rows of x."""
    from llama_cu_awq_b200 import _lib
    L = _lib.lib()
    out = {}
    pk, _ = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    s = torch.cuda.Stream()   # a stream of its own: the hook captures a CUDA graph, which the default stream does not allow
    for name, kind, K, N, nmat in kernel_shapes(cfg):
        pw, pz, gg = ((K + 31) // 32) * 4, ((K + 127) // 128 + 7) // 8, (K + 127) // 128
        keep, mats = [], (_lib.q4_qweight * nmat)()
        for i in range(nmat):
            w = torch.randint(-2**31, 2**31 - 1, (N, pw), dtype=torch.int32, device="cuda", generator=g)
            z = torch.randint(-2**31, 2**31 - 1, (N, pz), dtype=torch.int32, device="cuda", generator=g)
            sc = (torch.rand((N, gg), device="cuda", generator=g) * 0.018 + 0.002).half()
            keep += [w, z, sc]
            mats[i] = _lib.q4_qweight(w.data_ptr(), z.data_ptr(), sc.data_ptr())
        x = torch.randn(max(rows, 1) * K, device="cuda", generator=g).half()
        ys = [torch.zeros(max(4, rows) * N, dtype=torch.float16, device="cuda") for _ in range(3)]
        pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        us, nbytes = C.c_double(), C.c_double()
        torch.cuda.synchronize()
        if rows:
            if K % 128 or N % 32:
                continue
            st = L.q4_time_q4_rows_op(C.c_void_p(s.cuda_stream), kind, rows, C.c_void_p(ys[0].data_ptr()), C.c_void_p(ys[1].data_ptr()), C.c_void_p(ys[2].data_ptr()),
                                      C.c_void_p(x.data_ptr()), mats, nmat, K, N, 20, C.byref(us), C.byref(nbytes))
        else:
            st = L.q4_time_q4_op(C.c_void_p(s.cuda_stream), kind, C.c_void_p(ys[0].data_ptr()), C.c_void_p(ys[1].data_ptr()), C.c_void_p(ys[2].data_ptr()),
                                 C.c_void_p(x.data_ptr()), mats, nmat, K, N, 20, C.c_void_p(pos.data_ptr()), C.byref(us), C.byref(nbytes))
        if st != 0:
            out[name] = {"error": st}
            continue
        gbs = nbytes.value / (us.value * 1e-6) / 1e9
        out[name] = {"K": K, "N": N, "us": us.value, "bytes": nbytes.value, "gbs": gbs, "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "distinct_matrices": nmat}
        del keep
    return out


def gemm_table(torch):
    """The batched / prefill W4 dequant-GEMM (tcgen05) at M = 16, 64, 512 on the four 7B projection shapes, over distinct
    weight matrices: against the HBM roofline (algorithmic bytes) and against the measured sustained bf16 tensor rate."""
    from llama_cu_awq_b200 import _lib
    L = _lib.lib()
    pk, _ = peaks()
    g = torch.Generator(device="cuda").manual_seed(1)
    s = torch.cuda.Stream()
    out = {}
    for name, K, N, nmat in (("qkv_4096x12288", 4096, 12288, 6), ("gate_up_4096x22016", 4096, 22016, 4), ("down_11008x4096", 11008, 4096, 6),
                             ("o_4096x4096", 4096, 4096, 16)):
        pw, pz, gg = K // 8, ((K + 127) // 128 + 7) // 8, (K + 127) // 128
        keep, mats, wil = [], (_lib.q4_qweight * nmat)(), (C.c_void_p * nmat)()
        for i in range(nmat):
            w = torch.randint(-2**31, 2**31 - 1, (N, pw), dtype=torch.int32, device="cuda", generator=g)
            z = torch.randint(-2**31, 2**31 - 1, (N, pz), dtype=torch.int32, device="cuda", generator=g)
            sc = (torch.rand((N, gg), device="cuda", generator=g) * 0.018 + 0.002).half()
            wi = torch.empty_like(w)
            L.q4_gemm_interleave_weights(C.c_void_p(s.cuda_stream), C.c_void_p(wi.data_ptr()), C.c_void_p(w.data_ptr()), K, N)
            keep += [w, z, sc, wi]
            mats[i] = _lib.q4_qweight(w.data_ptr(), z.data_ptr(), sc.data_ptr())
            wil[i] = wi.data_ptr()
        wbytes = N * (pw * 4 + pz * 4 + gg * 2)
        for M in (16, 64, 512):
            x = torch.randn((M, K), device="cuda", generator=g).half()
            y = torch.zeros((M, N), dtype=torch.float16, device="cuda")
            nws = L.q4_matmul_q4_batched_workspace_bytes(M, K, N)
            ws = torch.zeros(nws, dtype=torch.uint8, device="cuda")
            us = C.c_double()
            torch.cuda.synchronize()
            st = L.q4_time_matmul_q4_batched(C.c_void_p(s.cuda_stream), C.c_void_p(y.data_ptr()), C.c_void_p(x.data_ptr()), mats, wil, nmat, M, K, N,
                                             C.c_void_p(ws.data_ptr()), nws, 10, C.byref(us))
            if st == 0:
                st = L.q4_matmul_q4_batched_status(C.c_void_p(s.cuda_stream), C.c_void_p(ws.data_ptr()))
            if st != 0:   # a device-side wait ran out: every further launch would cost the wait limit again
                out[f"{name}_M{M}"] = {"error": st}
                return out
            nbytes = wbytes + 2 * M * K + 2 * M * N
            tflops = 2.0 * M * K * N / (us.value * 1e-6) / 1e12
            gbs = nbytes / (us.value * 1e-6) / 1e9
            out[f"{name}_M{M}"] = {"us": us.value, "gbs": gbs, "frac_of_hbm_peak": gbs / pk["hbm_gbs"], "tflops": tflops,
                                   "frac_of_bf16_sustained": tflops / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]),
                                   "bound": "tensor" if M >= 512 else "hbm", "distinct_matrices": nmat}
        del keep
    return out


def allreduce_table(comm, dist, torch):
    """Microseconds per in-place fp16 all-reduce of one model vector (8, 10, 16 KB) and of the [rows x dim] messages of
    batched decode (32-256 KB): peer push (one CTA up to 64 KB, four above) vs NCCL."""
    from llama_cu_awq_b200 import _lib
    L = _lib.lib()
    out = {}
    have_nccl = False
    try:
        comm.attach_nccl(dist)
        have_nccl = True
    except Exception as e:  # NCCL cannot be opened: the table then has the peer push only
        out["nccl_error"] = str(e)[:120]
    s = torch.cuda.current_stream()
    for count in (4096, 5120, 8192, 16384, 32768, 65536, 131072):
        buf = torch.zeros(count, dtype=torch.float16, device="cuda")
        row = {}
        for name, backend in (("p2p_push", _lib.Q4_COMM_BACKEND_P2P), ("nccl", _lib.Q4_COMM_BACKEND_NCCL)):
            if backend == _lib.Q4_COMM_BACKEND_NCCL and not have_nccl:
                continue
            comm.set_backend(backend)
            torch.cuda.synchronize()
            dist.barrier()
            us = C.c_double()
            st = L.q4_time_all_reduce(comm.handle, C.c_void_p(s.cuda_stream), C.c_void_p(buf.data_ptr()), count, 200, C.byref(us))
            v = torch.tensor([us.value if st == 0 else -1.0], dtype=torch.float64, device="cuda")
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
            row[name] = float(v.item())
        out[str(2 * count)] = row
    comm.set_backend(_lib.Q4_COMM_BACKEND_P2P)
    out["unit"] = "us per call, max over ranks, 200 calls back to back"
    return out


def prefill_and_batch(t, cfg, fwd_path, value, rank, world, dist, torch, barrier, pk, per_op_anchor=True):
    """The two callers either side of the batch-1 decode step on the same model: a 512-token prompt processed in one
    pass (W4 GEMMs on the tensor cores) against the same 512 positions fed token by token, and eight sequences decoded
    together against eight times the batch-1 rate."""
    from llama_cu_awq_b200 import synth
    from llama_cu_awq_b200.model import Batch
    out = {}
    n_pre = 512
    ids = synth.synth_prompt(n_pre, cfg[5], seed=1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps):
        best = []
        for _ in range(reps):
            t.reset(ids, 0)
            barrier()
            with torch.cuda.stream(t.stream):
                e0.record(t.stream)
                fn()
                e1.record(t.stream)
            t.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
            if dist is not None:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            best.append(float(ms.item()))
        return sum(best[1:]) / (len(best) - 1)   # the first repetition warms up (workspaces, interleaved weight copies)

    def by_token():
        for _ in range(n_pre):
            t.forward(gen_token=False, path=fwd_path)

    def by_token_per_op():
        for _ in range(n_pre):
            t.forward(gen_token=False, path=1)

    ms_pre = timed(lambda: t.prefill(n_pre, gen_token=False), 4)
    one_pass = t.logits()
    ms_tok = timed(by_token, 2)
    fused = t.logits()
    if per_op_anchor:
        timed(by_token_per_op, 2)
        per_op = t.logits()   # the per-op kernels follow the reference's arithmetic op by op: the anchor of this comparison
        rel, cos = compare(one_pass, per_op)
        rel_f, cos_f = compare(fused, per_op)
    else:
        rel, cos = compare(one_pass, fused)
        rel_f, cos_f = None, None
    n_layers, dim, hidden = cfg[2], cfg[0], cfg[1]
    kv_dim = dim * cfg[4] // cfg[3]
    flops = 2.0 * n_pre * n_layers * (2 * dim * dim + 2 * dim * kv_dim + 3 * dim * hidden) / world
    out["prefill_512"] = {"ms": ms_pre, "tok_s": n_pre / ms_pre * 1e3, "ms_token_by_token": ms_tok, "speedup_vs_token_by_token": ms_tok / ms_pre,
                          "w4_gemm_tflops_per_gpu": flops / (ms_pre * 1e-3) / 1e12, "frac_of_bf16_sustained": flops / (ms_pre * 1e-3) / 1e12 / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]),
                          # position 511 of a 32-layer random-weight model: every path (this one, the fused token kernel) lies this far from
                          # the per-op kernels, whose own distance to the oracle grows the same way with depth and position
                          ("last_logits_vs_per_op_path" if per_op_anchor else "last_logits_vs_fused_token_path"): {"max_rel": rel, "cosine": cos},
                          "fused_token_path_vs_per_op_path": {"max_rel": rel_f, "cosine": cos_f}, "status": t.status()}

    n_seq, steps = 8, 64
    b = Batch(t, n_seq)
    prompts = np.stack([synth.synth_prompt(N_PROMPT, cfg[5], seed=10 + i) for i in range(n_seq)])
    times = []
    for rep in range(3):
        b.reset(prompts)
        for _ in range(N_PROMPT):
            b.forward()
        t.synchronize()
        barrier()
        with torch.cuda.stream(t.stream):
            e0.record(t.stream)
            for _ in range(steps):
                b.forward()
            e1.record(t.stream)
        t.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        times.append(float(ms.item()))
    ms_step = sum(times[1:]) / (len(times) - 1) / steps
    out["batch8_decode"] = {"ms_per_step": ms_step, "tok_s_all_sequences": n_seq / ms_step * 1e3, "vs_batch1_rate": n_seq / ms_step * 1e3 / value,
                            "positions": f"{N_PROMPT}..{N_PROMPT + steps}", "status": t.status()}
    b.close()
    return out


def extra_model(name, rank, world, dist, torch, barrier, pk):
    """A larger model of the metric at this tensor-parallel degree, generated on the device: tok/s, fraction of the
    weight-streaming roofline, and the share of the step that waits for the exchange between the ranks (step time minus
    the same step with every rank's exchange kept inside its own memory, measured with the test build of the library)."""
    from llama_cu_awq_b200 import _lib, synth
    from llama_cu_awq_b200.comm import ProcessComm
    from llama_cu_awq_b200.model import Transformer
    cfg = synth.CONFIGS[name]
    prompt = synth.synth_prompt(N_PROMPT, cfg[5], seed=0)
    res = {}
    for which in ("product", "test_build", "exchange_local"):
        lib = _lib.lib() if which == "product" else _lib.test_lib()
        if which == "exchange_local":
            lib.q4_test_set_fused_debug(16)
        comm = ProcessComm(rank, world, dist, lib=lib)
        t = Transformer(None, rank=rank, gpu_count=world, tp_mode=_lib.Q4_TP_HYBRID, comm=comm.handle, lib=lib, synthetic=(cfg, 0))
        ok = torch.tensor([1 if t.best_path() == 2 else 0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) != 1:
            t.close(); comm.close()
            return {"error": "the fused path does not serve this model at this degree"}
        barrier()
        toks, total_ms, tokens = time_generations(t, prompt, 2, 2, 1, barrier, torch, dist)
        st = t.status()
        if which == "product":
            mean_bytes = sum(t.token_bytes(p) for p in range(STEPS_PER_GEN - 1)) / (STEPS_PER_GEN - 1)
            res.update({"tok_s": toks, "us_per_token": 1e6 / toks, "bytes_per_token_per_gpu": mean_bytes,
                        "token_roofline_frac": mean_bytes * toks / 1e9 / pk["hbm_gbs"], "status": st})
            try:   # the same model's 512-token prefill and batch-8 decode at this degree
                if _lib.lib().q4_comm_nccl_available():
                    comm.attach_nccl(dist)
                    comm.set_backend(_lib.Q4_COMM_BACKEND_AUTO)
                res.update(prefill_and_batch(t, cfg, 2, toks, rank, world, dist, torch, barrier, pk, per_op_anchor=False))
            except Exception as e:
                res["prefill_batch_error"] = str(e)[:300]
        elif which == "test_build":
            res["exchange"] = {"us_per_token": 1e6 / toks, "build": "test build of the library (same kernel plus its measurement switches)"}
        else:
            lib.q4_test_set_fused_debug(0)
            res["exchange"]["us_per_token_exchange_kept_local"] = 1e6 / toks
            res["exposed_exchange_pct"] = 100.0 * (res["exchange"]["us_per_token"] - 1e6 / toks) / res["exchange"]["us_per_token"]
        t.close()
        comm.close()
        barrier()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="llama2-7b")
    ap.add_argument("--path", type=int, default=-1, help="forward path: 1 = CUDA-graph replay of per-op kernels (default: best available)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-op kernel table, the all-reduce table and the larger models")
    ap.add_argument("--leg", default="all", choices=["all", "prefill-batch"],
                    help="prefill-batch: only the 512-token prefill and the batch-8 decode of --model (profiling-sized run; prints their numbers, not the metric line)")
    ap.add_argument("--positions", type=int, default=0, help="positions per generation (default 272 = 16 prompt + 256 decode); smaller for profiling runs")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = max(args.warmup, 1)

    global STEPS_PER_GEN
    if args.positions > N_PROMPT:
        STEPS_PER_GEN = args.positions
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line))
        return

    import torch
    from llama_cu_awq_b200 import _lib, synth
    from llama_cu_awq_b200.model import Transformer
    from llama_cu_awq_b200.comm import ProcessComm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = synth.CONFIGS[args.model]
    prompt = synth.synth_prompt(N_PROMPT, cfg[5], seed=0)
    path = model_file(args.model, rank, dist)

    comm = ProcessComm(rank, world, dist) if world > 1 else None
    t = Transformer(path, rank=rank, gpu_count=world, tp_mode=_lib.Q4_TP_HYBRID if world > 1 else _lib.Q4_TP_NONE,
                    comm=comm.handle if comm else None)
    fwd_path = args.path if args.path >= 0 else t.best_path()
    if fwd_path == 2 and t.best_path() != 2:
        raise SystemExit("--path 2: the fused path does not serve this model")
    if dist is not None:
        # all ranks take the same path, and with the fused path (whose kernels exchange activations between the
        # ranks) every rank is prepared before any rank launches
        fp = torch.tensor([fwd_path], device="cuda")
        dist.all_reduce(fp, op=dist.ReduceOp.MIN)
        fwd_path = int(fp.item())

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    if args.leg == "prefill-batch":
        pk, _ = peaks()
        if comm is not None and _lib.lib().q4_comm_nccl_available():
            comm.attach_nccl(dist)
            comm.set_backend(_lib.Q4_COMM_BACKEND_AUTO)
        res = prefill_and_batch(t, cfg, fwd_path, 1.0, rank, world, dist, torch, barrier, pk, per_op_anchor=False)
        res["batch8_decode"].pop("vs_batch1_rate", None)
        if rank == 0:
            print(json.dumps({"leg": "prefill-batch", "model": args.model, "n_gpus": world, **res}))
        t.close()
        if comm:
            comm.close()
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- device-timed value ----
    sampler = ClockSampler(local_rank)
    value, total_ms, tokens_dev = time_generations(t, prompt, fwd_path, args.steps, args.warmup, barrier, torch, dist,
                                                   on_timed_start=sampler.start if rank == 0 else None)
    timed_tokens = (STEPS_PER_GEN - 1) * args.steps

    # ---- end to end through the public generation call ----
    t.generate(prompt, STEPS_PER_GEN, path=fwd_path)
    barrier()
    e2e_tok, e2e_sec = 0, 0.0
    for _ in range(args.steps):
        barrier()
        toks, timed, secs = t.generate(prompt, STEPS_PER_GEN, path=fwd_path)
        st = torch.tensor([secs], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        e2e_tok += timed
        e2e_sec += float(st.item())
    e2e = e2e_tok / e2e_sec
    clocks = sampler.stop() if rank == 0 else None
    tokens_match = bool((tokens_dev == toks[:STEPS_PER_GEN]).all())
    if dist is not None:   # and every rank holds the same ids
        mine = torch.from_numpy(np.concatenate([tokens_dev, toks[:STEPS_PER_GEN]]).astype(np.int64)).cuda()
        lo, hi = mine.clone(), mine.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        tokens_match = tokens_match and bool(torch.equal(lo, hi))

    # ---- parity of this very model: first positions against the CPU oracle (which is also the timed CPU baseline) ----
    parity = {"tokens_match_e2e": tokens_match, "limits": {"max_rel": MAX_REL, "cosine": MIN_COS}}
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        cpu = cpu_port(path, prompt, PARITY_POSITIONS)
    t.reset(prompt, 0)
    barrier()
    got = []
    for pos in range(PARITY_POSITIONS + 1):
        t.forward(gen_token=False, path=fwd_path)
        t.synchronize()
        got.append(t.logits())
    if cpu is not None:
        rels, coss = zip(*[compare(a, b) for a, b in zip(got, cpu[2])])
        parity.update({"positions": len(rels), "max_rel": max(rels), "cosine": min(coss), "against": "CPU oracle, same file, teacher-forced prompt"})
        # How far two faithful evaluations of the reference arithmetic lie apart on this very model: the oracle in the
        # reference kernels' summation order against the oracle with plain loops (fp32 sums in another order, nothing
        # else). Thirty-two layers of random weights amplify a last-bit difference, so this, not the per-op tolerance, is
        # the resolution of a whole-model logits comparison.
        ref_order = cpu_port(path, prompt, PARITY_POSITIONS, order=1)
        floor = max(compare(a, b)[0] for a, b in zip(ref_order[2], cpu[2]))
        rels1 = [compare(a, b)[0] for a, b in zip(got, ref_order[2])]
        parity.update({"oracle_reorder_max_rel": floor, "max_rel_vs_reference_order": max(rels1),
                       "accept": "cosine >= limit and max_rel <= max(limit, 2 x oracle_reorder_max_rel)"})
    parity["device_status"] = t.status()
    parity["ok"] = bool(tokens_match and parity["device_status"] == 0 and
                        (cpu is None or (parity["cosine"] >= MIN_COS and parity["max_rel"] <= max(MAX_REL, 2.0 * parity["oracle_reorder_max_rel"]))))

    # ---- dominant kernel against the HBM roofline ----
    pk, pk_kind = peaks()
    mean_bytes = sum(t.token_bytes(p) for p in range(STEPS_PER_GEN - 1)) / (STEPS_PER_GEN - 1)
    token_gbs = mean_bytes * value / 1e9
    extra = {}
    if world == 1 and not args.no_extras:
        extra["kernels"] = op_kernels(cfg, torch)
        extra["kernels_rows8"] = op_kernels(cfg, torch, rows=8)
        extra["gemm_tcgen05"] = gemm_table(torch)
    if fwd_path == 2:
        launches_per_token = 1  # one persistent cooperative kernel per token
        roof = {"bound": "hbm", "kernel": "fused_token_kernel (whole token: W4 GEMVs, attention, classifier)",
                "achieved": token_gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": token_gbs / pk["hbm_gbs"], "peak_kind": pk_kind,
                "traffic": FUSED_TRAFFIC_RATIO * mean_bytes, "traffic_source": "ncu capture of this kernel on the 4-layer model of the same layer shapes, scaled by algorithmic bytes",
                "bytes_per_launch": mean_bytes, "us_per_launch": 1e6 / value}
    else:
        launches_per_token = 4 + 9 * cfg[2] + (2 * cfg[2] + 1 if world > 1 else 0)
        k = (extra.get("kernels") or {}).get("ffn_gate_up_silu") or {}
        roof = {"bound": "hbm", "kernel": "q4_gemv_kernel (fused gate/up + SiLU)", "achieved": k.get("gbs"), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": k.get("frac_of_hbm_peak"), "peak_kind": pk_kind, "traffic": None, "bytes_per_launch": k.get("bytes"), "us_per_launch": k.get("us")}
    if not args.no_extras:
        try:
            # The same workload with the prompt (but its last position) in one pass, as a user of q4_generate gets it with
            # Q4_PATH_PROMPT_ONE_PASS: the metric above keeps the reference's token-by-token prompt so that the two arms
            # measure the same thing.
            v1, _, tok1 = time_generations(t, prompt, fwd_path, max(1, args.steps - 1), 1, barrier, torch, dist, prompt_one_pass=True)
            barrier()
            toks1, timed1, secs1 = t.generate(prompt, STEPS_PER_GEN, path=fwd_path, prompt_one_pass=True)
            st1 = torch.tensor([secs1], dtype=torch.float64, device="cuda")
            if dist is not None:
                dist.all_reduce(st1, op=dist.ReduceOp.MAX)
            extra["prompt_one_pass"] = {"value": v1, "e2e": timed1 / float(st1.item()), "unit": "tok/s",
                                        "tokens_match_e2e": bool((tok1 == toks1[:STEPS_PER_GEN]).all()),
                                        "first_generated_id_matches_token_by_token": bool(tok1[N_PROMPT] == tokens_dev[N_PROMPT])}
        except Exception as e:
            extra["prompt_one_pass_error"] = str(e)[:300]
        try:
            if comm is not None and _lib.lib().q4_comm_nccl_available():
                comm.attach_nccl(dist)   # the [rows x dim] all-reduces of the GEMM paths go through NCCL; one-token ones stay on the peer push
                comm.set_backend(_lib.Q4_COMM_BACKEND_AUTO)
            extra.update(prefill_and_batch(t, cfg, fwd_path, value, rank, world, dist, torch, barrier, pk))
        except Exception as e:   # reported, not fatal: the headline line stays valid
            extra["prefill_batch_error"] = str(e)[:300]
    if not args.no_extras:
        extra["status_after_extras"] = t.status()   # 0, or the code a bounded device-side wait recorded during the extra legs
    t.close()
    if comm:
        comm.close()

    # ---- N > 1: the collectives alone, and the models the metric names for tensor parallelism ----
    if world > 1 and not args.no_extras:
        c2 = ProcessComm(rank, world, dist)
        extra["allreduce"] = allreduce_table(c2, dist, torch)
        c2.close()
        barrier()
        models = {}
        names = ["llama2-13b"] + (["llama2-70b"] if world >= 4 else [])
        for name in names:
            try:
                models[f"{name}_tp{world}"] = extra_model(name, rank, world, dist, torch, barrier, pk)
            except Exception as e:  # reported, not fatal: the headline line stays valid
                models[f"{name}_tp{world}"] = {"error": str(e)[:200]}
                break
        extra["models"] = models

    line = {
        "metric": "decode tok/s @bs1", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 (int4 weights, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"{args.model} W4 g128, 16 synthetic prompt ids + {STEPS_PER_GEN - N_PROMPT} greedy tokens, batch 1 (-n {STEPS_PER_GEN})",
                   "parallelism": f"tp{world}" if world > 1 else "none", "forward_path": fwd_path,
                   "l2": "inputs larger than L2 (weights per token >> 126 MB); no flush needed",
                   "tokens_match_e2e": tokens_match},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 4 * N_PROMPT + 4 * STEPS_PER_GEN, "d2h_bytes_per_step": 8 * STEPS_PER_GEN},
        "gpu_launches": launches_per_token * timed_tokens,
        "roofline": roof,
        "token_roofline": {"bytes_per_token_per_gpu": mean_bytes, "achieved_gbs_per_gpu": token_gbs, "frac": token_gbs / pk["hbm_gbs"],
                           "frac_of_nominal_8tbs": token_gbs / 8000.0},
        "parity": parity,
        "extra": extra,
    }
    if cpu is not None and world == 1:
        line["cpu_baseline"] = {"value": cpu[0], "unit": "tok/s", "cores": cpu[1], "kind": "port",
                                "sample": f"positions 1-{PARITY_POSITIONS} of the same model and prompt, CPU oracle (OpenMP over output columns)"}
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    if not parity["ok"]:
        if rank == 0:
            print("bench.py: parity check failed (see the `parity` block): the numbers above are not valid", file=sys.stderr)
        sys.exit(1)


if __name__ == "__main__":
    main()
