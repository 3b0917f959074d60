// Fused decode path: ONE persistent cooperative kernel per token (one CTA per SM) instead of ~9 launches per layer.
// Replaces the launch sequence of run_llama_network (llama2_q4.cu:430-538), on one GPU or on every rank of a
// tensor-parallel group (hybrid split, llama2_q4.cu:45-50).
//
// Why: a 7B layer is 105 MB of weights = 16 us of HBM time; nine kernel boundaries per layer cost as much as the
// streaming itself. Weight addresses never depend on activations, so each CTA has a PRODUCER warp that walks the
// CTA's precomputed copy list and keeps a shared-memory ring (up to 12 entries of two slots) full with
// cp.async.bulk (TMA, 1-D, no multicast), running ahead across op boundaries, while 11 CONSUMER warps do the math.
// Dependent ops are separated by tagged activation words that the readers poll (see FParams), not by grid barriers.
//
// Stream layout (built once per matrix on the device from the file layout, bytes per weight unchanged):
//   unit  = 8 output columns x 1 group of 128 inputs = 512 B of nibbles + 32 B metadata (8 fp16 scales, 8 u8 zeros)
//   block = (8-column tile rt, k-tile kt of <= 16 groups): [2 chunk pairs][8 rows][lane] uint4, then [group] metadata,
//           so that one bulk copy fills a slot and every LDS.128 is conflict free (lane l = 2*group + half).
//   blocks are stored [rt][kt]; a block is ng*544 bytes, ng = min(16, G - 16*kt).
//
// Arithmetic of the W4 dot product (consumer): activations are re-expressed per group of 128 as 15-bit block
// fixed point X = rint(x / sx), sx = max|x| / 16256, split into two int8 digits (X = 128*xh + xl). Nibbles are
// extracted four at a time with one AND (even nibbles) / one AND (odd nibbles, kept as 16*q) and multiplied with
// DP4A into int32 accumulators: exact integer arithmetic, 6 instructions per 8 weights (the half2 FMA pipe of
// this GPU issues at half rate, which made the half2 formulation pipe-bound at ~50 % of HBM bandwidth). Per
// (column, group): y += scale * sx * (128*Sh + Sl - zero * sum(X)). The quantisation step of x is max|x|/32512 per
// element, below fp16's own rounding of the largest elements; nibbles, zero points and scales are used exactly.
//
// Every wait is bounded (mbarrier polls, tag polls and barrier spins are limited by the global timer); on expiry the
// kernel records Q4_ERR_TIMEOUT in a status word, all later waits fall through, and the kernel returns.
#include <math_constants.h>
#include <stdio.h>
#include <stdlib.h>

#include "q4_comm_internal.h"
#include "q4_model.h"

namespace {

constexpr int kSlotGroups = 16;
constexpr int kUnitBytes = 544;
constexpr int kSlotBytes = kSlotGroups * kUnitBytes;  // 8704
constexpr int kMaxEntries = 12;                    // ring entries: two slots each, filled by one bulk copy; the host picks
constexpr int kMinEntries = 4;                     // as many as fit next to the activation buffers (p.n_entries)
constexpr int kEntryBytes = 2 * kSlotBytes;
#ifndef Q4_FUSED_CW
#define Q4_FUSED_CW 11
#endif
constexpr int kCW = Q4_FUSED_CW;       // consumer warps (+1 producer warp: 12 warps = 3 per SM sub-partition)
constexpr int kCT = kCW * 32;          // consumer threads
constexpr int kAG = kCT / 8;           // attention lane groups (positions in flight per CTA)
static_assert(kCT % 16 == 0, "activation staging maps 16 consecutive threads to one group of 128 inputs");
constexpr int kThreads = 32 + kCT;     // + producer warp
constexpr int kSplitLen = 128;         // positions per attention split before a head is split further (measured best on 7B at 16..272 positions: 48 and 192 are 1 % slower, unsplit 3 %)
constexpr int kMaxSplit = 4;           // attention splits per head (merged in registers by the next phase)
constexpr int kAttnPartStride = 128 + 4;   // tagged words per attention partial: 128 outputs as fp16 (normalised by the split's own sum),
                                           // then max and sum as two 16-bit pieces each
constexpr int kTraceCols = 8;           // timestamps per phase: 0 start, 1 inputs staged, 2 weights consumed, 3 barrier passed, 4-7 staging detail
constexpr int kMaxUnitsPerCta = 64;    // units of one phase per CTA (host-checked)
constexpr int kClsChunk = 4096;        // halfs of one classifier row per slot (8192 B)
constexpr unsigned kPollLimit = 1u << 26;                        // polls, and
constexpr unsigned long long kDefaultWaitNs = 2000ULL * 1000 * 1000;  // default limit of a device-side wait: two seconds on the global timer (FParams::wait_ns)

// Measurement and test switches of the kernel (skip the math, skip the streaming, keep the exchange local) exist only in the
// test build of the library; in the product build the expression is the constant 0 and the branches are compiled out.
#ifdef Q4_TEST_BUILD
#define Q4_DBG(p) ((p).debug)
#else
#define Q4_DBG(p) 0
#endif

enum PhaseType { PH_EMBED = 0, PH_GEMV = 1, PH_ATTN = 2, PH_CLS = 3, PH_ARGMAX = 4 };
enum EpiKind { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU = 2 };

struct FMat {
    const uint8_t* blocks;  // stream layout
    uint32_t* out;          // tagged output vector (value | tag << 16), see "tagged activations" below
    __half* out_plain;      // V projection only: the KV cache (row pos at loff), written untagged as well
    int n;                  // outputs of this matrix
    int tile0;              // first tile of this matrix in the phase's tile space
};

struct FPhase {
    int type;
    int K, G, nkt;          // GEMV: inputs, groups, k-tiles; CLS: K = dim, nkt = chunks per row
    const uint32_t* xin;    // tagged activations (global), written by phase in_phase
    int in_phase;           // index of the phase that produced xin (its tag is what the readers wait for)
    int barrier_after;      // 1: grid barrier after this phase (else the consumers of its output wait on the tags)
    const __half* norm_w;   // RMSNorm weight applied while staging x, or null
    int nmat;
    int xbuf_out;           // EPI_RESIDUAL: residual-stream buffer this phase writes (it reads the other one)
    FMat m[3];
    int nunits, tpu;        // work units of the phase and tiles per unit (2 for gate/up pairs)
    int epi;
    long long loff;         // KV cache layer offset (halfs)
    int layer;
    int attn_in;            // GEMV: the input vector is the attention output, still split: merge the partials while staging
    int next_norm_n;        // elements of next_norm_w
    int xbuf_in;            // 0/1: the input is that buffer of the residual stream (sum of the ranks' partials); -1: xin
    const __half* next_norm_w;  // RMSNorm weight of the next phase that has one: requested into L2 one phase early
};
static_assert(sizeof(FPhase) % 16 == 0, "FPhase is copied in 16-byte pieces");

// One ring entry's copy, precomputed per CTA when the model is prepared (the list is the same for every token):
// the single producer thread only has to wait for a free entry and issue it.
struct CopyDesc {
    const uint8_t* src0;
    const uint8_t* src1;   // second piece when the entry's two slots are not adjacent in memory, else null
    uint32_t bytes0, bytes1;
    uint32_t pad[2];
};
static_assert(sizeof(CopyDesc) == 32, "CopyDesc is loaded as two 128-bit words");

struct FParams {
    const CopyDesc* desc;    // [grid][desc_stride]
    const int* desc_count;   // [grid]
    int desc_stride;
    const FPhase* phases;
    int nphases;
    q4_config cfg;
    int head_size, kv_n, kv_mul, n_heads, nsplit;
    float gpu_count;
    // state
    // Tagged activations: every element is a 32-bit word, fp16 value in the low half and the low 16 bits of
    // (tag_base + producing phase + 1) in the high half. A reader that needs the whole vector polls the words
    // themselves until all carry the expected tag, so most op boundaries need no grid barrier: one L2 round trip
    // instead of fence + arrive + poll. A buffer is rewritten only after every CTA has provably read it (the next
    // writer's own input wait implies it; phases with fewer units than CTAs end with a grid barrier, because a CTA
    // without units writes nothing that anyone waits for and could otherwise fall behind unnoticed).
    //
    // The residual stream is the one vector that all ranks of a tensor-parallel group share. It lives in the exchange
    // area of the communicator as g partial vectors ("slots", one per source rank) in two alternating buffers:
    // buffer 1 is written by the embedding and by every down projection, buffer 0 by every o projection. A rank's
    // epilogue stores half(own partial sum + old x / g) into its slot on EVERY rank (plain peer stores, tagged), and
    // a reader sums the g slots in rank order in fp32: that is the all-reduce of cuda_comm.h:203-300 without a
    // separate step, and every rank computes bit-identical sums. A buffer is rewritten only after all ranks have
    // provably read it: a writer of buffer b has consumed, from every rank, data that those ranks produced after
    // their last read of b (see the ordering notes at the epilogue).
    uint32_t* xb[2][Q4_MAX_GPUS];      // [buffer][rank p]: buffer base (g slots of kLLMaxDim words) in rank p's exchange area
    unsigned long long* cand[Q4_MAX_GPUS];  // rank p's candidate mailbox [2][Q4_MAX_GPUS][2]
    uint16_t* ll_logits[Q4_MAX_GPUS];  // rank p's gathered logits
    int g, rank, vocab_off;
    unsigned launch_parity;
    uint32_t *hb, *q, *knew, *vnew;
    unsigned tag_base;
    __half *logits, *kc, *vc;
    const __half *emb, *wcls;
    const float* rope;       // [seq_len][head_size/2] (cos, sin)
    uint32_t* attn_part;     // [heads*nsplit][kAttnPartStride], tagged with the attention phase
    float* cand_val;         // [grid]
    int* cand_idx;           // [grid]
    int* pos_dev;
    int* tokens_pinned;
    volatile int* pos_pinned;
    unsigned long long* bar_counter;
    unsigned long long bar_base;  // barriers completed by earlier launches
    int* status;
    int write_token;
    int no_handoff;              // 1: leave the token mailbox and the position alone (a sampling kernel follows on the stream)
    int debug;                   // test build only (Q4_TEST_BUILD; always 0 and compiled out of the product library):
                                 // 1 = consumers skip the GEMV math (pure streaming), 2 = no streaming (pure math),
                                 // 8 = raw ring throughput, 16 = tensor-parallel exchange kept local (no NVLink dependency)
    unsigned long long wait_ns;  // limit of every device-side wait on the global timer; on expiry the kernel records Q4_ERR_TIMEOUT
    int n_entries;               // ring entries of kEntryBytes each
    int split_len;               // positions per attention split (a head is split in ceil(T / split_len) parts, at most nsplit)
    unsigned long long* trace;   // optional: [2 CTAs][nphases][8] device timestamps (ns), or null
    unsigned long long* slot_trace;  // test build: [nphases][kCW][kSlotTraceSlots][4] stamps of CTA 0, or null
    // shared memory carve-up (bytes)
    int xq_bytes, meta_off, part_off, part_floats;
};

// ------------------------------------------------------------------------------------------------------------
// device helpers
// ------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b, int count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p; }"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and records the error) when the limit is hit or an error is already recorded.
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// A parity wait cannot tell round r of a ring position from round r - 2. The producer's waits are safe (it issued round
// r - 1 itself, after round r - 2 was released), but a consumer warp may ask for round r of a position whose round
// r - 1 belongs to other warps and is still in flight (bulk copies complete out of order, wildly so on a cold first
// launch): the test would pass on round r - 2's completion. Consumers therefore first wait until the producer has
// ISSUED round r at that position (`seq`, written before the copy is issued); from then on the barrier's current phase
// is r or r + 1 and the parity test is unambiguous. seq == nullptr: the caller is the producer.
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, int* status, unsigned long long limit_ns, const unsigned* seq = nullptr, unsigned want = 0) {
    unsigned long long t0 = 0;
    for (unsigned i = 0; i < kPollLimit; i++) {
        if ((!seq || *(const volatile unsigned*)seq == want) && mbar_try(b, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*(volatile int*)status != 0) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) break;
        }
    }
    if (atomicCAS(status, 0, Q4_ERR_TIMEOUT) == 0) status[1] = 0x40000 + (int)(smem_u32(b) & 0xFFFF);
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory"); }
__device__ __forceinline__ void phase_fetch_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ float fma_mixed(__half a, __half b, float c) {
    float d;
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(__half_as_ushort(a)), "h"(__half_as_ushort(b)), "f"(c));
    return d;
}

// a / d for small operands (a * d < 2^22) without the integer-division sequence: inv = 1.0f / d.
__device__ __forceinline__ int fast_div(unsigned a, float inv) { return (int)(((float)a + 0.5f) * inv); }

// Grid-wide barrier among the consumer threads of all CTAs (the producer warps never wait here).
__device__ __forceinline__ void grid_barrier(const FParams& p, unsigned& nbar, int ctid, int* s_abort) {
    consumer_sync();  // orders every consumer thread's stores before thread 0's release below (cumulativity)
    if (ctid == 0) {
        nbar++;
        const unsigned long long target = (p.bar_base + nbar) * (unsigned long long)gridDim.x;
        unsigned long long v;
        const int st = *(volatile int*)p.status;  // in flight together with the atomic
        asm volatile("atom.add.release.gpu.global.u64 %0, [%1], 1;" : "=l"(v) : "l"(p.bar_counter) : "memory");
        if (blockIdx.x < 256) p.status[4 + 256 + blockIdx.x] = (int)nbar;
        if (st != 0) *s_abort = 1;
        unsigned spins = 0;
        unsigned long long t0 = 0;
        for (;;) {
            asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p.bar_counter) : "memory");
            if (v >= target) break;
            if ((++spins & 63u) == 0) {
                if (*(volatile int*)p.status != 0) { *s_abort = 1; break; }
                const unsigned long long now = global_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > 2 * p.wait_ns) {   // longer than any single data wait, so that the root cause is what gets recorded
                    if (atomicCAS(p.status, 0, Q4_ERR_TIMEOUT) == 0) { p.status[1] = 0x50000 + (int)nbar; p.status[2] = (int)v; p.status[3] = (int)target; }
                    *s_abort = 1;
                    break;
                }
            }
        }
    }
    consumer_sync();
}

// Timestamps of CTA 0 and of the last CTA: [which][phase][0 start, 1 inputs staged, 2 slots done, 3 after the barrier]
#define TRACE(k)                                                                                             \
    do {                                                                                                     \
        if (p.trace && ctid == 0 && (cta == 0 || cta == grid - 1))                                           \
            p.trace[((size_t)(cta == 0 ? 0 : 1) * p.nphases + pi) * kTraceCols + (k)] = global_ns();                  \
    } while (0)

// Test build: per-slot clock stamps of CTA 0 (lane 0 of every consumer warp, first kSlotTraceSlots slots of every GEMV
// phase): 0 before the wait for the slot's weights, 1 after it, 2 after the math, 3 after finishing a unit.
constexpr int kSlotTraceSlots = 6;
#ifdef Q4_TEST_BUILD
#define SLOT_TRACE(k)                                                                                                      \
    do {                                                                                                                   \
        if (p.slot_trace && cta == 0 && lane == 0 && (int)((li - first) / kCW) < kSlotTraceSlots)                           \
            p.slot_trace[(((size_t)pi * kCW + cw) * kSlotTraceSlots + (li - first) / kCW) * 4 + (k)] = global_ns();         \
    } while (0)
#else
#define SLOT_TRACE(k) do {} while (0)
#endif

__device__ __forceinline__ float silu_mul(float g, float u) {
    float val = g;
    val *= 1.0f / (1.0f + expf(-val));
    val *= u;
    return val;
}

__device__ __forceinline__ float transpose_reduce8(const float acc[8], int lane) {
    float a4[4], a2[2], a1;
    const bool up16 = lane & 16, up8 = lane & 8, up4 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float keep = up16 ? acc[i + 4] : acc[i];
        float send = up16 ? acc[i] : acc[i + 4];
        a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        float keep = up8 ? a4[i + 2] : a4[i];
        float send = up8 ? a4[i] : a4[i + 2];
        a2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    {
        float keep = up4 ? a2[1] : a2[0];
        float send = up4 ? a2[0] : a2[1];
        a1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
    a1 += __shfl_xor_sync(0xffffffffu, a1, 1);
    return a1;
}

// Sum over the consumer threads; every consumer thread gets the total. red: kCW floats of shared memory.
// REUSE_BARRIER = false: the caller guarantees a consumer-wide barrier before `red` is written again.
template <bool REUSE_BARRIER = true>
__device__ __forceinline__ float consumer_sum(float v, float* red, int ctid) {
    v = warp_sum(v);
    if ((ctid & 31) == 0) red[ctid >> 5] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kCW; i++) t += red[i];
    if (REUSE_BARRIER) consumer_sync();
    return t;
}

// Tile t of a GEMV phase -> (matrix, 8-column tile inside the matrix).
__device__ __forceinline__ void tile_info(const FPhase& ph, int t, int& mi, int& rt) {
    if (ph.epi == EPI_SILU) { mi = t & 1; rt = t >> 1; return; }
    mi = 0;
    if (ph.nmat > 1 && t >= ph.m[1].tile0) mi = 1;
    if (ph.nmat > 2 && t >= ph.m[2].tile0) mi = 2;
    rt = t - ph.m[mi].tile0;
}

// Units of a phase are dealt to the CTAs round-robin (unit i of CTA c is c + i*grid): at any moment the CTAs stream
// neighbouring tiles, i.e. one contiguous region spread evenly over the memory channels. (Contiguous per-CTA ranges
// measured slower: 148 streams 170 KB apart.) The classifier's unit is a pair of rows, 16 KB contiguous.
__device__ __forceinline__ int unit_count(int nunits, int cta, int grid) { return nunits > cta ? (nunits - cta + grid - 1) / grid : 0; }
__device__ __forceinline__ int unit_at(int i, int cta, int grid) { return cta + i * grid; }

// ---- tagged activations -----------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t tag_of(const FParams& p, int phase) { return ((p.tag_base + (unsigned)phase + 1u) & 0xFFFFu) << 16; }
__device__ __forceinline__ uint32_t tagged(__half v, uint32_t tag_hi) { return tag_hi | (uint32_t)__half_as_ushort(v); }
// 8 consecutive tagged elements (two 128-bit loads). Returns the 8 fp16 values as a uint4 and ORs every tag mismatch into `bad`.
// Tagged words are exchanged between CTAs without a barrier, so both sides use strong (volatile) accesses: a weak load
// may be served from a stale copy for as long as it likes (observed: polling with ld.global.cg never saw the update),
// and the compiler may hoist it out of the wait loop.
__device__ __forceinline__ uint4 ld_poll(const uint4* p) {
    uint4 r;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ uint32_t ld_tagged(const uint32_t* p) {
    uint32_t r;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(r) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ void st_tagged(uint32_t* p, uint32_t v) { asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void st_tagged4(uint32_t* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 load_tagged8(const uint32_t* src, uint32_t tag_hi, uint32_t& bad) {
    const uint4 a = ld_poll(reinterpret_cast<const uint4*>(src)), b = ld_poll(reinterpret_cast<const uint4*>(src) + 1);
    bad |= ((a.x ^ tag_hi) | (a.y ^ tag_hi) | (a.z ^ tag_hi) | (a.w ^ tag_hi) | (b.x ^ tag_hi) | (b.y ^ tag_hi) | (b.z ^ tag_hi) | (b.w ^ tag_hi)) >> 16;
    return make_uint4(prmt(a.x, a.y, 0x5410), prmt(a.z, a.w, 0x5410), prmt(b.x, b.y, 0x5410), prmt(b.z, b.w, 0x5410));
}
// Bounded retry bookkeeping for the tag polls: returns false when the wait must be given up.
__device__ __forceinline__ bool keep_polling(unsigned& polls, unsigned long long& t0, int* status, unsigned long long limit_ns, int where = 0) {
    if ((++polls & 15u) == 0) {
        if (*(volatile int*)status != 0) return false;
        const unsigned long long now = global_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit_ns) {
            if (atomicCAS(status, 0, Q4_ERR_TIMEOUT) == 0) status[1] = where;  // where the first wait ran out (diagnostics)
            return false;
        }
    }
    return true;
}

// Words wd[b] (8 elements each) of the residual stream: waits for the g partial vectors (one per source rank) and sums
// them in rank order in fp32, rounded to fp16 once - the arithmetic of a fixed-order all-reduce. Up to four slots of two
// words are in flight per round trip (64 registers), so an 8-rank group costs two round trips per pair of words.
template <int NB>
__device__ __forceinline__ void load_x_batch(uint4 (&xv)[NB], const bool (&valid)[NB], const int (&wd)[NB], const uint32_t* base, int g,
                                             uint32_t want, int* status, unsigned long long limit_ns, int where) {
    unsigned polls = 0;
    unsigned long long t0 = 0;
    if (g == 1) {
        for (;;) {
            uint32_t bad = 0;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                xv[b] = make_uint4(0, 0, 0, 0);
                if (valid[b]) xv[b] = load_tagged8(base + wd[b] * 8, want, bad);
            }
            if (bad == 0 || !keep_polling(polls, t0, status, limit_ns, where)) break;
        }
        return;
    }
    constexpr int SB = NB < 2 ? NB : 2;   // words per sub-batch
#pragma unroll
    for (int b0 = 0; b0 < NB; b0 += SB) {
        float acc[SB][8];
#pragma unroll
        for (int b = 0; b < SB; b++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[b][j] = 0.f;
        bool any = false;
#pragma unroll
        for (int b = 0; b < SB; b++) any |= valid[b0 + b];
        for (int r0 = 0; r0 < g && any; r0 += 4) {
            uint4 a[SB][4];
            for (;;) {
                uint32_t bad = 0;
#pragma unroll
                for (int b = 0; b < SB; b++)
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        a[b][c] = make_uint4(0, 0, 0, 0);
                        if (valid[b0 + b] && r0 + c < g) a[b][c] = load_tagged8(base + (size_t)(r0 + c) * kLLMaxDim + wd[b0 + b] * 8, want, bad);
                    }
                if (bad == 0 || !keep_polling(polls, t0, status, limit_ns, where)) break;
            }
#pragma unroll
            for (int b = 0; b < SB; b++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    if (r0 + c < g) {
                        const __half2* ha = reinterpret_cast<const __half2*>(&a[b][c]);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const float2 fa = __half22float2(ha[j]);
                            acc[b][2 * j] += fa.x;
                            acc[b][2 * j + 1] += fa.y;
                        }
                    }
                }
        }
#pragma unroll
        for (int b = 0; b < SB; b++) {
            __half2* oh = reinterpret_cast<__half2*>(&xv[b0 + b]);
#pragma unroll
            for (int j = 0; j < 4; j++) oh[j] = __floats2half2_rn(acc[b][2 * j], acc[b][2 * j + 1]);
        }
    }
}

// Walks the slots of one CTA in issue order: phase by phase, unit by unit, tile by tile, k-tile by k-tile.
// The consumers enumerate the same order with plain arithmetic.
struct SlotCursor {
    int pi, u, u_end, tt, kt;   // u, u_end: index of the unit inside this CTA's list
    FPhase* cache;   // shared-memory copy of phases[pi] (the table itself lives in global memory)
    int cached_pi;
};
__device__ __forceinline__ void cursor_init(SlotCursor& c) { c.pi = -1; c.u = 0; c.u_end = 0; c.tt = 0; c.kt = 0; c.cached_pi = -1; }
__device__ __forceinline__ void copy_phase(FPhase* dst, const FPhase* src) {
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(dst);
#pragma unroll
    for (int i = 0; i < (int)(sizeof(FPhase) / 16); i++) d4[i] = __ldg(s4 + i);
}
// Next slot: source address, byte count and the phase it belongs to. False after the last phase.
__device__ __forceinline__ bool cursor_next(SlotCursor& c, const FParams& p, int cta, int grid, const uint8_t*& src, uint32_t& bytes, int& phase) {
    for (;;) {
        if (c.pi >= 0 && c.u < c.u_end) {
            const FPhase& ph = *c.cache;
            phase = c.pi;
            if (ph.type == PH_GEMV) {
                int mi, rt;
                tile_info(ph, unit_at(c.u, cta, grid) * ph.tpu + c.tt, mi, rt);
                const int ng = min(kSlotGroups, ph.G - c.kt * kSlotGroups);
                src = ph.m[mi].blocks + ((size_t)rt * ph.G + (size_t)c.kt * kSlotGroups) * kUnitBytes;
                bytes = ng * kUnitBytes;
                if (++c.kt == ph.nkt) { c.kt = 0; if (++c.tt == ph.tpu) { c.tt = 0; c.u++; } }
            } else {  // PH_CLS: unit = 2 rows (tt), row chunks kt
                const int row = unit_at(c.u, cta, grid) * 2 + c.tt;
                const int len = min(kClsChunk, ph.K - c.kt * kClsChunk);
                src = reinterpret_cast<const uint8_t*>(p.wcls + (size_t)row * ph.K + (size_t)c.kt * kClsChunk);
                bytes = len * 2;
                if (++c.kt == ph.nkt) { c.kt = 0; if (++c.tt == 2) { c.tt = 0; c.u++; } }
            }
            return true;
        }
        if (++c.pi >= p.nphases) return false;
        copy_phase(c.cache, p.phases + c.pi);
        const FPhase& ph = *c.cache;
        c.tt = 0;
        c.kt = 0;
        if (ph.type == PH_GEMV || ph.type == PH_CLS) {
            c.u = 0;
            c.u_end = unit_count(ph.nunits, cta, grid);
        } else {
            c.u = c.u_end = 0;
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// Staging of the activation vector into shared memory (all consumer threads).
// GEMV: optional RMSNorm (same arithmetic as gpu_kernels.h:72-105, result rounded to fp16), then block fixed point.
// xq uint4 index = ((kt*2 + j2)*4 + wi)*32 + lane, lane = 2*(group%16) + half; .x/.y = high digit for even/odd
// nibbles, .z/.w = low digit. xs_scale[kt*32 + lane] = sx of the group, xs_sum[kt*32 + lane] = sum X over the
// lane's 64 inputs.
// ------------------------------------------------------------------------------------------------------------
// One word (8 consecutive elements) of the attention output from the per-split partials (max, sum, un-normalised V sum):
// all splits' loads are issued together, merged in fixed split order, normalised and rounded to fp16 like the
// reference's attention output (gpu_kernels.h:335-336).
struct AttnWord {
    uint4 a[kMaxSplit];      // 8 fp16 values of the split's normalised output
    float2 ml[kMaxSplit];
};
// The partials arrive tagged (no grid barrier after the attention phase): every tag mismatch is ORed into `bad`.
__device__ __forceinline__ void attn_word_load(AttnWord& w, const FParams& p, int ns, int wd, bool valid, uint32_t want, uint32_t& bad) {
    const int h = (wd * 8) / 128, d = (wd * 8) % 128;
#pragma unroll
    for (int s = 0; s < kMaxSplit; s++) {
        w.ml[s] = make_float2(-CUDART_INF_F, 0.f);
        w.a[s] = make_uint4(0, 0, 0, 0);
        if (valid && s < ns) {
            const uint32_t* base = p.attn_part + ((size_t)h * p.nsplit + s) * kAttnPartStride;
            w.a[s] = load_tagged8(base + d, want, bad);
            const uint4 t = ld_poll(reinterpret_cast<const uint4*>(base + 128));
            bad |= ((t.x ^ want) | (t.y ^ want) | (t.z ^ want) | (t.w ^ want)) >> 16;
            w.ml[s] = make_float2(__uint_as_float((t.x & 0xFFFFu) | (t.y << 16)), __uint_as_float((t.z & 0xFFFFu) | (t.w << 16)));
        }
    }
}
__device__ __forceinline__ uint4 attn_word_merge(const AttnWord& w) {
    float M = -CUDART_INF_F;
#pragma unroll
    for (int s = 0; s < kMaxSplit; s++) M = fmaxf(M, w.ml[s].x);
    float L = 0.f, a[8];
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxSplit; s++) {
        if (w.ml[s].x != -CUDART_INF_F) {
            const float e = w.ml[s].y * __expf(w.ml[s].x - M);  // weight of the split = its sum, rescaled to the common max
            // (merge weights: the fast exponential's error is far below the fp16 outputs; the scores themselves use expf)
            L += e;
            const __half2* hh = reinterpret_cast<const __half2*>(&w.a[s]);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(hh[j]);
                a[2 * j] += f.x * e;
                a[2 * j + 1] += f.y * e;
            }
        }
    }
    uint4 out;
    __half2* oh = reinterpret_cast<__half2*>(&out);
    const float rl = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) oh[j] = __floats2half2_rn(a[2 * j] * rl, a[2 * j + 1] * rl);
    return out;
}

// Quantises one word (8 fp16 values, packed in a uint4) to 15-bit block fixed point and files it in xq / xs_*.
// X = rint(v * 16256 / amax) and its high digit rint(v * 127 / amax) come out of two FMAs with the 1.5 * 2^23 magic
// constant (the integer sits in the low mantissa bits), the low digit is X - 128 * hi (|lo| <= 64), and the digits
// are gathered into the DP4A operand words with byte permutes.
// NW words are processed in lockstep so that their shuffle and conversion chains overlap.
template <int NW>
__device__ __forceinline__ void quant_words(const uint4 (&hv)[NW], const int (&wd)[NW], int nwords, uint4* xq, float* xs_scale, int* xs_sum) {
    constexpr float kMagic = 12582912.0f;      // 1.5 * 2^23
    constexpr int kMagicBits = 0x4B400000;
    float amax[NW];
#pragma unroll
    for (int w = 0; w < NW; w++) {
        const __half2* h = reinterpret_cast<const __half2*>(&hv[w]);
        const __half2 m2 = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
        amax[w] = fmaxf(__low2float(m2), __high2float(m2));
    }
#pragma unroll
    for (int o = 1; o < 16; o <<= 1)   // 16 words = 1 group
#pragma unroll
        for (int w = 0; w < NW; w++) amax[w] = fmaxf(amax[w], __shfl_xor_sync(0xffffffffu, amax[w], o));
    int sum[NW];
    uint32_t he[NW], ho[NW], le[NW], lo[NW];
#pragma unroll
    for (int w = 0; w < NW; w++) {
        const __half2* h = reinterpret_cast<const __half2*>(&hv[w]);
        const float inv = amax[w] > 0.f ? 16256.0f / amax[w] : 0.f;
        const float inv128 = inv * (1.0f / 128.0f);
        int xb[8], hb[8], lb[8];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(h[j]);
            xb[2 * j] = __float_as_int(fmaf(f.x, inv, kMagic));
            xb[2 * j + 1] = __float_as_int(fmaf(f.y, inv, kMagic));
            hb[2 * j] = __float_as_int(fmaf(f.x, inv128, kMagic));
            hb[2 * j + 1] = __float_as_int(fmaf(f.y, inv128, kMagic));
        }
        int sm = (int)(0u - 8u * (unsigned)kMagicBits);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            sm += xb[j];
            lb[j] = xb[j] - (hb[j] << 7);   // low byte = X - 128 * hi (the magic constants cancel in the low byte)
        }
        sum[w] = sm;
        // byte 0 of four registers -> one word: (a, b) -> [a.b0, b.b0], then the two halves together
        he[w] = prmt(prmt(hb[0], hb[2], 0x0040), prmt(hb[4], hb[6], 0x0040), 0x5410);
        ho[w] = prmt(prmt(hb[1], hb[3], 0x0040), prmt(hb[5], hb[7], 0x0040), 0x5410);
        le[w] = prmt(prmt(lb[0], lb[2], 0x0040), prmt(lb[4], lb[6], 0x0040), 0x5410);
        lo[w] = prmt(prmt(lb[1], lb[3], 0x0040), prmt(lb[5], lb[7], 0x0040), 0x5410);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1)   // 8 words = the 64 inputs of one (group, half)
#pragma unroll
        for (int w = 0; w < NW; w++) sum[w] += __shfl_xor_sync(0xffffffffu, sum[w], o);
#pragma unroll
    for (int w = 0; w < NW; w++) {
        if (wd[w] < nwords) {
            const int g = wd[w] >> 4, c = (wd[w] >> 2) & 3, wi = wd[w] & 3;
            const int kt = g >> 4, lane = 2 * (g & 15) + (c >> 1), j2 = c & 1;
            xq[((kt * 2 + j2) * 4 + wi) * 32 + lane] = make_uint4(he[w], ho[w], le[w], lo[w]);
            if ((wd[w] & 7) == 0) { xs_scale[kt * 32 + lane] = amax[w] * (1.0f / 16256.0f); xs_sum[kt * 32 + lane] = sum[w]; }
        }
    }
}
__device__ __forceinline__ void quant_word(const uint4& hv, int wd, int nwords, uint4* xq, float* xs_scale, int* xs_sum) {
    const uint4 h1[1] = {hv};
    const int w1[1] = {wd};
    quant_words<1>(h1, w1, nwords, xq, xs_scale, xs_sum);
}

// Splits per head at sequence length T: short contexts are not split at all (one CTA per head, no partial traffic).
__device__ __forceinline__ int attn_splits_for(const FParams& p, int T) { return min(p.nsplit, max(1, (T + p.split_len - 1) / p.split_len)); }

// Words b0.. of one batch: SB words per thread in flight, CH rank slots per round trip. A word is processed as soon as
// the whole warp has it (the 16 threads of a group share a scale), so the words that are there early are done while the
// late ones - the outputs of the slowest CTA or rank - are still being polled. Plain inputs are quantised at once.
// RMSNorm inputs (DEFER) need the whole vector first: their words are summed over the ranks and handed back in xout
// (the reference rounds x * (w / rms) to fp16, gpu_kernels.h:100-102, and so does the caller). The sum of squares is
// NOT accumulated here: words complete in whatever order their tags arrive, and a float sum taken in arrival order
// would differ in the last bit from run to run, from CTA to CTA and from rank to rank.
template <int SB, int CH, bool MULTI, bool DEFER>
__device__ __forceinline__ void stage_words(const FPhase& ph, const FParams& p, const uint32_t* base, int g, uint32_t want, int it0, int iters,
                                            int nwords, uint4* xq, float* xs_scale, int* xs_sum, int ctid, float& ss, bool& gave_up,
                                            uint4* xout) {
    const int K = ph.K;
    int wds[SB];
    bool valid[SB];
    unsigned pending = 0;
#pragma unroll
    for (int b = 0; b < SB; b++) {
        wds[b] = ctid + (it0 + b) * kCT;
        valid[b] = it0 + b < iters && wds[b] < nwords && wds[b] * 8 < K;
        if (it0 + b < iters) pending |= 1u << b;   // uniform over the CTA
    }
    float acc[MULTI ? SB : 1][8];
#pragma unroll
    for (int b = 0; b < (MULTI ? SB : 1); b++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[b][j] = 0.f;
    unsigned polls = 0;
    unsigned long long t0 = 0;
    for (int r0 = 0; r0 < g && !gave_up; r0 += CH) {
        const bool last = r0 + CH >= g;
        unsigned pend = pending;
        while (pend) {
            uint4 a[SB][CH];
            uint32_t bad[SB];
#pragma unroll
            for (int b = 0; b < SB; b++) {
                bad[b] = 0;
#pragma unroll
                for (int c = 0; c < CH; c++) {
                    a[b][c] = make_uint4(0, 0, 0, 0);
                    if (((pend >> b) & 1u) && valid[b] && r0 + c < g) a[b][c] = load_tagged8(base + (size_t)(r0 + c) * kLLMaxDim + wds[b] * 8, want, bad[b]);
                }
            }
#pragma unroll
            for (int b = 0; b < SB; b++) {
                if (!((pend >> b) & 1u)) continue;
                if (!__all_sync(0xffffffffu, bad[b] == 0)) continue;
                pend &= ~(1u << b);
                uint4 hv = a[b][0];
                if (MULTI) {   // sum of the ranks' partials in rank order, fp32, rounded to fp16 once
                    constexpr int bb = MULTI ? 1 : 0;
#pragma unroll
                    for (int c = 0; c < CH; c++) {
                        if (r0 + c < g) {
                            const __half2* ha = reinterpret_cast<const __half2*>(&a[b][c]);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const float2 fa = __half22float2(ha[j]);
                                acc[b * bb][2 * j] += fa.x;
                                acc[b * bb][2 * j + 1] += fa.y;
                            }
                        }
                    }
                    if (!last) continue;
                    __half2* oh = reinterpret_cast<__half2*>(&hv);
#pragma unroll
                    for (int j = 0; j < 4; j++) oh[j] = __floats2half2_rn(acc[b * bb][2 * j], acc[b * bb][2 * j + 1]);
                }
                if (DEFER) {
                    xout[b] = hv;   // the caller squares and sums the words in index order once all have arrived
                } else {
                    quant_word(hv, wds[b], nwords, xq, xs_scale, xs_sum);
                }
            }
            if (pend) {
                int go = keep_polling(polls, t0, p.status, p.wait_ns, 0x100 + ph.in_phase) ? 1 : 0;
                go = __all_sync(0xffffffffu, go);
                if (!go) { gave_up = true; break; }
            }
        }
    }
}

__device__ void stage_x_quant(const FPhase& ph, const FParams& p, int pos, uint4* xq, float* xs_scale, int* xs_sum, float* red, int ctid,
                              unsigned long long* tr) {
    const int K = ph.K, nwords = ph.G * 16;
    const int iters = (nwords + kCT - 1) / kCT;
    const uint32_t want = tag_of(p, ph.in_phase);
    if (ph.attn_in) {
        const int ns = attn_splits_for(p, pos + 1);
        // two words per thread in flight (all splits of both): one L2 round trip for K <= 2 * kCT * 8
        for (int it0 = 0; it0 < iters; it0 += 2) {
            AttnWord w0, w1;
            const int wd0 = ctid + it0 * kCT, wd1 = wd0 + kCT;
            unsigned polls = 0;
            unsigned long long t0 = 0;
            for (;;) {   // this poll is the op boundary between the attention phase and the o projection
                uint32_t bad = 0;
                attn_word_load(w0, p, ns, wd0, wd0 < nwords && wd0 * 8 < K, want, bad);
                attn_word_load(w1, p, ns, wd1, it0 + 1 < iters && wd1 < nwords && wd1 * 8 < K, want, bad);
                if (bad == 0 || !keep_polling(polls, t0, p.status, p.wait_ns, 0x80000 + ph.in_phase)) break;
            }
            if (tr && it0 == 0) tr[4] = global_ns();
            // (a word index past the vector quantises zeros and stores nothing)
            const uint4 hv2[2] = {attn_word_merge(w0), attn_word_merge(w1)};
            const int wd2[2] = {wd0, wd1};
            quant_words<2>(hv2, wd2, nwords, xq, xs_scale, xs_sum);
        }
        consumer_sync();
        return;
    }
    const uint32_t* base = ph.xbuf_in >= 0 ? p.xb[ph.xbuf_in][p.rank] : ph.xin;
    const int g = ph.xbuf_in >= 0 ? p.g : 1;
    float ss = 0.f;
    bool gave_up = false;
    if (!ph.norm_w) {
        if (g == 1)
            for (int it0 = 0; it0 < iters; it0 += 4)
                stage_words<4, 1, false, false>(ph, p, base, 1, want, it0, iters, nwords, xq, xs_scale, xs_sum, ctid, ss, gave_up, nullptr);
        else
            for (int it0 = 0; it0 < iters; it0 += 2)
                stage_words<2, 4, true, false>(ph, p, base, g, want, it0, iters, nwords, xq, xs_scale, xs_sum, ctid, ss, gave_up, nullptr);
        if (tr) tr[6] = global_ns();
        consumer_sync();
        return;
    }
    // RMSNorm inputs have K = dim <= 4 * kCT * 8 (host-checked): the whole vector fits the threads' registers
    uint4 xv[4], wv[4];
#pragma unroll
    for (int b = 0; b < 4; b++) {
        const int wd = ctid + b * kCT;
        xv[b] = wv[b] = make_uint4(0, 0, 0, 0);
        if (b < iters && wd < nwords && wd * 8 < K) wv[b] = *reinterpret_cast<const uint4*>(ph.norm_w + wd * 8);
    }
    if (g == 1) {
        stage_words<4, 1, false, true>(ph, p, base, 1, want, 0, iters, nwords, xq, xs_scale, xs_sum, ctid, ss, gave_up, xv);
    } else {
        stage_words<2, 4, true, true>(ph, p, base, g, want, 0, iters, nwords, xq, xs_scale, xs_sum, ctid, ss, gave_up, xv);
        if (iters > 2) stage_words<2, 4, true, true>(ph, p, base, g, want, 2, iters, nwords, xq, xs_scale, xs_sum, ctid, ss, gave_up, xv + 2);
    }
    if (tr) tr[4] = global_ns();
    // sum of squares in a fixed order: word index inside the thread, shuffle tree inside the warp, warp index last
#pragma unroll
    for (int b = 0; b < 4; b++) {
        const __half2* xh = reinterpret_cast<const __half2*>(&xv[b]);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 xf2 = __half22float2(xh[j]);
            ss = fmaf(xf2.x, xf2.x, ss);
            ss = fmaf(xf2.y, xf2.y, ss);
        }
    }
    ss = consumer_sum<false>(ss, red, ctid);   // the staging's closing barrier comes before any other use of `red`
    ss /= K;
    ss += 1e-5f;
    const float inv_rms = 1.0f / sqrtf(ss);
    if (tr) tr[5] = global_ns();
#pragma unroll
    for (int b0 = 0; b0 < 4; b0 += 2) {
        if (b0 < iters) {  // uniform over the block: the shuffles in quant_words see all lanes
            // val = x * (inv_rms * w), rounded to fp16 once (gpu_kernels.h:100-102); two words in lockstep (a word
            // index past the vector holds zeros and stores nothing)
            uint4 hv[2];
            int wd2[2];
#pragma unroll
            for (int b = 0; b < 2; b++) {
                const __half2* xh = reinterpret_cast<const __half2*>(&xv[b0 + b]);
                const __half2* wh = reinterpret_cast<const __half2*>(&wv[b0 + b]);
                __half2* oh = reinterpret_cast<__half2*>(&hv[b]);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 xf2 = __half22float2(xh[j]), wf2 = __half22float2(wh[j]);
                    oh[j] = __floats2half2_rn(xf2.x * (inv_rms * wf2.x), xf2.y * (inv_rms * wf2.y));
                }
                wd2[b] = ctid + (b0 + b) * kCT;
            }
            quant_words<2>(hv, wd2, nwords, xq, xs_scale, xs_sum);
        }
    }
    if (tr) tr[6] = global_ns();
    consumer_sync();
}

// Classifier input: final RMSNorm, fp16, plain layout.
__device__ void stage_x_f16(const FPhase& ph, const FParams& p, __half* xf, float* red, int ctid) {
    const int K = ph.K;
    const uint32_t want = tag_of(p, ph.in_phase);
    float ss = 0.f;
    // first pass: wait for the tagged words, keep the values in shared memory, sum the squares
    for (int wd = ctid; wd * 8 < K; wd += kCT) {
        uint4 xv1[1];
        const bool valid1[1] = {true};
        const int wd1[1] = {wd};
        load_x_batch<1>(xv1, valid1, wd1, p.xb[ph.xbuf_in][p.rank], p.g, want, p.status, p.wait_ns, 0x60000 + ph.in_phase);
        const uint4 v = xv1[0];
        reinterpret_cast<uint4*>(xf)[wd] = v;
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(h[j]);
            ss = fmaf(f.x, f.x, ss);
            ss = fmaf(f.y, f.y, ss);
        }
    }
    ss = consumer_sum(ss, red, ctid);
    ss /= K;
    ss += 1e-5f;
    const float inv_rms = 1.0f / sqrtf(ss);
    for (int i = ctid; i < K; i += kCT) {
        float val = __half2float(xf[i]);
        val *= inv_rms * __half2float(ph.norm_w[i]);
        xf[i] = __float2half(val);
    }
    consumer_sync();
}

// Four columns x 32 inputs: 64 DP4As in 16 independent accumulator chains (columns innermost), so that two warps
// per scheduler are enough to keep the half-rate DP4A pipe busy.
template <int RB>
__device__ __forceinline__ void dot_rows4(const uint4 (&w)[4], const uint4 (&xv)[4], int (&ah)[8], int (&ah16)[8], int (&al)[8], int (&al16)[8]) {
#pragma unroll
    for (int wi = 0; wi < 4; wi++) {
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const uint32_t word = wi == 0 ? w[r].x : wi == 1 ? w[r].y : wi == 2 ? w[r].z : w[r].w;
            const uint32_t e = word & 0x0F0F0F0Fu, o = word & 0xF0F0F0F0u;
            ah[RB + r] = dp4a_us(e, xv[wi].x, ah[RB + r]);
            ah16[RB + r] = dp4a_us(o, xv[wi].y, ah16[RB + r]);
            al[RB + r] = dp4a_us(e, xv[wi].z, al[RB + r]);
            al16[RB + r] = dp4a_us(o, xv[wi].w, al16[RB + r]);
        }
    }
}

// One slot of a GEMV phase: 8 columns x ng groups. Returns via `part` (8 floats per slot in shared memory).
__device__ __forceinline__ void gemv_slot(const uint8_t* slot, int ng, int kt, const uint4* xq, const float* xs_scale, const int* xs_sum,
                                          float* part, int lane) {
    const int nl = 2 * ng;
    const bool active = lane < nl;
    float facc[8];
#pragma unroll
    for (int r = 0; r < 8; r++) facc[r] = 0.f;
    if (active) {
        int ah[8], ah16[8], al[8], al16[8];
#pragma unroll
        for (int r = 0; r < 8; r++) { ah[r] = 0; ah16[r] = 0; al[r] = 0; al16[r] = 0; }
        const uint4* wb = reinterpret_cast<const uint4*>(slot) + lane;
        const uint4* xb = xq + (kt * 2) * 4 * 32 + lane;
        // loads run one quarter step (4 columns of one 32-input chunk) ahead of the math
        uint4 x0[4], x1[4], wa[4], wbuf[4];
#pragma unroll
        for (int wi = 0; wi < 4; wi++) x0[wi] = xb[wi * 32];
#pragma unroll
        for (int r = 0; r < 4; r++) wa[r] = wb[r * nl];
#pragma unroll
        for (int r = 0; r < 4; r++) wbuf[r] = wb[(4 + r) * nl];
#pragma unroll
        for (int wi = 0; wi < 4; wi++) x1[wi] = xb[(4 + wi) * 32];
        dot_rows4<0>(wa, x0, ah, ah16, al, al16);
#pragma unroll
        for (int r = 0; r < 4; r++) wa[r] = wb[(8 + r) * nl];
        dot_rows4<4>(wbuf, x0, ah, ah16, al, al16);
#pragma unroll
        for (int r = 0; r < 4; r++) wbuf[r] = wb[(12 + r) * nl];
        dot_rows4<0>(wa, x1, ah, ah16, al, al16);
        const uint8_t* meta = slot + ng * 512 + (lane >> 1) * 32;
        const uint4 sc = *reinterpret_cast<const uint4*>(meta);
        const uint2 zz = *reinterpret_cast<const uint2*>(meta + 16);
        const float sx = xs_scale[kt * 32 + lane];
        const int sumx = xs_sum[kt * 32 + lane];
        dot_rows4<4>(wbuf, x1, ah, ah16, al, al16);
        const __half* sh = reinterpret_cast<const __half*>(&sc);
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const int z = (int)(((r < 4 ? zz.x : zz.y) >> (8 * (r & 3))) & 0xFFu);
            const int ri = ((ah[r] + (ah16[r] >> 4)) << 7) + al[r] + (al16[r] >> 4) - z * sumx;
            facc[r] = (float)ri * (__half2float(sh[r]) * sx);
        }
    }
    const float tot = transpose_reduce8(facc, lane);
    if ((lane & 3) == 0) part[lane >> 2] = tot;
}

// ------------------------------------------------------------------------------------------------------------
// The kernel
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) fused_token_kernel(const FParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[kMaxEntries], empty_bar[kMaxEntries];
    __shared__ unsigned s_round[kMaxEntries];   // round last issued by the producer per ring position
    const int kEntries = p.n_entries;
    __shared__ float red[kCW];
    __shared__ int s_abort;
    __shared__ __align__(16) FPhase s_cph;     // consumers' phase descriptor
    __shared__ __align__(16) FPhase s_next;    // the next one, on its way in
    __shared__ uint64_t unit_bar[kMaxUnitsPerCta];  // per unit of the current phase: completes when all its slots are done

    uint8_t* ring = smem;
    uint4* xq = reinterpret_cast<uint4*>(smem + (size_t)p.n_entries * kEntryBytes);
    float* xs_scale = reinterpret_cast<float*>(smem + p.meta_off);
    int* xs_sum = reinterpret_cast<int*>(smem + p.meta_off) + 32 * 16;   // up to 16 k-tiles... sized by host
    float* part = reinterpret_cast<float*>(smem + p.part_off);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, grid = gridDim.x;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < kMaxEntries; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 2); s_round[s] = 0xFFFFFFFFu; }
        for (int s = 0; s < kMaxUnitsPerCta; s++) mbar_init(&unit_bar[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 0) {
        // ================= producer: stream every phase's weights of this CTA into the ring =================
        // (Requesting weights into L2 ahead of the ring was measured and dropped: it slows the stream down.)
        if (Q4_DBG(p) & 2) return;
        // The whole warp walks this CTA's precomputed copy list: 32 descriptors are fetched at a time (one per lane),
        // then lane 0 issues them one by one as ring entries free up. One entry = two consecutive slots of a phase,
        // one bulk copy when they are adjacent in memory.
        const CopyDesc* dl = p.desc + (size_t)cta * p.desc_stride;
        const int nd = p.desc_count[cta];
        unsigned ent = 0, pround = 0, prnd = 0;   // entries issued; ring position pe, the parity of its round and the round
        int pe = 0;
        bool ok = true;
        for (int base = 0; base < nd && ok; base += 32) {
            uint4 d0 = make_uint4(0, 0, 0, 0), d1 = d0;
            if (base + lane < nd) {
                const uint4* dp = reinterpret_cast<const uint4*>(dl + base + lane);
                d0 = __ldg(dp);
                d1 = __ldg(dp + 1);
            }
            const int cnt = min(32, nd - base);
            for (int i = 0; i < cnt; i++) {
                const uint32_t s0l = __shfl_sync(0xffffffffu, d0.x, i), s0h = __shfl_sync(0xffffffffu, d0.y, i);
                const uint32_t s1l = __shfl_sync(0xffffffffu, d0.z, i), s1h = __shfl_sync(0xffffffffu, d0.w, i);
                const uint32_t b0 = __shfl_sync(0xffffffffu, d1.x, i), b1 = __shfl_sync(0xffffffffu, d1.y, i);
                int good = 1;
                if (lane == 0) {
                    const int e = pe;
                    if (!mbar_wait(&empty_bar[e], pround ^ 1u, p.status, p.wait_ns)) {
                        good = 0;
                    } else {
                        uint8_t* dst = ring + (size_t)e * kEntryBytes;
                        const uint8_t* src0 = reinterpret_cast<const uint8_t*>(((unsigned long long)s0h << 32) | s0l);
                        *(volatile unsigned*)&s_round[e] = prnd;
                        mbar_expect_tx(&full_bar[e], b0 + b1);
                        bulk_g2s(dst, src0, b0, &full_bar[e]);
                        if (b1) bulk_g2s(dst + b0, reinterpret_cast<const uint8_t*>(((unsigned long long)s1h << 32) | s1l), b1, &full_bar[e]);
                        ent++;
                        if (++pe == kEntries) { pe = 0; pround ^= 1u; prnd++; }
                    }
                }
                good = __shfl_sync(0xffffffffu, good, 0);
                if (!good) { ok = false; break; }
            }
        }
        if (lane != 0) return;
        // Before this thread (the last owner of the CTA's shared memory as far as the copy engine is concerned) leaves:
        // every bulk copy it issued must have landed. On the normal path the consumers have waited for all of them
        // already; after an error the newest copy of each ring entry may still be in flight.
        if (*(volatile int*)p.status != 0) {
            const unsigned first = ent > (unsigned)kEntries ? ent - (unsigned)kEntries : 0;
            for (unsigned i = first; i < ent; i++) {
                const unsigned long long t0 = global_ns();
                while (!mbar_try(&full_bar[i % kEntries], (i / kEntries) & 1)) {
                    if (global_ns() - t0 > 50ULL * 1000 * 1000) break;  // 50 ms: far beyond any copy's flight time
                }
            }
        }
        return;
    }

    // ================= consumers =================
    const int ctid = tid - 32, cw = warp - 1;
    unsigned sbase = 0, ent0 = 0, nbar = 0;   // slots and ring entries consumed by earlier phases
    bool failed = false;  // a bounded wait ran out: skip the remaining slots, keep taking part in the barriers
    const int pos = *p.pos_dev;
    const int HS = p.head_size;
    const float inv_entries = 1.0f / (float)kEntries;

    // Phase descriptors are fetched one phase ahead with asynchronous copies (no register is held, nothing waits on the
    // L2 round trip): the copy of phase pi + 1 into s_next is issued at the top of phase pi and completed before the
    // barrier that closes phase pi; the next phase starts by moving it to the fixed place the code reads it from.
    constexpr int kPhaseVecs = (int)(sizeof(FPhase) / 16);
    auto fetch_phase = [&](int which) {
        if (which < p.nphases && ctid < kPhaseVecs)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(reinterpret_cast<int4*>(&s_next) + ctid)),
                         "l"(reinterpret_cast<const int4*>(p.phases + which) + ctid) : "memory");
    };
    fetch_phase(0);
    phase_fetch_wait();
    consumer_sync();
    for (int pi = 0; pi < p.nphases; pi++) {
        if (ctid < kPhaseVecs) reinterpret_cast<int4*>(&s_cph)[ctid] = reinterpret_cast<const int4*>(&s_next)[ctid];
        consumer_sync();
        fetch_phase(pi + 1);   // by the threads that have just read s_next
        const FPhase& ph = s_cph;
        // all consumer threads leave together (named barriers count live threads), never one by one:
        // s_abort is written by thread 0 inside grid_barrier and read after the barrier's closing consumer_sync
        if (s_abort != 0) return;
        if (ctid == 0 && cta < 256) p.status[4 + cta] = pi;  // progress marker (diagnostics after a timeout)
        TRACE(0);
        // the next RMSNorm weight vector is cold in HBM: one CTA requests it into L2 a phase ahead of its use
        if (ph.next_norm_w && cta == pi % grid && ctid * 64 < ph.next_norm_n)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(ph.next_norm_w + ctid * 64));

        if (Q4_DBG(p) & 8) {
            // measurement only: raw ring throughput over the real weight layout (no staging, no math, no barriers)
            if (ph.type == PH_GEMV || ph.type == PH_CLS) {
                const int tpu = ph.type == PH_GEMV ? ph.tpu : 2;
                const int nslots = unit_count(ph.nunits, cta, grid) * tpu * ph.nkt;
                const unsigned first = (cw + kCW - (sbase % kCW)) % kCW;
                for (unsigned li = first; li < (unsigned)nslots; li += kCW) {
                    const unsigned en = ent0 + (li >> 1);
                    const int e = en % kEntries;
                    if (failed || !mbar_wait(&full_bar[e], (en / kEntries) & 1, p.status, p.wait_ns, &s_round[e], en / kEntries)) { failed = true; continue; }
                    if (lane == 0) mbar_arrive(&empty_bar[e], (!(li & 1) && li + 1 == (unsigned)nslots) ? 2 : 1);
                }
                sbase += nslots;
                ent0 += (nslots + 1) >> 1;
            }
            phase_fetch_wait();
            consumer_sync();
            continue;
        }
        if (ph.type == PH_EMBED) {
            // copy_embedding_kernel (gpu_kernels.h:61-69): the token id comes from the pinned host mailbox
            if (cta * kCT + ctid < p.cfg.dim / 8) {
                const int token = p.tokens_pinned[pos];
                const uint4* src = reinterpret_cast<const uint4*>(p.emb + (size_t)token * p.cfg.dim);
                const uint32_t tg = tag_of(p, pi);
                // every rank files the row as slot 0 of its own buffer 1 and zeros as the other ranks' partials
                for (int i = cta * kCT + ctid; i < p.cfg.dim / 8; i += grid * kCT) {
                    const uint4 v = src[i];
                    uint32_t* dst = p.xb[1][p.rank] + (size_t)i * 8;
                    st_tagged4(dst, make_uint4(tg | (v.x & 0xFFFFu), tg | (v.x >> 16), tg | (v.y & 0xFFFFu), tg | (v.y >> 16)));
                    st_tagged4(dst + 4, make_uint4(tg | (v.z & 0xFFFFu), tg | (v.z >> 16), tg | (v.w & 0xFFFFu), tg | (v.w >> 16)));
                    for (int r = 1; r < p.g; r++) {
                        st_tagged4(dst + (size_t)r * kLLMaxDim, make_uint4(tg, tg, tg, tg));
                        st_tagged4(dst + (size_t)r * kLLMaxDim + 4, make_uint4(tg, tg, tg, tg));
                    }
                }
            }
            phase_fetch_wait();
            consumer_sync();  // closes the phase: the next descriptor is in place, this one may be replaced from now on

        } else if (ph.type == PH_GEMV) {
            if (ctid < kMaxUnitsPerCta) {   // re-armed for this phase's slots per unit; the staging's closing barrier orders it before the first arrival
                asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&unit_bar[ctid])) : "memory");
                mbar_init(&unit_bar[ctid], ph.tpu * ph.nkt);
            }
            stage_x_quant(ph, p, pos, xq, xs_scale, xs_sum, red, ctid,
                          (p.trace && ctid == 0 && cta == 0) ? p.trace + (size_t)pi * kTraceCols : nullptr);
            TRACE(1);
            // Slots of this CTA, in the producer's order; slot i belongs to consumer warp i % kCW. A unit (tile, or gate
            // tile + up tile) is finished by the warp that owns its LAST slot: it waits until the unit's other slots have
            // been counted in (they were started earlier by other warps), sums the per-slot partials in slot order and
            // writes the outputs at once - no CTA-wide step between the math and the stores.
            // Phase constants live in registers: the descriptor is not re-read inside the loops.
            const int nunits = ph.nunits, tpu = ph.tpu, nkt = ph.nkt, G = ph.G, dbg = Q4_DBG(p), epi = ph.epi;
            const int my_units = unit_count(nunits, cta, grid);
            const int spu = tpu * nkt, nslots = my_units * spu;
            const unsigned first = (cw + kCW - (sbase % kCW)) % kCW;  // first slot of this warp in the phase
            const uint32_t out_tag = tag_of(p, pi);
            const float inv_nkt = 1.0f / (float)nkt, inv_spu = 1.0f / (float)spu;
            // (lane = 8 * slot + column; slots 4..7 of an 8-rank group in the second register)
            uint32_t resid = 0, resid2 = 0;
            int resid_unit = -1;
            const uint32_t* const oldx = epi == EPI_RESIDUAL ? p.xb[ph.xbuf_out ^ 1][p.rank] + (size_t)(lane >> 3) * kLLMaxDim + (lane & 7) : nullptr;
            if (epi == EPI_RESIDUAL) {
                for (int ul = 0; ul < my_units && resid_unit < 0; ul++)
                    if ((unsigned)((ul + 1) * spu - 1) % kCW == first) resid_unit = ul;
                if (resid_unit >= 0) {
                    const int n0 = unit_at(resid_unit, cta, grid) * 8;
                    if ((lane >> 3) < p.g) resid = ld_tagged(oldx + n0);
                    if ((lane >> 3) + 4 < p.g) resid2 = ld_tagged(oldx + 4 * (size_t)kLLMaxDim + n0);
                }
            }
            for (unsigned li = first; li < (unsigned)nslots; li += kCW) {   // li = (local unit * tpu + tile) * nkt + kt
                const int kt = li - fast_div(li, inv_nkt) * nkt;
                const int ng = min(kSlotGroups, G - kt * kSlotGroups);
                const unsigned en = ent0 + (li >> 1);
                const int eq = fast_div(en, inv_entries), e = (int)en - eq * kEntries;
                int off = 0;
                if (li & 1) { const int ktp = kt > 0 ? kt - 1 : nkt - 1; off = min(kSlotGroups, G - ktp * kSlotGroups) * kUnitBytes; }
                SLOT_TRACE(0);
                if (!(dbg & 2) && (failed || !mbar_wait(&full_bar[e], eq & 1, p.status, p.wait_ns, &s_round[e], (unsigned)eq))) { failed = true; continue; }
                SLOT_TRACE(1);
                if (!(dbg & 1)) gemv_slot(ring + (size_t)e * kEntryBytes + off, ng, kt, xq, xs_scale, xs_sum, part + (size_t)li * 8, lane);
                __syncwarp();
                SLOT_TRACE(2);
                const int ul = fast_div(li, inv_spu);
                // One arrive instruction, two lanes: lane 0 releases the ring entry (an entry is released by its two slots;
                // a phase's odd last slot releases it alone), lane 1 counts the slot in for its unit (release: the slot's
                // partials are written).
                if (lane < 2 && !(lane == 0 && (dbg & 2)))
                    mbar_arrive(lane == 0 ? &empty_bar[e] : &unit_bar[ul], (lane == 0 && !(li & 1) && li + 1 == (unsigned)nslots) ? 2 : 1);
                if ((int)li - ul * spu != spu - 1) continue;
                // ---- this warp finishes unit ul ----
                // output index of this lane's column, looked up before the wait (shared-memory reads off the critical path)
                int mi, rt;
                tile_info(ph, unit_at(ul, cta, grid) * tpu, mi, rt);
                if (spu > 1) {   // every lane waits (acquire): no warp-level hand-over needed afterwards
                    unsigned polls = 0;
                    unsigned long long t0 = 0;
                    while (!mbar_try(&unit_bar[ul], 0)) {
                        if ((++polls & 1023u) == 0) {
                            if (*(volatile int*)p.status != 0) break;
                            const unsigned long long now = global_ns();
                            if (t0 == 0) t0 = now;
                            else if (now - t0 > 2 * p.wait_ns) {   // longer than any data wait: the root cause gets recorded first
                                if (atomicCAS(p.status, 0, Q4_ERR_TIMEOUT) == 0) p.status[1] = 0x90000 + pi;
                                break;
                            }
                        }
                    }
                }
                float oldf = 0.f;
                if (epi == EPI_RESIDUAL) {
                    // Old x = the other buffer's g partials (this CTA staged that whole buffer in an earlier phase, so
                    // they have arrived), summed in rank order in fp32 and rounded to fp16 as every reader sums them.
                    uint32_t o1 = resid, o2 = resid2;
                    if (ul != resid_unit) {
                        const int n0 = unit_at(ul, cta, grid) * 8;
                        o1 = (lane >> 3) < p.g ? ld_tagged(oldx + n0) : 0u;
                        o2 = (lane >> 3) + 4 < p.g ? ld_tagged(oldx + 4 * (size_t)kLLMaxDim + n0) : 0u;
                    }
                    const float f1 = __half2float(__ushort_as_half((unsigned short)(o1 & 0xFFFFu)));
                    const float f2 = __half2float(__ushort_as_half((unsigned short)(o2 & 0xFFFFu)));
                    float o = 0.f;
#pragma unroll
                    for (int s2 = 0; s2 < 4; s2++) {
                        const float v = __shfl_sync(0xffffffffu, f1, (lane & 7) + 8 * s2);
                        if (s2 < p.g) o += v;
                    }
#pragma unroll
                    for (int s2 = 0; s2 < 4; s2++) {
                        const float v = __shfl_sync(0xffffffffu, f2, (lane & 7) + 8 * s2);
                        if (s2 + 4 < p.g) o += v;
                    }
                    oldf = __half2float(__float2half(o));
                }
                if (lane < 8) {
                    const int r = lane;
                    const float* pu = part + (size_t)ul * spu * 8 + r;
                    // per-slot partials in slot order; four loads in flight at a time
                    auto sum_slots = [&](const float* q) {
                        float acc = 0.f;
                        for (int k2 = 0; k2 < nkt; k2 += 4) {
                            const float v0 = q[k2 * 8], v1 = k2 + 1 < nkt ? q[(k2 + 1) * 8] : 0.f;
                            const float v2 = k2 + 2 < nkt ? q[(k2 + 2) * 8] : 0.f, v3 = k2 + 3 < nkt ? q[(k2 + 3) * 8] : 0.f;
                            acc += v0; acc += v1; acc += v2; acc += v3;
                        }
                        return acc;
                    };
                    float sum = sum_slots(pu);
                    const int n = rt * 8 + r;
                    if (epi == EPI_SILU) {
                        const float up = sum_slots(pu + nkt * 8);
                        st_tagged(ph.m[0].out + n, tagged(__float2half(silu_mul(sum, up)), out_tag));
                    } else if (epi == EPI_RESIDUAL) {
                        // This rank's partial of the new x goes into its slot on every rank. Ordering: a rank that writes
                        // buffer b has, for every other rank, consumed data which that rank produced after its last read
                        // of b (o projection: the peer's down-projection partials of the previous layer, read while
                        // staging QKV; down projection: the peer's o-projection partials, read while staging gate/up),
                        // so no reader is overtaken.
                        sum += oldf / p.gpu_count;   // each rank adds x / g (gpu_kernels.h:237-238)
                        const uint32_t word = tagged(__float2half(sum), out_tag);
                        const size_t off2 = (size_t)p.rank * kLLMaxDim + n;
                        if (Q4_DBG(p) & 16) {
                            // measurement only: the same stores, but all into this rank's own area (zeros as the peers'
                            // partials), so that no step waits on NVLink: step time minus this = exposed exchange time
                            for (int r2 = 0; r2 < p.g; r2++)
                                st_tagged(p.xb[ph.xbuf_out][p.rank] + (size_t)r2 * kLLMaxDim + n, r2 == p.rank ? word : out_tag);
                        } else {
                            for (int peer = 0; peer < p.g; peer++) st_tagged(p.xb[ph.xbuf_out][peer] + off2, word);
                        }
                    } else {
                        const FMat& m = ph.m[mi];
                        const __half hv = __float2half(sum);
                        st_tagged(m.out + n, tagged(hv, out_tag));
                        if (m.out_plain) m.out_plain[ph.loff + (long long)pos * m.n + n] = hv;   // V row into the cache for later tokens
                    }
                }
                SLOT_TRACE(3);
            }
            sbase += nslots;
            ent0 += (nslots + 1) >> 1;
            TRACE(2);
            phase_fetch_wait();
            if (ph.barrier_after) grid_barrier(p, nbar, ctid, &s_abort);
            else consumer_sync();  // closes the phase
            TRACE(3);

        } else if (ph.type == PH_ATTN) {
            // ---- attention of one query per head over positions 0..pos, split over CTAs (llama2_q4.cu:410-427) ----
            float* sm_m = reinterpret_cast<float*>(xq);          // [kAG]
            float* sm_l = sm_m + kAG;                            // [kAG]
            float* sm_acc = sm_l + kAG;                          // [kAG][128]
            const int lane8 = ctid & 7, grp = ctid >> 3;
            const int d0 = lane8 * 16;                           // this lane's 16 head dims; RoPE partner dims are d0 ^ 64
            const bool upper = d0 >= 64;
            const int i0 = upper ? d0 - 64 : d0;
            const int T = pos + 1;
            const float alpha = (float)(1.0 / sqrt((double)HS));
            const int ns = attn_splits_for(p, T);
            const int nitems = p.n_heads * ns;
            const uint32_t want = tag_of(p, ph.in_phase), out_tag = tag_of(p, pi);
            const __half* kc = p.kc + ph.loff;
            const __half* vc = p.vc + ph.loff;
            // (cos, sin) of this position for dims i0..i0+15: RoPE of gpu_kernels.h:340-363, tabulated at load time
            float2 cs[16];
            {
                const float4* tp = reinterpret_cast<const float4*>(p.rope + ((size_t)pos * (HS / 2) + i0) * 2);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float4 t4 = __ldg(tp + j);
                    cs[2 * j] = make_float2(t4.x, t4.y);
                    cs[2 * j + 1] = make_float2(t4.z, t4.w);
                }
            }
            for (int id = cta; id < nitems; id += grid) {
                const int h = id / ns, split = id % ns;
                const int kvh = h / p.kv_mul;
                const int units = (T + kAG - 1) / kAG;
                const int u0 = (int)((long long)units * split / ns), u1 = (int)((long long)units * (split + 1) / ns);
                const int t0 = u0 * kAG, t1 = min(u1 * kAG, T);
                const size_t col = (size_t)kvh * HS + d0;
                // first step's K/V rows are requested before anything else so that their latency overlaps the query set-up
                uint4 kn[2], vn[2];
                auto fetch = [&](int tb) {
                    int t = tb + grp;
                    if (t >= t1) t = t0;
                    if (tb < t1 && t != pos) {   // the new position's K and V come from the tagged staging vectors
                        const uint4* vr = reinterpret_cast<const uint4*>(vc + (size_t)t * p.kv_n + col);
                        vn[0] = __ldcg(vr); vn[1] = __ldcg(vr + 1);
                        const uint4* kr = reinterpret_cast<const uint4*>(kc + (size_t)t * p.kv_n + col);
                        kn[0] = __ldcg(kr); kn[1] = __ldcg(kr + 1);
                    }
                };
                fetch(t0);
                // rotated query (fp16-rounded like the reference's in-place rotation)
                float qf[16];
                {
                    const uint32_t* qp = p.q + (size_t)h * HS + i0;
                    uint4 lo4[2], hi4[2];
                    unsigned polls = 0;
                    unsigned long long tw = 0;
                    for (;;) {   // the query arrives tagged from the QKV phase: this poll is the op boundary
                        uint32_t bad = 0;
                        lo4[0] = load_tagged8(qp, want, bad); lo4[1] = load_tagged8(qp + 8, want, bad);
                        hi4[0] = load_tagged8(qp + 64, want, bad); hi4[1] = load_tagged8(qp + 72, want, bad);
                        if (bad == 0 || !keep_polling(polls, tw, p.status, p.wait_ns, 0x20000 + pi)) break;
                    }
                    const __half* lo = reinterpret_cast<const __half*>(lo4);
                    const __half* hi = reinterpret_cast<const __half*>(hi4);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float l0 = __half2float(lo[j]), h0 = __half2float(hi[j]);
                        const float r = upper ? (l0 * cs[j].y + h0 * cs[j].x) : (l0 * cs[j].x - h0 * cs[j].y);
                        qf[j] = __half2float(__float2half(r));
                    }
                }
                float m = -CUDART_INF_F, l = 0.f, acc[16];
#pragma unroll
                for (int j = 0; j < 16; j++) acc[j] = 0.f;
                for (int tb = t0; tb < t1; tb += kAG) {
                    const int t = tb + grp;
                    const bool valid = t < t1;
                    const int tt = valid ? t : t0;
                    const uint4 kcur[2] = {kn[0], kn[1]}, vcur[2] = {vn[0], vn[1]};
                    fetch(tb + kAG);  // next step's rows in flight during this step's math
                    float kf[16], vf[16];
                    if (tt == pos) {
                        // the new key is un-rotated in knew: rotate it here; the head group's first query head also files it
                        const uint32_t* kp = p.knew + (size_t)kvh * HS + i0;
                        const uint32_t* vp = p.vnew + (size_t)kvh * HS + d0;
                        uint4 lo4[2], hi4[2], vnew4[2];
                        unsigned polls = 0;
                        unsigned long long tw = 0;
                        for (;;) {
                            uint32_t bad = 0;
                            lo4[0] = load_tagged8(kp, want, bad); lo4[1] = load_tagged8(kp + 8, want, bad);
                            hi4[0] = load_tagged8(kp + 64, want, bad); hi4[1] = load_tagged8(kp + 72, want, bad);
                            vnew4[0] = load_tagged8(vp, want, bad); vnew4[1] = load_tagged8(vp + 8, want, bad);
                            if (bad == 0 || !keep_polling(polls, tw, p.status, p.wait_ns, 0x30000 + pi)) break;
                        }
                        {
                            const __half2* hh = reinterpret_cast<const __half2*>(vnew4);
#pragma unroll
                            for (int j = 0; j < 8; j++) { const float2 a = __half22float2(hh[j]); vf[2 * j] = a.x; vf[2 * j + 1] = a.y; }
                        }
                        const __half* lo = reinterpret_cast<const __half*>(lo4);
                        const __half* hi = reinterpret_cast<const __half*>(hi4);
                        uint4 store[2];
                        __half* sh = reinterpret_cast<__half*>(store);
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const float l0 = __half2float(lo[j]), h0 = __half2float(hi[j]);
                            const float r = upper ? (l0 * cs[j].y + h0 * cs[j].x) : (l0 * cs[j].x - h0 * cs[j].y);
                            sh[j] = __float2half(r);
                            kf[j] = __half2float(sh[j]);
                        }
                        if (valid && (h % p.kv_mul) == 0) {
                            uint4* dst = reinterpret_cast<uint4*>(p.kc + ph.loff + (size_t)pos * p.kv_n + col);
                            dst[0] = store[0];
                            dst[1] = store[1];
                        }
                    } else {
                        const __half2* hh = reinterpret_cast<const __half2*>(kcur);
#pragma unroll
                        for (int j = 0; j < 8; j++) { const float2 a = __half22float2(hh[j]); kf[2 * j] = a.x; kf[2 * j + 1] = a.y; }
                    }
                    if (tt != pos) {
                        const __half2* hh = reinterpret_cast<const __half2*>(vcur);
#pragma unroll
                        for (int j = 0; j < 8; j++) { const float2 a = __half22float2(hh[j]); vf[2 * j] = a.x; vf[2 * j + 1] = a.y; }
                    }
                    float sc = 0.f;
#pragma unroll
                    for (int j = 0; j < 16; j++) sc = fmaf(kf[j], qf[j], sc);
                    sc += __shfl_xor_sync(0xffffffffu, sc, 1);
                    sc += __shfl_xor_sync(0xffffffffu, sc, 2);
                    sc += __shfl_xor_sync(0xffffffffu, sc, 4);
                    if (valid) {
                        sc = __half2float(__float2half(sc * alpha));  // scores are fp16 in the reference (gpu_kernels.h:171-175)
                        const float mn = fmaxf(m, sc);
                        const float corr = expf(m - mn);
                        const float pr = expf(sc - mn);
                        l = l * corr + pr;
#pragma unroll
                        for (int j = 0; j < 16; j++) acc[j] = fmaf(pr, vf[j], acc[j] * corr);
                        m = mn;
                    }
                }
                // merge the lane groups of this CTA; the splits of a head are merged by the consumers of the o projection
                // while they stage their input (stage_x_quant, attn_in), so no second grid-wide step is needed here
                // first the four lane groups of each warp (lanes 8 and 16 apart) in registers, then the warps through shared memory
#pragma unroll
                for (int o = 8; o <= 16; o <<= 1) {
                    const float mo = __shfl_xor_sync(0xffffffffu, m, o), lo2 = __shfl_xor_sync(0xffffffffu, l, o);
                    const float mn = fmaxf(m, mo);
                    const float ca = m == -CUDART_INF_F ? 0.f : __expf(m - mn), cb = mo == -CUDART_INF_F ? 0.f : __expf(mo - mn);
                    l = l * ca + lo2 * cb;
#pragma unroll
                    for (int j = 0; j < 16; j++) acc[j] = acc[j] * ca + __shfl_xor_sync(0xffffffffu, acc[j], o) * cb;
                    m = mn;
                }
                if (lane == 0) { sm_m[cw] = m; sm_l[cw] = l; }
                if (lane < 8) {
#pragma unroll
                    for (int j = 0; j < 16; j++) sm_acc[cw * 128 + d0 + j] = acc[j];
                }
                consumer_sync();
                // Slot (h, split) of a fixed [heads][nsplit] layout. The CTA that writes a head's last split in use also stamps
                // the head's unused slots with this launch's tag: every slot is rewritten by every launch, so a slot that
                // comes into use when the context grows never holds a tag from thousands of launches ago that could equal
                // (modulo 2^16) the tag its first reader waits for.
                uint32_t* outp = p.attn_part + ((size_t)h * p.nsplit + split) * kAttnPartStride;
                if (split == ns - 1 && ctid < kAttnPartStride)
                    for (int s2 = ns; s2 < p.nsplit; s2++) st_tagged(p.attn_part + ((size_t)h * p.nsplit + s2) * kAttnPartStride + ctid, out_tag);
                if (ctid < HS) {
                    float M = -CUDART_INF_F;
#pragma unroll
                    for (int g2 = 0; g2 < kCW; g2++) M = fmaxf(M, sm_m[g2]);
                    float a = 0.f, L = 0.f;
#pragma unroll
                    for (int g2 = 0; g2 < kCW; g2++) {
                        if (sm_m[g2] != -CUDART_INF_F) {
                            const float w = __expf(sm_m[g2] - M);
                            a += sm_acc[g2 * 128 + ctid] * w;
                            L += sm_l[g2] * w;
                        }
                    }
                    // the split's own softmax-weighted V average (|.| <= max |V|, safe in fp16) plus its (max, sum)
                    st_tagged(outp + ctid, tagged(__float2half(L > 0.f ? a / L : 0.f), out_tag));
                    if (ctid == 0) {
                        const uint32_t mb = __float_as_uint(M), lb = __float_as_uint(L);
                        st_tagged4(outp + 128, make_uint4(out_tag | (mb & 0xFFFFu), out_tag | (mb >> 16), out_tag | (lb & 0xFFFFu), out_tag | (lb >> 16)));
                    }
                }
                if (id + grid < nitems) consumer_sync();   // the merge buffers are reused by this CTA's next item
            }
            TRACE(2);
            phase_fetch_wait();
            consumer_sync();   // no grid barrier: the partials are tagged and the o projection polls them
            TRACE(3);

        } else if (ph.type == PH_CLS) {
            // ---- classifier: fp16 rows streamed through the same ring; per-CTA argmax candidate ----
            __half* xf = reinterpret_cast<__half*>(xq);
            stage_x_f16(ph, p, xf, red, ctid);
            TRACE(1);
            const int nunits = ph.nunits, nkt = ph.nkt, K = ph.K;
            const float inv_nkt = 1.0f / (float)nkt;
            const int lt = unit_count(nunits, cta, grid) * 2;        // rows of this CTA (units are row pairs)
            const int nslots = lt * nkt;
            const unsigned first = (cw + kCW - (sbase % kCW)) % kCW;
            for (unsigned li = first; li < (unsigned)nslots; li += kCW) {
                {
                    const int kc = li - fast_div(li, inv_nkt) * nkt;
                    const int len = min(kClsChunk, K - kc * kClsChunk);
                    const unsigned en = ent0 + (li >> 1);
                    const int eq = fast_div(en, inv_entries), e = (int)en - eq * kEntries;
                    int off = 0;
                    if (li & 1) { const int kcp = kc > 0 ? kc - 1 : nkt - 1; off = min(kClsChunk, K - kcp * kClsChunk) * 2; }
                    if (!(Q4_DBG(p) & 2) && (failed || !mbar_wait(&full_bar[e], eq & 1, p.status, p.wait_ns, &s_round[e], (unsigned)eq))) { failed = true; continue; }
                    const uint4* wv = reinterpret_cast<const uint4*>(ring + (size_t)e * kEntryBytes + off);
                    const uint4* xv = reinterpret_cast<const uint4*>(xf + kc * kClsChunk);
                    float a4[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) a4[j] = 0.f;
                    const int nvec = len >> 3;
                    for (int i = lane; i < nvec; i += 128) {
                        uint4 w[4], xx[4];
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int ii = i + u * 32;
                            w[u] = ii < nvec ? wv[ii] : make_uint4(0, 0, 0, 0);
                            xx[u] = ii < nvec ? xv[ii] : make_uint4(0, 0, 0, 0);
                        }
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const __half* wh = reinterpret_cast<const __half*>(&w[u]);
                            const __half* xh = reinterpret_cast<const __half*>(&xx[u]);
#pragma unroll
                            for (int j = 0; j < 8; j++) a4[j] = fma_mixed(wh[j], xh[j], a4[j]);
                        }
                    }
                    float a = ((a4[0] + a4[1]) + (a4[2] + a4[3])) + ((a4[4] + a4[5]) + (a4[6] + a4[7]));
                    a = warp_sum(a);
                    if (lane == 0) part[li] = a;
                    __syncwarp();
                    if (lane == 0 && !(Q4_DBG(p) & 2)) mbar_arrive(&empty_bar[e], (!(li & 1) && li + 1 == (unsigned)nslots) ? 2 : 1);
                }
            }
            sbase += nslots;
            ent0 += (nslots + 1) >> 1;
            consumer_sync();
            float best = -CUDART_INF_F;
            int bi = 0x7fffffff;
            for (int e = ctid; e < lt; e += kCT) {
                float sum = 0.f;
                for (int kc = 0; kc < nkt; kc++) sum += part[e * nkt + kc];
                const int n = p.vocab_off + unit_at(e >> 1, cta, grid) * 2 + (e & 1);   // global vocabulary index
                const __half hv = __float2half(sum);
                if (p.g == 1) p.logits[n] = hv;
                else   // the all-gather of the logits: this rank's slice goes to every rank (plain peer stores)
                    for (int peer = 0; peer < p.g; peer++) p.ll_logits[(Q4_DBG(p) & 16) ? p.rank : peer][n] = __half_as_ushort(hv);
                const float v = __half2float(hv);
                if (v > best || (v == best && n < bi)) { best = v; bi = n; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
            }
            float* cv = reinterpret_cast<float*>(part);  // reuse after the logits are out
            consumer_sync();
            if (lane == 0) { cv[cw] = best; reinterpret_cast<int*>(cv)[kCW + cw] = bi; }
            consumer_sync();
            if (ctid == 0) {
                for (int w2 = 1; w2 < kCW; w2++) {
                    const float ov = cv[w2];
                    const int oi = reinterpret_cast<int*>(cv)[kCW + w2];
                    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
                }
                p.cand_val[cta] = best;
                p.cand_idx[cta] = bi;
            }
            TRACE(2);
            phase_fetch_wait();
            grid_barrier(p, nbar, ctid, &s_abort);
            TRACE(3);

        } else if (ph.type == PH_ARGMAX) {
            // ---- greedy hand-off (gpu_kernels.h:456-501): lowest index among equal maxima ----
            if (cta == 0 && cw == 0) {
                float best = -CUDART_INF_F;
                int bi = 0x7fffffff;
                for (int c = lane; c < grid; c += 32) {
                    const float ov = __ldcg(p.cand_val + c);
                    const int oi = __ldcg(p.cand_idx + c);
                    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
                }
                if (p.g > 1) {
                    // Exchange of the ranks' candidates: two tagged 64-bit words per rank, stored into every rank's
                    // mailbox. The system-scope fence orders this rank's logits slice (stored by all its CTAs before
                    // the grid barrier above) before the candidate, so a rank that holds all candidates also holds all
                    // logits. Every rank picks the same winner (highest value, lowest index).
                    const unsigned long long tg = (unsigned long long)(tag_of(p, pi) >> 16) << 32;
                    const size_t slot = ((size_t)p.launch_parity * Q4_MAX_GPUS + p.rank) * 2;
                    if (lane == 0) {
                        __threadfence_system();
                        for (int peer = 0; peer < p.g; peer++) {
                            // (debug 16: into this rank's own mailbox, once per rank slot)
                            unsigned long long* dst = (Q4_DBG(p) & 16) ? p.cand[p.rank] + ((size_t)p.launch_parity * Q4_MAX_GPUS + peer) * 2 : p.cand[peer] + slot;
                            asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(dst), "l"(tg | __float_as_uint(best)) : "memory");
                            asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(dst + 1), "l"(tg | (unsigned)bi) : "memory");
                        }
                    }
                    best = -CUDART_INF_F;
                    bi = 0x7fffffff;
                    if (lane < p.g) {
                        const unsigned long long* src = p.cand[p.rank] + ((size_t)p.launch_parity * Q4_MAX_GPUS + lane) * 2;
                        unsigned long long w0, w1;
                        unsigned polls = 0;
                        unsigned long long t0 = 0;
                        for (;;) {
                            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w0) : "l"(src) : "memory");
                            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w1) : "l"(src + 1) : "memory");
                            if (((w0 ^ tg) >> 32) == 0 && ((w1 ^ tg) >> 32) == 0) { best = __uint_as_float((unsigned)w0); bi = (int)(unsigned)w1; break; }
                            if (!keep_polling(polls, t0, p.status, p.wait_ns, 0x70000 + lane)) break;
                        }
                    }
                    __threadfence_system();
#pragma unroll
                    for (int o = 4; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
                    }
                }
                if (lane == 0 && !p.no_handoff) {
                    int token_pos = *p.pos_pinned;
                    token_pos++;
                    if (p.write_token) p.tokens_pinned[token_pos] = (bi == 0x7fffffff) ? 0 : bi;
                    *p.pos_pinned = token_pos;
                    *p.pos_dev = token_pos;
                }
            }
            if (cta == 0 && p.g > 1) {
                // all candidates are in, hence all logits slices: copy the gathered vector where the host reads it
                consumer_sync();
                const uint4* src = reinterpret_cast<const uint4*>(p.ll_logits[p.rank]);
                uint4* dst = reinterpret_cast<uint4*>(p.logits);
                for (int i = ctid; i < p.cfg.vocab_size / 8; i += kCT) dst[i] = __ldcg(src + i);
                for (int i = (p.cfg.vocab_size / 8) * 8 + ctid; i < p.cfg.vocab_size; i += kCT)
                    p.logits[i] = __ushort_as_half(__ldcg(p.ll_logits[p.rank] + i));
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// Stream-layout builder (device): one block of 40 threads per (tile, group) unit.
// ------------------------------------------------------------------------------------------------------------
__global__ void repack_kernel(uint8_t* dst, const uint32_t* w, const uint32_t* z, const __half* s, int K, int N, int PW, int PZ, int G) {
    const int rt = blockIdx.y, g = blockIdx.x;
    const int kt = g / kSlotGroups, gl = g % kSlotGroups;
    const int ng = min(kSlotGroups, G - kt * kSlotGroups), nl = 2 * ng;
    uint8_t* block = dst + ((size_t)rt * G + (size_t)kt * kSlotGroups) * kUnitBytes;
    const int t = threadIdx.x;
    if (t < 32) {
        const int r = t >> 2, c = t & 3;  // row, chunk of 32 inputs inside the group
        const int h = c >> 1, j2 = c & 1, lane = 2 * gl + h;
        const int word0 = g * 16 + c * 4;
        uint4 v = make_uint4(0, 0, 0, 0);
        const uint32_t* src = w + (size_t)(rt * 8 + r) * PW;
        if (word0 + 0 < PW) v.x = src[word0 + 0];
        if (word0 + 1 < PW) v.y = src[word0 + 1];
        if (word0 + 2 < PW) v.z = src[word0 + 2];
        if (word0 + 3 < PW) v.w = src[word0 + 3];
        reinterpret_cast<uint4*>(block)[(j2 * 8 + r) * nl + lane] = v;
    } else if (t < 40) {
        const int r = t - 32, n = rt * 8 + r;
        uint8_t* meta = block + ng * 512 + gl * 32;
        reinterpret_cast<__half*>(meta)[r] = s[(size_t)n * G + g];
        meta[16 + r] = (uint8_t)((z[(size_t)n * PZ + (g >> 3)] >> (4 * (g & 7))) & 0xFu);
        meta[24 + r] = 0;
    }
}

// (cos, sin) of every position and frequency, with the reference's expressions (gpu_kernels.h:346-350).
__global__ void rope_table_kernel(float2* out, int seq_len, int head_size, float theta) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int half_hs = head_size / 2;
    if (i >= seq_len * half_hs) return;
    const int pos = i / half_hs, d = i % half_hs;
    const int head_dim = (d * 2) % head_size;
    const float freq = 1.0f / powf(theta, head_dim / (float)head_size);
    const float val = pos * freq;
    out[i] = make_float2(cosf(val), sinf(val));
}

// Builds the per-CTA copy lists with the same cursor the consumers' slot arithmetic mirrors: entries never span a
// phase, two consecutive slots of a phase share an entry. One thread per CTA of the decode kernel; runs once.
__global__ void build_desc_kernel(const FParams p, CopyDesc* desc, int* desc_count, int grid) {
    __shared__ __align__(16) FPhase cache;
    const int cta = blockIdx.x;
    SlotCursor rc;
    cursor_init(rc);
    rc.cache = &cache;
    const uint8_t* src;
    uint32_t bytes;
    int phase;
    CopyDesc* out = desc + (size_t)cta * p.desc_stride;
    int n = 0;
    bool have = cursor_next(rc, p, cta, grid, src, bytes, phase);
    while (have && n < p.desc_stride) {
        CopyDesc d;
        d.src0 = src;
        d.bytes0 = bytes;
        d.src1 = nullptr;
        d.bytes1 = 0;
        d.pad[0] = d.pad[1] = 0;
        const int phaseA = phase;
        have = cursor_next(rc, p, cta, grid, src, bytes, phase);
        if (have && phase == phaseA) {
            if (src == d.src0 + d.bytes0) d.bytes0 += bytes;
            else { d.src1 = src; d.bytes1 = bytes; }
            have = cursor_next(rc, p, cta, grid, src, bytes, phase);
        }
        out[n++] = d;
    }
    desc_count[cta] = have ? -1 : n;  // -1: list too short (host bug)
}

size_t stream_bytes(int K, int N) { return (size_t)(N / 8) * q4_groups(K) * kUnitBytes; }

}  // namespace

struct q4_fused {
    std::vector<void*> allocs;
    FPhase* d_phases = nullptr;
    int nphases = 0;
    FParams params;
    size_t smem_bytes = 0;
    int grid = 0;
    int barriers_per_launch = 0;
    unsigned long long launches = 0;
    bool unsupported = false;
    unsigned long long* trace = nullptr;
    unsigned long long* slot_trace = nullptr;
    Q4LLArea* ll_local = nullptr;   // this rank's exchange area (inside the communicator's inbox, or own allocation at g = 1)
    size_t attn_part_bytes = 0;
    bool armed = false;             // buffers and counters are in their initial state or in step with the launches so far
    unsigned long long wait_ns = kDefaultWaitNs;
};

#ifdef Q4_TEST_BUILD
// Switches of the test build (see Q4_DBG): set through exported functions, never through the environment.
static int g_test_debug = 0, g_test_split_len = 0, g_test_entries = 0;
static int g_test_fail_alloc = -1;   // >= 0: the allocation with this running index fails once (host-side fault injection)
static int g_test_alloc_index = 0;
extern "C" void q4_test_set_fused_debug(int bits) { g_test_debug = bits; }
extern "C" void q4_test_set_split_len(int positions) { g_test_split_len = positions; }
extern "C" void q4_test_set_ring_entries(int n) { g_test_entries = n; }
extern "C" void q4_test_fail_fused_alloc(int index) { g_test_fail_alloc = index; g_test_alloc_index = 0; }
#endif

static int fused_alloc(q4_fused* f, void** p, size_t bytes) {
#ifdef Q4_TEST_BUILD
    if (g_test_fail_alloc >= 0 && g_test_alloc_index++ == g_test_fail_alloc) { g_test_fail_alloc = -1; return Q4_ERR_CUDA; }
#endif
    Q4_CUDA_TRY(cudaMalloc(p, bytes));
    f->allocs.push_back(*p);
    return Q4_OK;
}

static int make_stream(q4_fused* f, const DevQW& q, const uint8_t** out) {
    uint8_t* d = nullptr;
    if (int e = fused_alloc(f, (void**)&d, stream_bytes(q.K, q.N))) return e;
    repack_kernel<<<dim3(q4_groups(q.K), q.N / 8), 64>>>(d, q.w.weight, q.w.zeros, (const __half*)q.w.scales, q.K, q.N, q4_pw(q.K),
                                                        q4_pz(q.K), q4_groups(q.K));
    Q4_CUDA_TRY(cudaGetLastError());
    *out = d;
    return Q4_OK;
}

void q4_fused_free(q4_model* m) {
    if (!m->fused) return;
    for (void* p : m->fused->allocs) cudaFree(p);
    delete m->fused;
    m->fused = nullptr;
}

// Called by q4_model_reset. Launch and barrier counters (and with them the activation tags) simply keep counting
// across generations; only after a recorded error is everything re-armed from zero. In a tensor-parallel group the
// ranks' tags must stay in step and a rank's exchange area is written by its peers, so after an error (as after
// q4_model_prepare) every rank has to finish its reset before any rank launches again: the callers put a host
// barrier there.
void q4_fused_reset(q4_model* m) {
    if (!m->fused || m->fused->unsupported) return;
    q4_fused* f = m->fused;
    int st = 0;
    cudaDeviceSynchronize();
    if (f->armed && cudaMemcpy(&st, f->params.status, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess && st == 0) return;
    f->armed = false;
    const q4_config& c = m->cfg;
    bool ok = true;
    ok &= cudaMemset(f->params.bar_counter, 0, sizeof(unsigned long long)) == cudaSuccess;
    ok &= cudaMemset(f->params.status, 0, (4 + 4 * 256) * sizeof(int)) == cudaSuccess;
    ok &= cudaMemset(f->ll_local->x, 0, sizeof(f->ll_local->x)) == cudaSuccess;
    ok &= cudaMemset(f->ll_local->cand, 0, sizeof(f->ll_local->cand)) == cudaSuccess;
    ok &= cudaMemset(f->params.hb, 0, 4 * (size_t)c.hidden_dim) == cudaSuccess;
    ok &= cudaMemset(f->params.q, 0, 4 * (size_t)c.dim) == cudaSuccess;
    ok &= cudaMemset(f->params.attn_part, 0, f->attn_part_bytes) == cudaSuccess;
    ok &= cudaMemset(f->params.knew, 0, 4 * (size_t)m->kv_n) == cudaSuccess;
    ok &= cudaMemset(f->params.vnew, 0, 4 * (size_t)m->kv_n) == cudaSuccess;
    ok &= cudaDeviceSynchronize() == cudaSuccess;  // the memsets run on the default stream; forward calls use the caller's stream
    f->launches = 0;
    f->armed = ok;
}

// Limit of every device-side wait of the fused kernel (default two seconds); takes effect with the next launch.
void q4_fused_set_wait_limit(q4_model* m, unsigned long long ns) {
    if (m->fused && !m->fused->unsupported) m->fused->wait_ns = ns ? ns : kDefaultWaitNs;
}

int q4_fused_status(q4_model* m) {
    if (!m->fused || m->fused->unsupported) return Q4_OK;
    int st[4] = {0, 0, 0, 0};
    Q4_CUDA_TRY(cudaMemcpy(st, m->fused->params.status, sizeof(st), cudaMemcpyDeviceToHost));
    if (st[0] != 0) {
        fprintf(stderr, "q4 fused path: a bounded device-side wait ran out (status %d, location 0x%x)\n", st[0], st[1]);
#ifdef Q4_TEST_BUILD
        if (g_test_debug & 32) {
            int prog[256];
            cudaMemcpy(prog, m->fused->params.status + 4, sizeof(prog), cudaMemcpyDeviceToHost);
            fprintf(stderr, "  phase reached per CTA:");
            for (int i = 0; i < m->fused->grid && i < 256; i++) fprintf(stderr, " %d", prog[i]);
            fprintf(stderr, "\n  detail 0x%x 0x%x; barriers arrived per CTA:", st[2], st[3]);
            cudaMemcpy(prog, m->fused->params.status + 4 + 256, sizeof(prog), cudaMemcpyDeviceToHost);
            for (int i = 0; i < m->fused->grid && i < 256; i++) fprintf(stderr, " %d", prog[i]);
            fprintf(stderr, "\n");
        }
#endif
    }
    return st[0];
}

static int fused_build(q4_model* m, q4_fused* f);

// Builds the fused path's state into a private object and publishes it in the model only when every step has
// succeeded. A model that the path cannot serve is remembered as such (an empty object with `unsupported` set); any
// other failure (out of memory, a CUDA error) frees what was allocated and leaves the model as it was, so that a later
// call starts from scratch instead of launching a half-built state.
int q4_fused_prepare(q4_model* m) {
    if (m->fused) return m->fused->unsupported ? Q4_ERR_UNSUPPORTED_SIZE : Q4_OK;
    q4_fused* f = new q4_fused();
    int e = fused_build(m, f);
    if (e == Q4_OK) {
        m->fused = f;
        q4_fused_reset(m);
        if (cudaDeviceSynchronize() != cudaSuccess || !f->armed) e = Q4_ERR_CUDA;
        if (e == Q4_OK) return Q4_OK;
        m->fused = nullptr;
    }
    for (void* p : f->allocs) cudaFree(p);
    f->allocs.clear();
    if (e == Q4_ERR_UNSUPPORTED_SIZE && f->unsupported) {
        m->fused = f;
        return e;
    }
    delete f;
    return e;
}

static int fused_build(q4_model* m, q4_fused* f) {
    const q4_config& c = m->cfg;
    const int g = m->g;
    if (m->column || m->head_size != 128 || (c.dim % 128) || (m->h_kc % 8) || c.dim > 4 * kCT * 8 ||   // 4 = staging batch
        c.dim > kLLMaxDim || c.vocab_size > kLLMaxVocab || (m->v_n % 2) || (m->kv_n % 128) || (m->q_n % 128) ||
        (g > 1 && (!m->comm || q4_comm_world(m->comm) != g || q4_comm_rank(m->comm) != m->rank))) {
        f->unsupported = true;
        return Q4_ERR_UNSUPPORTED_SIZE;
    }
    int dev = 0, sms = 0, coop = 0;
    Q4_CUDA_TRY(cudaGetDevice(&dev));
    Q4_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    Q4_CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) { f->unsupported = true; return Q4_ERR_UNSUPPORTED_SIZE; }
    f->grid = sms;

    FParams& p = f->params;
    memset(&p, 0, sizeof(p));
    p.cfg = c;
    p.head_size = m->head_size;
    p.kv_n = m->kv_n;
    p.kv_mul = m->kv_mul;
    p.n_heads = c.n_heads / g;    // this rank's query heads
    p.nsplit = std::min(kMaxSplit, std::max(1, sms / p.n_heads));
    p.gpu_count = (float)g;
    p.g = g;
    p.rank = m->rank;
    p.vocab_off = m->rank * m->v_n;
    p.logits = (__half*)m->logits;
    p.kc = (__half*)m->kc; p.vc = (__half*)m->vc;
    p.emb = (const __half*)m->emb; p.wcls = (const __half*)m->wcls;
    p.pos_dev = m->pos;
    p.tokens_pinned = (int*)m->shared->tokens;
    p.pos_pinned = &m->shared->pos;
    int e;
#define FTRY(expr) do { e = (expr); if (e != Q4_OK) return e; } while (0)
    if (g > 1) {
        for (int r = 0; r < g; r++) {
            Q4LLArea* a = q4_comm_ll_area(m->comm, r);
            if (!a) { f->unsupported = true; return Q4_ERR_UNSUPPORTED_SIZE; }
            p.xb[0][r] = &a->x[0][0][0];
            p.xb[1][r] = &a->x[1][0][0];
            p.cand[r] = &a->cand[0][0][0];
            p.ll_logits[r] = a->logits;
        }
        f->ll_local = q4_comm_ll_area(m->comm, m->rank);
    } else {
        FTRY(fused_alloc(f, (void**)&f->ll_local, sizeof(Q4LLArea)));
        p.xb[0][0] = &f->ll_local->x[0][0][0];
        p.xb[1][0] = &f->ll_local->x[1][0][0];
        p.cand[0] = &f->ll_local->cand[0][0][0];
        p.ll_logits[0] = f->ll_local->logits;
    }
    FTRY(fused_alloc(f, (void**)&p.hb, 4 * (size_t)c.hidden_dim));
    FTRY(fused_alloc(f, (void**)&p.q, 4 * (size_t)c.dim));
    FTRY(fused_alloc(f, (void**)&p.knew, 4 * (size_t)m->kv_n));
    FTRY(fused_alloc(f, (void**)&p.vnew, 4 * (size_t)m->kv_n));
    Q4_CUDA_TRY(cudaMemset(p.hb, 0, 4 * (size_t)c.hidden_dim));
    Q4_CUDA_TRY(cudaMemset(p.q, 0, 4 * (size_t)c.dim));
    Q4_CUDA_TRY(cudaMemset(p.knew, 0, 4 * (size_t)m->kv_n));
    Q4_CUDA_TRY(cudaMemset(p.vnew, 0, 4 * (size_t)m->kv_n));
    f->attn_part_bytes = sizeof(uint32_t) * (size_t)p.n_heads * p.nsplit * kAttnPartStride;
    FTRY(fused_alloc(f, (void**)&p.attn_part, f->attn_part_bytes));
    Q4_CUDA_TRY(cudaMemset(p.attn_part, 0, f->attn_part_bytes));
    {
        float2* rope = nullptr;
        const int n = c.seq_len * (m->head_size / 2);
        FTRY(fused_alloc(f, (void**)&rope, sizeof(float2) * (size_t)n));
        rope_table_kernel<<<q4_div_up(n, 256), 256>>>(rope, c.seq_len, m->head_size, c.rope_theta);
        Q4_CUDA_TRY(cudaGetLastError());
        p.rope = reinterpret_cast<const float*>(rope);
    }
    FTRY(fused_alloc(f, (void**)&p.cand_val, sizeof(float) * sms));
    FTRY(fused_alloc(f, (void**)&p.cand_idx, sizeof(int) * sms));
    FTRY(fused_alloc(f, (void**)&p.bar_counter, sizeof(unsigned long long)));
    FTRY(fused_alloc(f, (void**)&p.status, (4 + 4 * 256) * sizeof(int)));

    std::vector<FPhase> ph;
    int max_K = c.dim, max_part = 0, nbar = 0;
    bool too_many_units = false;
    int x_writer = 0;  // index of the phase that last wrote the residual stream x
    const uint32_t* const kXbuf0 = reinterpret_cast<const uint32_t*>(1);  // markers for "the residual stream, buffer 0 / 1"
    const uint32_t* const kXbuf1 = reinterpret_cast<const uint32_t*>(2);
    auto gemv_phase = [&](int K, const uint32_t* xin, int in_phase, const __half* norm_w, int epi) {
        FPhase a;
        memset(&a, 0, sizeof(a));
        a.type = PH_GEMV;
        a.K = K;
        a.G = q4_groups(K);
        a.nkt = q4_div_up(a.G, kSlotGroups);
        a.xin = xin;
        a.xbuf_in = -1;
        if (xin == kXbuf0 || xin == kXbuf1) { a.xbuf_in = xin == kXbuf1; a.xin = nullptr; }
        a.in_phase = in_phase;
        a.norm_w = norm_w;
        a.epi = epi;
        a.tpu = 1;
        return a;
    };
    auto finish = [&](FPhase& a) {
        const int max_units = q4_div_up(a.nunits, sms);
        if (max_units > kMaxUnitsPerCta) too_many_units = true;
        if (a.nunits < sms) a.barrier_after = 1;   // some CTAs have no unit: keep them in step (see "tagged activations")
        max_part = std::max(max_part, max_units * a.tpu * a.nkt * 8);
        max_K = std::max(max_K, a.K);
        ph.push_back(a);
        if (a.barrier_after) nbar++;
        return (int)ph.size() - 1;
    };
    {
        FPhase a;
        memset(&a, 0, sizeof(a));
        a.type = PH_EMBED;  // writes x tagged; no barrier
        ph.push_back(a);
        x_writer = 0;
    }
    for (int l = 0; l < c.n_layers; l++) {
        const DevLayer& L = m->layers[l];
        const long long loff = (long long)l * c.seq_len * m->kv_n;
        const uint8_t *sq, *sk, *sv, *so, *sg, *su, *sd;
        FTRY(make_stream(f, L.q, &sq)); FTRY(make_stream(f, L.k, &sk)); FTRY(make_stream(f, L.v, &sv)); FTRY(make_stream(f, L.o, &so));
        FTRY(make_stream(f, L.gate, &sg)); FTRY(make_stream(f, L.up, &su)); FTRY(make_stream(f, L.down, &sd));
        int qkv_phase;
        {   // QKV (+ attention RMSNorm): q, k, v -> tagged staging vectors; v also straight into its cache row
            FPhase a = gemv_phase(c.dim, kXbuf1, x_writer, (const __half*)L.rms_att, EPI_STORE);
            a.nmat = 3;
            a.m[0] = FMat{sq, p.q, nullptr, m->q_n, 0};
            a.m[1] = FMat{sk, p.knew, nullptr, m->kv_n, m->q_n / 8};
            a.m[2] = FMat{sv, p.vnew, p.vc, m->kv_n, m->q_n / 8 + m->kv_n / 8};
            a.nunits = m->q_n / 8 + 2 * (m->kv_n / 8);
            a.loff = loff;
            qkv_phase = finish(a);
        }
        {   // attention: waits on the tags of q / knew / vnew and writes tagged per-split partials (no grid barrier)
            FPhase a;
            memset(&a, 0, sizeof(a));
            a.type = PH_ATTN;
            a.loff = loff;
            a.layer = l;
            a.in_phase = qkv_phase;
            ph.push_back(a);
        }
        {   // O projection + residual: polls the attention partials (tagged by the attention phase)
            FPhase a = gemv_phase(m->o_kc, nullptr, (int)ph.size() - 1, nullptr, EPI_RESIDUAL);
            a.attn_in = 1;
            a.nmat = 1;
            a.xbuf_out = 0;
            a.m[0] = FMat{so, nullptr, nullptr, c.dim, 0};
            a.nunits = c.dim / 8;
            x_writer = finish(a);
        }
        int silu_phase;
        {   // gate/up + SiLU (+ ffn RMSNorm): unit = gate tile + the same up tile
            FPhase a = gemv_phase(c.dim, kXbuf0, x_writer, (const __half*)L.rms_ffn, EPI_SILU);
            a.nmat = 2;
            a.m[0] = FMat{sg, p.hb, nullptr, m->h_kc, 0};
            a.m[1] = FMat{su, p.hb, nullptr, m->h_kc, 0};
            a.nunits = m->h_kc / 8;
            a.tpu = 2;
            silu_phase = finish(a);
        }
        {   // down projection + residual
            FPhase a = gemv_phase(m->h_kc, p.hb, silu_phase, nullptr, EPI_RESIDUAL);
            a.nmat = 1;
            a.xbuf_out = 1;
            a.m[0] = FMat{sd, nullptr, nullptr, c.dim, 0};
            a.nunits = c.dim / 8;
            x_writer = finish(a);
        }
    }
    {
        FPhase a;
        memset(&a, 0, sizeof(a));
        a.type = PH_CLS;
        a.K = c.dim;
        a.nkt = q4_div_up(c.dim, kClsChunk);
        a.xbuf_in = 1;
        a.in_phase = x_writer;
        a.norm_w = (const __half*)m->rms_final;
        a.nunits = m->v_n / 2;  // row pairs
        a.barrier_after = 1;
        max_part = std::max(max_part, q4_div_up(a.nunits, sms) * 2 * a.nkt);
        ph.push_back(a);
        nbar++;
        FPhase b;
        memset(&b, 0, sizeof(b));
        b.type = PH_ARGMAX;
        ph.push_back(b);
    }
    {
        const __half* nw = nullptr;
        for (int i = (int)ph.size() - 1; i >= 0; i--) {
            ph[i].next_norm_w = nw;
            ph[i].next_norm_n = c.dim;
            if (ph[i].norm_w) nw = ph[i].norm_w;
        }
    }
    if (too_many_units) { f->unsupported = true; return Q4_ERR_UNSUPPORTED_SIZE; }
    Q4_CUDA_TRY(cudaDeviceSynchronize());  // repacks done
    f->nphases = (int)ph.size();
    FTRY(fused_alloc(f, (void**)&f->d_phases, sizeof(FPhase) * ph.size()));
    Q4_CUDA_TRY(cudaMemcpy(f->d_phases, ph.data(), sizeof(FPhase) * ph.size(), cudaMemcpyHostToDevice));
    p.phases = f->d_phases;
    p.nphases = f->nphases;
    f->barriers_per_launch = nbar;
    {   // per-CTA copy lists
        long long max_slots = 0;
        for (const FPhase& a : ph) {
            if (a.type == PH_GEMV) max_slots += ((long long)q4_div_up(a.nunits, sms) * a.tpu * a.nkt + 1) / 2 + 1;
            if (a.type == PH_CLS) max_slots += ((long long)q4_div_up(a.nunits, sms) * 2 * a.nkt + 1) / 2 + 1;
        }
        p.desc_stride = (int)max_slots + 8;
        CopyDesc* d = nullptr;
        int* dc = nullptr;
        FTRY(fused_alloc(f, (void**)&d, sizeof(CopyDesc) * (size_t)p.desc_stride * sms));
        FTRY(fused_alloc(f, (void**)&dc, sizeof(int) * sms));
        build_desc_kernel<<<sms, 1>>>(p, d, dc, sms);
        Q4_CUDA_TRY(cudaGetLastError());
        std::vector<int> counts(sms);
        Q4_CUDA_TRY(cudaMemcpy(counts.data(), dc, sizeof(int) * sms, cudaMemcpyDeviceToHost));
        for (int cnt : counts)
            if (cnt < 0) { f->unsupported = true; return Q4_ERR_UNSUPPORTED_SIZE; }
        p.desc = d;
        p.desc_count = dc;
    }

    // shared memory: ring | xq (or attention / classifier scratch) | x scales + sums | partial sums
    const int max_G = q4_groups(max_K), max_kt = q4_div_up(max_G, kSlotGroups);
    int xq_bytes = max_kt * 2 * 4 * 32 * 16;                                  // quantised activations
    xq_bytes = std::max(xq_bytes, (int)((2 * kAG + kAG * 128) * sizeof(float)));  // attention scratch
    xq_bytes = std::max(xq_bytes, 2 * c.dim);                                 // classifier x
    p.xq_bytes = (int)align_up(xq_bytes, 128);
    const int meta_bytes = 32 * 16 * 4 * 2;   // 16 k-tiles x 32 lanes, scale + sum
    if (max_kt > 16) { f->unsupported = true; return Q4_ERR_UNSUPPORTED_SIZE; }
    p.part_floats = std::max(max_part, 64);
    // the ring gets whatever shared memory the activation buffers leave (227 KB per CTA, 1 KB kept for static data)
    const size_t other = (size_t)p.xq_bytes + meta_bytes + sizeof(float) * p.part_floats;
    const size_t budget = 225 * 1024;   // + about 1.3 KB of static shared memory = 227 KB per CTA
    int n_entries = other < budget ? (int)((budget - other) / kEntryBytes) : 0;
    n_entries = std::min(n_entries, kMaxEntries);
    if (n_entries < kMinEntries) { f->unsupported = true; return Q4_ERR_UNSUPPORTED_SIZE; }
#ifdef Q4_TEST_BUILD
    if (g_test_entries > 0) n_entries = std::max(kMinEntries, std::min(n_entries, g_test_entries));
#endif
    p.n_entries = n_entries;
    p.meta_off = n_entries * kEntryBytes + p.xq_bytes;
    p.part_off = p.meta_off + meta_bytes;
    f->smem_bytes = (size_t)p.part_off + sizeof(float) * p.part_floats;
    Q4_CUDA_TRY(cudaFuncSetAttribute(fused_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)f->smem_bytes));
    int per_sm = 0;
    Q4_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_token_kernel, kThreads, f->smem_bytes));
    if (per_sm < 1) {
        fprintf(stderr, "q4 fused path: kernel does not fit one SM (%zu B shared memory, %d threads)\n", f->smem_bytes, kThreads);
        f->unsupported = true;
        return Q4_ERR_UNSUPPORTED_SIZE;
    }
#undef FTRY
    return Q4_OK;
}

int q4_fused_forward(q4_model* m, cudaStream_t s, int gen_token, int no_handoff) {
    q4_fused* f = m->fused;
    if (!f || f->unsupported) return Q4_ERR_UNSUPPORTED_SIZE;
    if (!f->armed) return Q4_ERR_CUDA;   // the last re-arm did not complete
    FParams p = f->params;
    p.write_token = gen_token;
    p.no_handoff = no_handoff;
    p.trace = f->trace;
    p.slot_trace = f->slot_trace;
    p.debug = 0;
    p.split_len = kSplitLen;
    p.wait_ns = f->wait_ns;
#ifdef Q4_TEST_BUILD
    p.debug = g_test_debug & 31;
    if (g_test_split_len > 0) p.split_len = g_test_split_len;
#endif
    p.bar_base = f->launches * (unsigned long long)f->barriers_per_launch;
    p.tag_base = (unsigned)((f->launches * (unsigned long long)f->nphases) & 0xFFFFu);
    p.launch_parity = (unsigned)(f->launches & 1);
    f->launches++;
    void* args[] = {&p};
    Q4_CUDA_TRY(cudaLaunchCooperativeKernel((void*)fused_token_kernel, dim3(f->grid), dim3(kThreads), args, f->smem_bytes, s));
    return Q4_OK;
}

#ifdef Q4_TEST_BUILD
// Test build only: the fused path's W4 dot product (activation staging to block fixed point + gemv_slot) on a caller's
// activation vector, outside the token kernel, so that tests can feed it vectors the model never produces on its own
// (outliers, empty groups, subnormals, the largest fp16 values). One CTA per 8-column tile; plain loads, not tuned.
namespace {
__global__ void __launch_bounds__(kCT) test_gemv_kernel(const uint8_t* blocks, const __half* x, __half* y, int K, int G, int nkt) {
    extern __shared__ __align__(128) uint8_t tsm[];
    const int ctid = threadIdx.x, cw = ctid >> 5, lane = ctid & 31, rt = blockIdx.x;
    uint4* xq = reinterpret_cast<uint4*>(tsm);
    float* xs_scale = reinterpret_cast<float*>(tsm + (size_t)nkt * 2 * 4 * 32 * 16);
    int* xs_sum = reinterpret_cast<int*>(xs_scale) + 32 * 16;
    float* part = reinterpret_cast<float*>(xs_sum + 32 * 16);
    uint8_t* slots = reinterpret_cast<uint8_t*>(part + 16 * 8);
    const int nwords = G * 16;
    for (int w0 = 0; w0 < nwords; w0 += kCT) {   // every thread takes part in every round: the shuffles need whole warps
        const int wd = w0 + ctid;
        uint4 hv = make_uint4(0, 0, 0, 0);
        if (wd < nwords) {
            __half* h = reinterpret_cast<__half*>(&hv);
            for (int j = 0; j < 8; j++) h[j] = wd * 8 + j < K ? x[wd * 8 + j] : __float2half(0.f);
        }
        quant_word(hv, wd, nwords, xq, xs_scale, xs_sum);
    }
    __syncthreads();
    for (int kt = cw; kt < nkt; kt += kCW) {
        const int ng = min(kSlotGroups, G - kt * kSlotGroups);
        const uint4* src = reinterpret_cast<const uint4*>(blocks + ((size_t)rt * G + (size_t)kt * kSlotGroups) * kUnitBytes);
        uint4* dst = reinterpret_cast<uint4*>(slots + (size_t)cw * kSlotBytes);
        for (int i = lane; i < ng * kUnitBytes / 16; i += 32) dst[i] = src[i];
        __syncwarp();
        gemv_slot(reinterpret_cast<const uint8_t*>(dst), ng, kt, xq, xs_scale, xs_sum, part + kt * 8, lane);
        __syncwarp();
    }
    __syncthreads();
    if (ctid < 8) {
        float sum = 0.f;
        for (int kt = 0; kt < nkt; kt++) sum += part[kt * 8 + ctid];
        y[rt * 8 + ctid] = __float2half(sum);
    }
}
}  // namespace

extern "C" int q4_test_fused_gemv(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* w, int K, int N) {
    if (!y || !x || !w || K <= 0 || N <= 0 || (N & 7) || (K & 7)) return Q4_ERR_INVALID;
    const int G = q4_groups(K), nkt = q4_div_up(G, kSlotGroups);
    if (nkt > 16) return Q4_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t* blocks = nullptr;
    Q4_CUDA_TRY(cudaMalloc((void**)&blocks, stream_bytes(K, N)));
    repack_kernel<<<dim3(G, N / 8), 64, 0, s>>>(blocks, w->weight, w->zeros, (const __half*)w->scales, K, N, q4_pw(K), q4_pz(K), G);
    const size_t smem = (size_t)nkt * 2 * 4 * 32 * 16 + 32 * 16 * 4 * 2 + 16 * 8 * 4 + (size_t)kCW * kSlotBytes;
    cudaError_t e = cudaFuncSetAttribute(test_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) {
        test_gemv_kernel<<<N / 8, kCT, smem, s>>>(blocks, (const __half*)x, (__half*)y, K, G, nkt);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    cudaFree(blocks);
    Q4_CUDA_TRY(e);
    return Q4_OK;
}
// Test build only: arms (first call) and reads back (later calls) the per-slot stamps of CTA 0; returns the phase count.
extern "C" int q4_test_model_slot_trace(q4_model* m, unsigned long long* out) {
    if (!m) return Q4_ERR_INVALID;
    if (int e = q4_fused_prepare(m)) return e;
    q4_fused* f = m->fused;
    const size_t n = (size_t)f->nphases * kCW * kSlotTraceSlots * 4;
    if (!f->slot_trace) {
        if (int e = fused_alloc(f, (void**)&f->slot_trace, n * sizeof(unsigned long long))) return e;
        Q4_CUDA_TRY(cudaMemset(f->slot_trace, 0, n * sizeof(unsigned long long)));
    }
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    if (out) Q4_CUDA_TRY(cudaMemcpy(out, f->slot_trace, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return f->nphases;
}
#endif  // Q4_TEST_BUILD

// Profiling hook: arms per-phase timestamps (CTA 0 and the last CTA) for the following fused launches and, when
// `out` is given, copies the last launch's stamps out. Layout [2][nphases][4] of nanoseconds; also returns the
// phase types so that the caller can group them.
extern "C" int q4_model_trace(q4_model* m, unsigned long long* out, int* phase_types, int max_phases) {
    if (!m) return Q4_ERR_INVALID;
    if (int e = q4_fused_prepare(m)) return e;
    q4_fused* f = m->fused;
    const size_t n = (size_t)2 * f->nphases * kTraceCols;
    if (!f->trace) {
        if (int e = fused_alloc(f, (void**)&f->trace, n * sizeof(unsigned long long))) return e;
        Q4_CUDA_TRY(cudaMemset(f->trace, 0, n * sizeof(unsigned long long)));
    }
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    if (out && phase_types && max_phases >= f->nphases) {
        Q4_CUDA_TRY(cudaMemcpy(out, f->trace, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        std::vector<FPhase> ph(f->nphases);
        Q4_CUDA_TRY(cudaMemcpy(ph.data(), f->d_phases, sizeof(FPhase) * f->nphases, cudaMemcpyDeviceToHost));
        for (int i = 0; i < f->nphases; i++) phase_types[i] = ph[i].type * 16 + (ph[i].type == PH_GEMV ? ph[i].epi * 4 + (ph[i].norm_w ? 1 : 0) : 0);
    }
    return f->nphases;
}
