// Batched / prefill W4 g128 dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only:
//   Y[M][N] = X[M][K] * deq(W)[K][N],  deq(W)(k, n) = (q(n, k) - z(n, k / 128)) * s(n, k / 128)
// fp16 in, fp32 accumulation in tensor memory, fp16 out. The reference has no batched path: it pushes a prompt through
// the batch-1 GEMV token by token (llama2_q4.cu:710-735, mat_vec_kernel_int4 gpu_kernels.h:179-248); M rows here are M
// applications of that GEMV, and that is what the tests compare against.
//
// Swap-AB: the weights fill the 128-row M side of the MMA (tile = 128 output features), the batch is the MMA's N side
// (16, 64 or 256 rows of X per tile), so small batches still use whole instructions: D[128 x MT] += A[128 x 16] * B[MT x 16]^T.
//
// One CTA per SM, persistent over work units (feature tile, batch tile, K split), four roles:
//   warp 0      weight producer: TMA (cp.async.bulk.tensor.2d, no multicast, this GPU's memory only) of packed weight chunks
//               (128 features x 256 inputs = 128 B per row, 128-byte swizzle) into a staging ring
//   warp 14     X producer: TMA of X tiles (MT x 64, 128-byte swizzle) straight into the (deep) B operand ring
//   warps 2-9   converters: a warp takes every eighth 64-input block, reads its nibbles from the staging ring (conflict free
//               thanks to the swizzle), dequantises them to fp16 in registers (LOP3 magic-number unpack, one exact
//               subtract, one rounding multiply) and stores them into its own A operand stage in the K-major
//               128-byte-swizzled layout the MMA descriptors describe
//   warp 1      MMA: one elected thread issues tcgen05.mma.cta_group::1.kind::f16 (4 per 64-input stage) into a TMEM
//               accumulator and tcgen05.commit's the stage back to the producer / converters
//   warps 10-13 epilogue: tcgen05.ld the accumulator (lane = feature, column = batch row), convert, store
// K is split over work units when there are fewer feature tiles than SMs; the partial sums go through an fp32 workspace
// and the unit that arrives last adds them in split order (deterministic) and writes Y.
//
// Every wait is bounded by the global timer; on expiry the kernel records Q4_ERR_TIMEOUT in the workspace's status word,
// lets all later waits fall through, waits (bounded) for its own copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include <stdio.h>

#include <mutex>

#include "q4_common.cuh"

namespace {

constexpr int kBN = 128;        // output features per tile = rows of the MMA
constexpr int kBK = 64;         // inputs per pipeline stage (one 128-byte swizzle row of fp16)
constexpr int kChunkK = 256;    // inputs per packed-weight copy: 32 words = 128 B per feature row
constexpr int kKbPerChunk = kChunkK / kBK;
constexpr int kConvWarps = 8, kEpiWarps = 4;
constexpr int kFirstConvWarp = 2, kFirstEpiWarp = kFirstConvWarp + kConvWarps;   // epilogue warps 10..13: warp % 4 covers the four TMEM lane quarters
constexpr int kXWarp = kFirstEpiWarp + kEpiWarps;                // 14: X-tile producer
constexpr int kGemmThreads = (kXWarp + 1) * 32;                  // 480
constexpr int kAStageBytes = kBN * kBK * 2;                      // 16 KB
constexpr int kPStageBytes = kBN * (kChunkK / 8) * 4;            // 16 KB
constexpr unsigned long long kGemmWaitNs = 300ULL * 1000 * 1000;   // limit of every device-side wait
constexpr int kMaxStages = 16;

template <int MT> struct GemmCfg {
    // Converter warps = A operand stages (each warp owns one 16 KB stage). What is left of the 227 KB goes to the two rings
    // that hide memory latency: X tiles (MT x 128 B each, from L2, about a microsecond) and packed-weight chunks (16 KB
    // each, from HBM, about two microseconds); the converters hold up to kConverters blocks more in registers. The staging
    // ring has an even length, so that a slot always serves the same four converter warps.
    //              A stages     X ring          weight staging
    //   MT = 16    8 (128 KB)   16 (32 KB)      4 (64 KB)
    //   MT = 64    4 (64 KB)     8 (64 KB)      6 (96 KB)
    //   MT = 256   4 (64 KB)     4 (128 KB)     2 (32 KB)    (bound by the tensor pipe, not by the conversion)
    static constexpr int kConverters = MT <= 16 ? 8 : 4;
    static constexpr int kBStages = MT >= 256 ? 4 : MT >= 64 ? 8 : 16;
    static constexpr int kPStages = MT >= 256 ? 2 : MT >= 64 ? 6 : 4;
    static constexpr int kBStageBytes = MT * kBK * 2;
    static constexpr int kTmemCols = MT < 32 ? 32 : MT;                    // power of two >= 32
    static constexpr size_t kSmemBytes = (size_t)kConverters * kAStageBytes + (size_t)kBStages * kBStageBytes + (size_t)kPStages * kPStageBytes + 1024;
};

struct GemmParams {
    const uint32_t* zeros;
    const __half* scales;
    __half* y;
    const __half* residual;   // optional [M][N]: y = product + residual * residual_scale, rounded once (may alias y)
    float residual_scale;
    float* partials;     // [feature tile][batch tile][split][MT][128] fp32, used when splits > 1
    int* counters;       // [feature tile][batch tile]
    int* status;         // [0] error code, [1] where
    int M, K, N, G, PZ;
    int n_tiles, m_tiles, splits, n_chunks, total_units;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long gtimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mb_init(uint64_t* b, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(b)), "r"(count)); }
__device__ __forceinline__ void mb_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mb_arrive(uint64_t* b) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(b)) : "memory"); }
__device__ __forceinline__ bool mb_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(smem_addr(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit is hit (the error is recorded) or an error is already on record.
__device__ __forceinline__ bool mb_wait(uint64_t* b, uint32_t parity, int* status, int where) {
    unsigned long long t0 = 0;
    for (unsigned i = 0;; i++) {
        if (mb_try(b, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*(volatile int*)status != 0) return false;
            const unsigned long long now = gtimer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kGemmWaitNs) break;
        }
    }
    if (atomicCAS(status, 0, Q4_ERR_TIMEOUT) == 0) status[1] = where;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_addr(dst)),
                 "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                   "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr));
    // the registers are listed as operands of the wait, so that no use of them can be scheduled ahead of it
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]), "+r"(v[10]),
                   "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                 :
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile [rows][64 halfs] stored with the 128-byte swizzle: rows of
// 128 B, groups of 8 rows 1024 B apart (stride byte offset), leading byte offset unused (1), descriptor version 1,
// layout type 2 (SWIZZLE_128B). The tile base is 1024-byte aligned (base offset 0). Advancing 16 inputs along K inside
// the swizzled row = + 32 bytes on the start address.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ULL << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ULL << 46) | (2ULL << 61);
}
// Instruction descriptor, kind::f16: D fp32 (bits 4-5 = 1), A and B fp16 (0), both K-major (0), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kBN >> 4) << 24); }

// One packed word (8 nibbles) -> 8 fp16 weights in input order. INTERLEAVED: the word's nibbles hold inputs 0,2,4,6,1,3,5,7
// (prepared by q4_gemm_interleave_weights), so the two mask patterns yield the pairs (0,1) (2,3) (4,5) (6,7) directly; the file
// layout yields (0,4) (1,5) (2,6) (3,7) and needs four byte permutes. (q - z) is exact in fp16 (|q - z| <= 15), the
// multiplication by the fp16 scale rounds once.
template <bool INTERLEAVED>
__device__ __forceinline__ uint4 dequant8(uint32_t w, uint32_t zlo, uint32_t zhi, __half2 s2) {
    const __half2 sixteenth = u2h2(0x2C002C00u);
    const __half2 a = __hmul2(__hsub2(u2h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), u2h2(zlo)), s2);
    const __half2 b = __hmul2(__hfma2(u2h2(lop3_and_or(w, 0x00F000F0u, 0x64006400u)), sixteenth, u2h2(zhi)), s2);
    w >>= 8;
    const __half2 c = __hmul2(__hsub2(u2h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), u2h2(zlo)), s2);
    const __half2 d = __hmul2(__hfma2(u2h2(lop3_and_or(w, 0x00F000F0u, 0x64006400u)), sixteenth, u2h2(zhi)), s2);
    if (INTERLEAVED) return make_uint4(h22u(a), h22u(b), h22u(c), h22u(d));
    // a = (0,4) b = (1,5) c = (2,6) d = (3,7)
    return make_uint4(prmt(h22u(a), h22u(b), 0x5410), prmt(h22u(c), h22u(d), 0x5410), prmt(h22u(a), h22u(b), 0x7632), prmt(h22u(c), h22u(d), 0x7632));
}

struct UnitInfo { int tile, mt, split, c0, c1; };
__device__ __forceinline__ UnitInfo unit_info(const GemmParams& p, int u) {
    UnitInfo i;
    i.split = u % p.splits;
    const int t = u / p.splits;
    i.mt = t % p.m_tiles;
    i.tile = t / p.m_tiles;
    i.c0 = (int)((long long)p.n_chunks * i.split / p.splits);
    i.c1 = (int)((long long)p.n_chunks * (i.split + 1) / p.splits);
    return i;
}

// Every chunk is processed as four 64-input blocks, also the last chunk of a K that is not a multiple of 256: TMA fills
// what lies outside the tensors with zeros on both operands, so the extra blocks add nothing. That keeps the pipeline
// regular: block q of a CTA (counted over all its units) is converted by converter warp q % NC into operand stage
// q % NC, which that warp alone ever fills - every barrier is then waited on by one party, phase after phase without
// gaps (a parity wait cannot tell phase k from phase k + 2).
template <int MT, bool INTERLEAVED>
__global__ void __launch_bounds__(kGemmThreads, 1)
q4_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    using Cfg = GemmCfg<MT>;
    constexpr int NC = Cfg::kConverters, NP = Cfg::kPStages, NB = Cfg::kBStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = smem;
    uint8_t* sB = sA + (size_t)NC * kAStageBytes;
    uint8_t* sP = sB + (size_t)NB * Cfg::kBStageBytes;
    __shared__ uint64_t full_p[kMaxStages], empty_p[kMaxStages], full_a[kMaxStages], empty_a[kMaxStages], full_b[kMaxStages], empty_b[kMaxStages], tmem_full,
        tmem_empty;
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kMaxStages; s++) {
            mb_init(&full_p[s], 1); mb_init(&empty_p[s], kKbPerChunk);   // a chunk's four blocks go to four converter warps
            mb_init(&full_a[s], 1); mb_init(&empty_a[s], 1); mb_init(&full_b[s], 1); mb_init(&empty_b[s], 1);
        }
        mb_init(&tmem_full, 1);
        mb_init(&tmem_empty, kEpiWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // tensor memory for the accumulator: the whole warp allocates, the address lands in shared memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem_base)), "r"(Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&s_tmem_base;
    // everything above overlaps the tail of the previous kernel on the stream (programmatic dependent launch); from here
    // on this kernel reads what that kernel wrote
    griddep_wait();
    griddep_launch_dependents();

    if (warp == 0) {
        // ===================== weight producer =====================
        // keeps the packed-weight staging ring full: it waits only for free staging slots, so it runs ahead of the math and
        // across unit boundaries
        if (lane == 0) {
            unsigned pit = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
                const UnitInfo ui = unit_info(p, u);
                for (int c = ui.c0; c < ui.c1; c++, pit++) {
                    const int ps = pit % NP;
                    if (!mb_wait(&empty_p[ps], ((pit / NP) & 1) ^ 1, p.status, 0x100)) { ok = false; break; }
                    mb_expect_tx(&full_p[ps], kPStageBytes);
                    tma_load_2d(sP + (size_t)ps * kPStageBytes, &map_w, c * (kChunkK / 8), ui.tile * kBN, &full_p[ps]);
                }
            }
            if (!ok) {   // after an error the newest copy of every ring position may still be in flight: give each up to 50 ms
                for (unsigned i = pit > (unsigned)NP ? pit - NP : 0; i < pit; i++) {
                    const unsigned long long t0 = gtimer();
                    while (!mb_try(&full_p[i % NP], (i / NP) & 1) && gtimer() - t0 < 50ULL * 1000 * 1000) {}
                }
            }
        }
    } else if (warp == kXWarp) {
        // ===================== X producer =====================
        // loads the X tile of every 64-input block as soon as the MMA has released that slot of the (deep) B ring
        if (lane == 0) {
            unsigned q = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
                const UnitInfo ui = unit_info(p, u);
                for (int kb = ui.c0 * kKbPerChunk; kb < ui.c1 * kKbPerChunk; kb++, q++) {
                    const int s = q % NB;
                    if (!mb_wait(&empty_b[s], ((q / NB) & 1) ^ 1, p.status, 0x200)) { ok = false; break; }
                    mb_expect_tx(&full_b[s], Cfg::kBStageBytes);
                    tma_load_2d(sB + (size_t)s * Cfg::kBStageBytes, &map_x, kb * kBK, ui.mt * MT, &full_b[s]);
                }
            }
            if (!ok) {
                for (unsigned i = q > (unsigned)NB ? q - NB : 0; i < q; i++) {
                    const unsigned long long t0 = gtimer();
                    while (!mb_try(&full_b[i % NB], (i / NB) & 1) && gtimer() - t0 < 50ULL * 1000 * 1000) {}
                }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        // one thread does it all: the instructions are asynchronous, and at small batch tiles their issue rate is what
        // bounds the kernel, so nothing else shares this warp's issue slots
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(MT);
            const uint64_t adesc0 = umma_desc(smem_addr(sA)), bdesc0 = umma_desc(smem_addr(sB));
            unsigned q = 0, uit = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x, uit++) {
                const UnitInfo ui = unit_info(p, u);
                if (!mb_wait(&tmem_empty, (uit & 1) ^ 1, p.status, 0x300)) { ok = false; break; }   // the epilogue has drained the accumulator
                const int nkb = (ui.c1 - ui.c0) * kKbPerChunk;
                for (int i = 0; i < nkb; i++, q++) {
                    const int s = q % NC, sb = q % NB;
                    if (!mb_wait(&full_a[s], (q / NC) & 1, p.status, 0x400) || !mb_wait(&full_b[sb], (q / NB) & 1, p.status, 0x500)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t ad = adesc0 + (uint64_t)((s * kAStageBytes) >> 4), bd = bdesc0 + (uint64_t)((sb * Cfg::kBStageBytes) >> 4);
#pragma unroll
                    for (int k16 = 0; k16 < kBK / 16; k16++) tc_mma_f16(tmem_base, ad + 2 * k16, bd + 2 * k16, idesc, (i == 0 && k16 == 0) ? 0u : 1u);
                    tc_commit(&empty_a[s]);    // both arrive when these MMAs have read their operands
                    tc_commit(&empty_b[sb]);
                }
                tc_commit(&tmem_full);
            }
        }
    } else if (warp < kFirstEpiWarp) {
        // ===================== converters =====================
        // Warp w converts blocks q = w, w + NC, ...: a whole 128-feature x 64-input operand stage per block, four feature
        // rows per lane, so that the fixed cost of a hand-over (barrier round trips, store drain) is paid once per 8192
        // weights and NC blocks are in flight at once.
        const int cw = warp - kFirstConvWarp;
        if (cw < NC) {
            const int sw = lane & 7;   // rows lane + 32 i share lane & 7, hence the swizzle term
            bool ok = true;
            unsigned q = 0;            // first block of the current unit
            // zero points and scales of this warp's next block, requested one block of its own ahead
            uint32_t z_next[4] = {0, 0, 0, 0};
            __half s_next[4];
            auto fetch_meta = [&](int tile, int kb) {
                const int g = kb >> 1;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int n = tile * kBN + lane + 32 * i;
                    z_next[i] = 0;
                    s_next[i] = __float2half(0.f);
                    if (n < p.N && g < p.G) {
                        z_next[i] = (__ldg(p.zeros + (size_t)n * p.PZ + (g >> 3)) >> (4 * (g & 7))) & 0xFu;
                        s_next[i] = __ldg(p.scales + (size_t)n * p.G + g);
                    }
                }
            };
            bool have_meta = false;
            for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x) {
                const UnitInfo ui = unit_info(p, u);
                const unsigned nkb = (unsigned)(ui.c1 - ui.c0) * kKbPerChunk;
                // this warp's first block of the unit
                unsigned i = (cw + NC - (q % NC)) % NC;
                if (!have_meta && i < nkb) fetch_meta(ui.tile, ui.c0 * kKbPerChunk + i);
                for (; i < nkb && ok; i += NC) {
                    const unsigned qi = q + i;                      // this block's number: stage qi % NC == cw
                    const int kb = ui.c0 * kKbPerChunk + (int)i;    // 64-input block inside K
                    const unsigned pit = qi / kKbPerChunk;          // chunk number (chunks are four blocks, always)
                    const int kbl = qi % kKbPerChunk, ps = pit % NP;
                    uint32_t zz[4];
                    __half ss[4];
#pragma unroll
                    for (int r4 = 0; r4 < 4; r4++) { zz[r4] = z_next[r4]; ss[r4] = s_next[r4]; }
                    have_meta = false;
                    if (i + NC < nkb) { fetch_meta(ui.tile, kb + NC); have_meta = true; }
                    if (!mb_wait(&full_p[ps], (pit / NP) & 1, p.status, 0x600)) { ok = false; break; }
                    uint4 pk[8];   // rows lane + 32 r4, the block's two 16-byte pieces of each row
#pragma unroll
                    for (int r4 = 0; r4 < 4; r4++)
#pragma unroll
                        for (int h = 0; h < 2; h++)
                            pk[r4 * 2 + h] = *reinterpret_cast<const uint4*>(sP + (size_t)ps * kPStageBytes + (lane + 32 * r4) * 128 + (((kbl * 2 + h) ^ sw) << 4));
                    __syncwarp();
                    if (lane == 0) mb_arrive(&empty_p[ps]);   // the nibbles are in registers: one of the chunk's four releases
                    if (!mb_wait(&empty_a[cw], ((qi / NC) & 1) ^ 1, p.status, 0x700)) { ok = false; break; }
                    uint8_t* stage = sA + (size_t)cw * kAStageBytes;
#pragma unroll
                    for (int r4 = 0; r4 < 4; r4++) {
                        const int r = lane + 32 * r4;
                        uint32_t zlo, zhi;
                        zero_consts(zz[r4], zlo, zhi);
                        const __half2 s2 = __half2half2(ss[r4]);
                        uint8_t* arow = stage + (r >> 3) * 1024 + sw * 128;
                        const uint32_t words[8] = {pk[r4 * 2].x, pk[r4 * 2].y, pk[r4 * 2].z, pk[r4 * 2].w, pk[r4 * 2 + 1].x, pk[r4 * 2 + 1].y, pk[r4 * 2 + 1].z, pk[r4 * 2 + 1].w};
#pragma unroll
                        for (int j = 0; j < 8; j++) *reinterpret_cast<uint4*>(arow + ((j ^ sw) << 4)) = dequant8<INTERLEAVED>(words[j], zlo, zhi, s2);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores before the MMA's async-proxy reads
                    __syncwarp();
                    if (lane == 0) mb_arrive(&full_a[cw]);
                }
                q += nkb;
            }
        }
    } else if (warp < kFirstEpiWarp + kEpiWarps) {
        // ===================== epilogue =====================
        const int qtr = warp & 3;              // the TMEM lane quarter this warp may read
        const int r = qtr * 32 + lane;
        const int etid = (warp - kFirstEpiWarp) * 32 + lane;
        unsigned uit = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < p.total_units && ok; u += gridDim.x, uit++) {
            const UnitInfo ui = unit_info(p, u);
            const int n = ui.tile * kBN + r;
            // The residual may be y itself, so a residual load cannot be moved across a store of y by the compiler: the
            // loads of a 16-row chunk are issued together and one chunk ahead of the stores, the first chunk's while the MMAs
            // of the unit still run.
            float res_next[16];
            auto load_res = [&](int c0, float (&res)[16]) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int m = ui.mt * MT + c0 + j;
                    res[j] = (n < p.N && m < p.M) ? __half2float(p.residual[(size_t)m * p.N + n]) : 0.f;
                }
            };
            const bool add_res = p.residual != nullptr && p.splits == 1;
            if (add_res) load_res(0, res_next);
            if (!mb_wait(&tmem_full, uit & 1, p.status, 0x800)) { ok = false; break; }
            tc_fence_after();
            float* part = p.partials + (((size_t)(ui.tile * p.m_tiles + ui.mt) * p.splits + ui.split) * MT) * kBN;
#pragma unroll 1
            for (int c0 = 0; c0 < MT; c0 += 16) {
                uint32_t v[16];
                float res[16];
                if (add_res) {
#pragma unroll
                    for (int j = 0; j < 16; j++) res[j] = res_next[j];
                    if (c0 + 16 < MT) load_res(c0 + 16, res_next);
                }
                tc_ld16(tmem_base + ((uint32_t)(qtr * 32) << 16) + (uint32_t)c0, v);
                if (p.splits == 1) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int m = ui.mt * MT + c0 + j;
                        if (n < p.N && m < p.M) {
                            float val = __uint_as_float(v[j]);
                            if (add_res) val += res[j] * p.residual_scale;
                            p.y[(size_t)m * p.N + n] = __float2half(val);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) part[(size_t)(c0 + j) * kBN + r] = __uint_as_float(v[j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mb_arrive(&tmem_empty);
            if (p.splits > 1) {
                // the unit that arrives last at the tile's counter adds the partial sums in split order and writes Y
                __threadfence();
                asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * 32) : "memory");
                if (etid == 0) {
                    const int old = atomicAdd(p.counters + ui.tile * p.m_tiles + ui.mt, 1);
                    s_last = old == p.splits - 1;
                    if (s_last) p.counters[ui.tile * p.m_tiles + ui.mt] = 0;   // ready for the next launch
                }
                asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * 32) : "memory");
                if (s_last) {
                    __threadfence();
                    const float* base = p.partials + ((size_t)(ui.tile * p.m_tiles + ui.mt) * p.splits) * MT * kBN + r;
                    const int rows = min(MT, p.M - ui.mt * MT);
                    // eight batch rows at a time, all their loads in flight together (the partial sums come from L2); the
                    // splits are added in split order, so the result does not depend on which unit arrived last
                    for (int c0 = 0; c0 < rows; c0 += 8) {
                        float acc[8];
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[j] = 0.f;
                        float res[8];
#pragma unroll
                        for (int j = 0; j < 8; j++)   // all eight before any store of y (the residual may be y)
                            res[j] = (p.residual && c0 + j < rows && n < p.N) ? __half2float(p.residual[(size_t)(ui.mt * MT + c0 + j) * p.N + n]) : 0.f;
                        for (int s = 0; s < p.splits; s++) {
                            float v[8];
#pragma unroll
                            for (int j = 0; j < 8; j++) v[j] = c0 + j < rows ? __ldcg(base + ((size_t)s * MT + c0 + j) * kBN) : 0.f;
#pragma unroll
                            for (int j = 0; j < 8; j++) acc[j] += v[j];
                        }
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (c0 + j < rows && n < p.N) {
                                const size_t at = (size_t)(ui.mt * MT + c0 + j) * p.N + n;
                                if (p.residual) acc[j] += res[j] * p.residual_scale;
                                p.y[at] = __float2half(acc[j]);
                            }
                    }
                }
                asm volatile("bar.sync 2, %0;" ::"n"(kEpiWarps * 32) : "memory");   // s_last is rewritten by the next unit
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
    }
}

// dst word: nibble i holds input order[i] of the same 8 inputs, order = 0,2,4,6,1,3,5,7
__global__ void interleave_kernel(uint32_t* dst, const uint32_t* src, size_t nwords) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nwords; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t w = src[i];
        const uint32_t even = w & 0x0F0F0F0Fu, odd = (w >> 4) & 0x0F0F0F0Fu;   // bytes: inputs 0,2,4,6 / 1,3,5,7
        // pack the four bytes of each into four consecutive nibbles
        const uint32_t e = (even & 0xFu) | ((even >> 4) & 0xF0u) | ((even >> 8) & 0xF00u) | ((even >> 12) & 0xF000u);
        const uint32_t o = (odd & 0xFu) | ((odd >> 4) & 0xF0u) | ((odd >> 8) & 0xF00u) | ((odd >> 12) & 0xF000u);
        dst[i] = e | (o << 16);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
std::mutex g_encode_mu;
EncodeTiledFn g_encode = nullptr;

int get_encode(EncodeTiledFn* out) {
    std::lock_guard<std::mutex> lk(g_encode_mu);
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        Q4_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return Q4_ERR_CUDA;
        g_encode = (EncodeTiledFn)fn;
    }
    *out = g_encode;
    return Q4_OK;
}

int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner, uint64_t outer, uint64_t row_bytes, uint32_t box_inner,
                uint32_t box_outer) {
    EncodeTiledFn enc;
    if (int e = get_encode(&enc)) return e;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    const CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { fprintf(stderr, "q4 gemm: cuTensorMapEncodeTiled failed (%d)\n", (int)r); return Q4_ERR_CUDA; }
    return Q4_OK;
}

struct GemmPlan { int mt, m_tiles, n_tiles, splits, n_chunks, units; size_t partial_floats; };

// Batch tile (the MMA's N), and how far K is split so that the work units fill the SMs evenly.
GemmPlan make_plan(int M, int K, int N, int sms) {
    GemmPlan g;
    g.mt = M <= 16 ? 16 : M <= 64 ? 64 : 256;
    g.m_tiles = q4_div_up(M, g.mt);
    g.n_tiles = q4_div_up(N, kBN);
    g.n_chunks = q4_div_up(K, kChunkK);
    const int base = g.n_tiles * g.m_tiles;
    int best = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= 16 && s <= g.n_chunks; s++) {
        if (s > 1 && g.n_chunks / s < 2) break;   // at least two chunks (512 inputs) per unit
        const int units = base * s;
        // time of the slowest SM in chunk steps: its units' chunks, plus per unit a fixed cost (pipeline fill, epilogue)
        // and, when K is split, the partial-sum round trip, which grows with the batch tile
        const double per_unit = (double)q4_div_up(g.n_chunks, s) + 1.0 + (s > 1 ? 0.5 + g.mt / 64.0 : 0.0);
        const double cost = q4_div_up(units, sms) * per_unit;
        if (cost < best_cost * 0.97) { best_cost = cost; best = s; }
    }
    g.splits = best;
    g.units = base * best;
    g.partial_floats = best > 1 ? (size_t)g.units * g.mt * kBN : 0;
    return g;
}

int sm_count(int* out) {
    int dev = 0;
    Q4_CUDA_TRY(cudaGetDevice(&dev));
    Q4_CUDA_TRY(cudaDeviceGetAttribute(out, cudaDevAttrMultiProcessorCount, dev));
    return Q4_OK;
}

// Workspace layout, the same for every shape, so that calls of different shapes can share one workspace (the tile counters
// must read zero at the start of every call): status words | tile counters | fp32 partial sums.
constexpr size_t kWsHeader = 256;
constexpr int kWsMaxTiles = 8192;
constexpr size_t kWsPartials = kWsHeader + sizeof(int) * kWsMaxTiles;

template <int MT, bool IL>
int launch_gemm(cudaStream_t s, int grid, const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p) {
    const size_t smem = GemmCfg<MT>::kSmemBytes;
    Q4_CUDA_TRY(cudaFuncSetAttribute(q4_gemm_kernel<MT, IL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    Q4Launch L(dim3(grid), dim3(kGemmThreads), smem, s);   // programmatic dependent launch: the prologue overlaps the previous kernel's tail
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_gemm_kernel<MT, IL>, mw, mx, p));
    return Q4_OK;
}

}  // namespace

extern "C" size_t q4_matmul_q4_batched_workspace_bytes(int M, int K, int N) {
    if (M <= 0 || K <= 0 || N <= 0) return 0;
    int sms = 148;
    sm_count(&sms);
    const GemmPlan g = make_plan(M, K, N, sms);
    return kWsPartials + g.partial_floats * sizeof(float);
}

extern "C" int q4_gemm_interleave_weights(void* stream, uint32_t* dst, const uint32_t* weight, int K, int N) {
    if (!dst || !weight || K <= 0 || N <= 0) return Q4_ERR_INVALID;
    const size_t nwords = (size_t)N * q4_pw(K);
    interleave_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(dst, weight, nwords);
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}

extern "C" int q4_matmul_q4_batched(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* w, const uint32_t* weight_interleaved, int M, int K,
                                    int N, void* workspace, size_t workspace_bytes) {
    return q4_matmul_q4_batched_residual(stream, y, x, w, weight_interleaved, M, K, N, nullptr, 0.f, workspace, workspace_bytes);
}

extern "C" int q4_matmul_q4_batched_residual(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* w, const uint32_t* weight_interleaved, int M,
                                             int K, int N, const uint16_t* residual, float residual_scale, void* workspace, size_t workspace_bytes) {
    if (!y || !x || !w || !workspace || M <= 0 || K <= 0 || N <= 0) return Q4_ERR_INVALID;
    if ((K % 128) || (N % 8)) return Q4_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)x & 15) || ((uintptr_t)w->weight & 15) || ((uintptr_t)weight_interleaved & 15) || ((uintptr_t)workspace & 15)) return Q4_ERR_INVALID;
    if (workspace_bytes < q4_matmul_q4_batched_workspace_bytes(M, K, N)) return Q4_ERR_LIMIT;
    cudaStream_t s = (cudaStream_t)stream;
    int sms = 0;
    if (int e = sm_count(&sms)) return e;
    const GemmPlan g = make_plan(M, K, N, sms);
    GemmParams p;
    p.zeros = w->zeros;
    p.scales = (const __half*)w->scales;
    p.y = (__half*)y;
    p.residual = (const __half*)residual;
    p.residual_scale = residual_scale;
    p.status = (int*)workspace;
    p.counters = (int*)((char*)workspace + kWsHeader);
    p.partials = (float*)((char*)workspace + kWsPartials);
    if (g.n_tiles * g.m_tiles > kWsMaxTiles) return Q4_ERR_UNSUPPORTED_SIZE;
    p.M = M; p.K = K; p.N = N;
    p.G = q4_groups(K);
    p.PZ = q4_pz(K);
    p.n_tiles = g.n_tiles; p.m_tiles = g.m_tiles; p.splits = g.splits; p.n_chunks = g.n_chunks; p.total_units = g.units;
    // (status word and tile counters start at zero: the caller zeroes the workspace once, the kernel leaves the counters at
    // zero; after a recorded time-out the caller zeroes it again)
    CUtensorMap mw, mx;
    const uint32_t* wsrc = weight_interleaved ? weight_interleaved : w->weight;
    if (int e = make_map_2d(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, wsrc, (uint64_t)q4_pw(K), (uint64_t)N, (uint64_t)q4_pw(K) * 4, kChunkK / 8, kBN)) return e;
    if (int e = make_map_2d(&mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2, kBK, (uint32_t)g.mt)) return e;
    const int grid = g.units < sms ? g.units : sms;
    const bool il = weight_interleaved != nullptr;
    if (g.mt == 16) return il ? launch_gemm<16, true>(s, grid, mw, mx, p) : launch_gemm<16, false>(s, grid, mw, mx, p);
    if (g.mt == 64) return il ? launch_gemm<64, true>(s, grid, mw, mx, p) : launch_gemm<64, false>(s, grid, mw, mx, p);
    return il ? launch_gemm<256, true>(s, grid, mw, mx, p) : launch_gemm<256, false>(s, grid, mw, mx, p);
}

extern "C" int q4_matmul_q4_batched_status(void* stream, const void* workspace) {
    if (!workspace) return Q4_ERR_INVALID;
    int st[2] = {0, 0};
    Q4_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    Q4_CUDA_TRY(cudaMemcpy(st, workspace, sizeof(st), cudaMemcpyDeviceToHost));
    if (st[0]) fprintf(stderr, "q4 gemm: a bounded device-side wait ran out (status %d, location 0x%x)\n", st[0], st[1]);
    return st[0];
}

// Measurement hook: q4_matmul_q4_batched over `nmat` distinct weight matrices of one shape, captured as one CUDA graph
// and replayed `reps` times between two events on `stream` (weights from HBM rather than L2, no launch gaps timed).
extern "C" int q4_time_matmul_q4_batched(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* mats, const uint32_t* const* interleaved, int nmat,
                                         int M, int K, int N, void* workspace, size_t workspace_bytes, int reps, double* us_per_launch) {
    if (!mats || nmat < 1 || reps < 1 || !us_per_launch) return Q4_ERR_INVALID;
    cudaStream_t s = (cudaStream_t)stream;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    Q4_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    int e = Q4_OK;
    for (int i = 0; i < nmat && e == Q4_OK; i++)
        e = q4_matmul_q4_batched(s, y, x, &mats[i], interleaved ? interleaved[i] : nullptr, M, K, N, workspace, workspace_bytes);
    cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (e != Q4_OK) { if (graph) cudaGraphDestroy(graph); return e; }
    Q4_CUDA_TRY(ce);
    Q4_CUDA_TRY(cudaGraphInstantiate(&exec, graph, 0));
    cudaEvent_t e0, e1;
    Q4_CUDA_TRY(cudaEventCreate(&e0));
    Q4_CUDA_TRY(cudaEventCreate(&e1));
    for (int r = 0; r < 3; r++) Q4_CUDA_TRY(cudaGraphLaunch(exec, s));
    Q4_CUDA_TRY(cudaEventRecord(e0, s));
    for (int r = 0; r < reps; r++) Q4_CUDA_TRY(cudaGraphLaunch(exec, s));
    Q4_CUDA_TRY(cudaEventRecord(e1, s));
    Q4_CUDA_TRY(cudaEventSynchronize(e1));
    float ms = 0.f;
    Q4_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    *us_per_launch = 1e3 * ms / ((double)reps * nmat);
    return Q4_OK;
}
