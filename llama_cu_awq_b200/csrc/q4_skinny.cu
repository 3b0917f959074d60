// AWQ W4 g128 dequantize-and-multiply for a handful of rows (1 <= M <= 16): the projections of batched decode.
//
// The reference has one sequence per process (RunState, common.h:62-78) and its mat_vec_kernel_int4 family
// (gpu_kernels.h:179-283) reads every weight once per token; with several sequences decoded together the weights are
// still read once per STEP, so the op stays bound by HBM as long as the per-weight work is small. That is what this
// kernel is built for; the tcgen05 GEMM (q4_gemm.cu) takes over from M > 16, where the contraction starts to matter.
//
// Work split: a unit is 16 * MT output features of one launch over the whole K axis; one persistent CTA (12 warps; 8 for
// 9-16 rows) per SM walks the units; warp w takes the w-th share of a unit's 128-input groups, and the warps' partial
// tiles are summed in warp order through shared memory (fixed order: results are bit-reproducible). Inside a warp the product runs on mma.sync m16n8k16 (fp16 in, fp32 out) with
// the weights as the 16-row operand and the batch as the 8-column one. The k index of an MMA is only a summation
// label, so the packed words are used as they lie in the file: thread (g, t) of the warp loads 16 bytes = 32 inputs of
// feature rows g and g + 8 at input offset 32 t of the group, unpacks a word into the half2 pairs (q0,q4) (q1,q5)
// (q2,q6) (q3,q7) with the zero point subtracted exactly (magic-number trick, no int -> float conversion), and feeds
// them as the A fragment; the B fragment is the same eight inputs of batch row g in the same pairing. Per group the
// fp32 tile is scaled by the group's fp16 scale in fp32, as the reference does (gpu_kernels.h:222-228), so weights
// are never rounded to fp16 after scaling.
//
// Epilogues: plain, residual (y = product + residual * scale: matmul(QWeight)'s accum form, gpu_kernels.h:237-238),
// and SiLU (ffn_matvec_silu_kernel, gpu_kernels.h:251-283: the CTA holds 16 gate and the same 16 up features and writes
// silu(gate) * up without rounding gate or up to fp16 first).
#include "q4_common.cuh"

namespace {

struct SkMat {
    const uint32_t* w;
    const uint32_t* z;
    const __half* s;
    __half* y;
    int ldy;     // halfs between rows of y
    int tile0;   // first 16-feature tile of this matrix in the launch
};

struct SkParams {
    const __half* x;   // [M][K]
    int M, K, PW, PZ, G;
    int nmat;
    SkMat m[3];
    int total_tiles;
    const __half* residual;   // [M][ldy of m[0]] or null
    float rscale;
};

__device__ __forceinline__ void mma_f16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One packed word minus the zero point as four half2: (q0,q4) (q1,q5) (q2,q6) (q3,q7), exact.
// (w & 0x000F000F) | 0x6400 is the half 1024 + q; (w & 0x00F000F0) | 0x5400 is the half 64 + q (one unit of q is 16 ulps there).
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t zlo, uint32_t zhi, uint32_t d[4]) {
    d[0] = h22u(__hsub2(u2h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), u2h2(zlo)));
    d[1] = h22u(__hsub2(u2h2(lop3_and_or(w, 0x00F000F0u, 0x54005400u)), u2h2(zhi)));
    w >>= 8;
    d[2] = h22u(__hsub2(u2h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), u2h2(zlo)));
    d[3] = h22u(__hsub2(u2h2(lop3_and_or(w, 0x00F000F0u, 0x54005400u)), u2h2(zhi)));
}

#ifndef SK_WARPS
#define SK_WARPS 12
#endif
#ifndef SK_D1
#define SK_D1 3
#endif
#ifndef SK_D2
#define SK_D2 2
#endif
#ifndef SK_D22
#define SK_D22 3
#endif
// warps of a CTA = K slices of a unit
__host__ __device__ constexpr int warps_of(int MT, int NT) { return NT == 2 ? 8 : SK_WARPS; }   // (16 batch rows need the registers of 8-warp CTAs)

// MT: 16-feature tiles per unit (1 or 2); NT: 8-row batch tiles (1: M <= 8, 2: M <= 16); SILU: tile 0 = gate, tile 1 = up.
// Persistent: one CTA per SM walks units blockIdx.x, blockIdx.x + gridDim.x, ...; a warp's weight loads run D groups ahead
// of its math ACROSS unit boundaries and its x fragments one group ahead (a unit gives a warp only G / kWarps groups - four
// at K = 4096 - so a pipeline that restarted per unit would spend its time on load latency, and one-unit CTAs would
// quantise the work badly over the SMs). Measured on the four 7B ops with 8 rows (us): 8 warps with 4 groups ahead
// 4.4 / 10.4 / 11.9 / 19.9; 12 warps with 2-3 ahead 4.5 / 9.4 / 10.6 / 16.6; 16 warps with 2 ahead 4.8 / 9.6 / 11.6 / 19.2.
template <int MT, int NT, bool SILU>
__global__ void __launch_bounds__(warps_of(MT, NT) * 32, 1) q4_skinny_kernel(const SkParams p) {
    constexpr int kWarps = warps_of(MT, NT);
    extern __shared__ float red_raw[];
    float (*red)[kWarps][MT][NT][4][32] = reinterpret_cast<float (*)[kWarps][MT][NT][4][32]>(red_raw);   // [2]: double buffered by unit parity
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int units = SILU ? p.total_tiles : p.total_tiles / MT;
    const int my_units = blockIdx.x < units ? (units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // this warp's groups of every unit
    const int g_begin = (int)((long long)p.G * warp / kWarps), g_end = (int)((long long)p.G * (warp + 1) / kWarps);
    const int gpw = g_end - g_begin;
    const int total = my_units * gpw;   // (unit, group) steps of this warp, unit-major

    // rows of unit u: tile mt holds features f0 .. f0 + 15 of matrix mi
    auto unit_tile = [&](int u, int mt, int& mi, int& f0) {
        const int unit = blockIdx.x + u * gridDim.x;
        int tile;
        if (SILU) {
            mi = mt;
            tile = unit;
        } else {
            tile = unit * MT + mt;
            mi = 0;
            if (p.nmat > 1 && tile >= p.m[1].tile0) mi = 1;
            if (p.nmat > 2 && tile >= p.m[2].tile0) mi = 2;
            tile -= p.m[mi].tile0;
        }
        f0 = tile * 16;
    };

    // A step's operands per thread: 16 bytes of packed weights, the zeros word and the scale for each of its 2 MT rows.
    constexpr int D = MT == 1 ? SK_D1 : (NT == 1 ? SK_D2 : SK_D22);
    struct Stage {
        uint4 w[MT][2];
        uint32_t zw[MT][2];
        __half sc[MT][2];
    };
    Stage st[D];
    // prefetch cursor: step index, its unit, its group within the warp's slice, and the unit's row pointers (row g of each
    // tile; row g + 8 lies 8 rows further)
    int pf = 0, pf_u = 0, pf_gi = 0;
    const uint4* pw[MT];
    const uint32_t* pz[MT];
    const __half* ps[MT];
    auto set_rows = [&](int u) {
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            int mi, f0;
            unit_tile(u, mt, mi, f0);
            const size_t row = (size_t)f0 + g;
            pw[mt] = reinterpret_cast<const uint4*>(p.m[mi].w + row * p.PW) + t;
            pz[mt] = p.m[mi].z + row * p.PZ;
            ps[mt] = p.m[mi].s + row * p.G;
        }
    };
    auto prefetch = [&](Stage& d) {
        if (pf < total) {
            const int grp = g_begin + pf_gi;
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    d.w[mt][hh] = ldg_stream(pw[mt] + hh * 2 * p.PW + 4 * grp);
                    d.zw[mt][hh] = __ldg(pz[mt] + hh * 8 * p.PZ + (grp >> 3));
                    d.sc[mt][hh] = __ldg(ps[mt] + hh * 8 * p.G + grp);
                }
            pf++;
            if (++pf_gi == gpw) {
                pf_gi = 0;
                pf_u++;
                if (pf < total) set_rows(pf_u);
            }
        }
    };
    if (total > 0) set_rows(0);
#pragma unroll
    for (int d = 0; d < D; d++) prefetch(st[d]);
    griddep_wait();
    griddep_launch_dependents();

    // x: the batch rows' 32 inputs of this thread's quarter of a group, fetched one step ahead
    const __half* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        xok[nt] = g + 8 * nt < p.M;
        xrow[nt] = p.x + (size_t)(xok[nt] ? g + 8 * nt : 0) * p.K + 32 * t;
    }
    uint4 xn[NT][4];
    auto load_x = [&](int grp) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                xn[nt][j] = make_uint4(0, 0, 0, 0);
                if (xok[nt]) xn[nt][j] = *reinterpret_cast<const uint4*>(xrow[nt] + 128 * grp + 8 * j);
            }
    };

    float acc[MT][NT][4];
    auto clear_acc = [&]() {
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;
    };
    clear_acc();

    // End of unit u for this warp: its K slice goes to shared memory; after the CTA barrier the first NT * 4 warps add the
    // kWarps slices in warp order (fixed order: bit-reproducible), apply the epilogue and store, while the others move on.
    auto unit_end = [&](int u) {
        const int par = u & 1;
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) red[par][warp][mt][nt][e][lane] = acc[mt][nt][e];
        clear_acc();
        __syncthreads();
        // thread = (nt, e, lane): element (feature f0 + g + 8 (e >> 1), batch row 8 nt + 2 t + (e & 1)) of every tile
        for (int i = threadIdx.x; i < NT * 4 * 32; i += kWarps * 32) {
            const int l = i & 31, e = (i >> 5) & 3, nt = i >> 7;
            const int row = 8 * nt + 2 * (l & 3) + (e & 1);
            float v[MT];
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; w++) sum += red[par][w][mt][nt][e][l];
                v[mt] = sum;
            }
            if (row >= p.M) continue;
            if (SILU) {
                int mi, f0;
                unit_tile(u, 0, mi, f0);
                float val = v[0];
                val *= 1.0f / (1.0f + expf(-val));
                val *= v[MT - 1];
                p.m[0].y[(size_t)row * p.m[0].ldy + f0 + (l >> 2) + 8 * (e >> 1)] = __float2half(val);
            } else {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    int mi, f0;
                    unit_tile(u, mt, mi, f0);
                    const SkMat& mm = p.m[mi];
                    const size_t at = (size_t)row * mm.ldy + f0 + (l >> 2) + 8 * (e >> 1);
                    float val = v[mt];
                    if (p.residual) val += __half2float(p.residual[at]) * p.rscale;
                    mm.y[at] = __float2half(val);
                }
            }
        }
        // the buffer of parity `par` is written again at unit u + 2, after every thread has passed the barrier of unit u + 1,
        // which the threads that read it here reach only when they are done
    };

    if (gpw == 0) {   // fewer groups than warps: this warp only takes part in the reductions
        for (int u = 0; u < my_units; u++) unit_end(u);
        return;
    }
    int u = 0, gi = 0;
    load_x(g_begin);
    for (int base = 0; base < total; base += D) {
#pragma unroll
        for (int d = 0; d < D; d++) {
            if (base + d >= total) break;
            const int grp = g_begin + gi;
            // this step's x pairs in the unpack's order; the next step's x leaves now
            uint32_t xp[NT][4][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int j = 0; j < 4; j++) permute_x8(xn[nt][j], xp[nt][j]);
            const int gi_next = gi + 1 == gpw ? 0 : gi + 1;
            if (base + d + 1 < total) load_x(g_begin + gi_next);
            const Stage& cur = st[d];
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                uint32_t zlo[2], zhi[2];
                float sc[2];
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint32_t z = (cur.zw[mt][hh] >> (4 * (grp & 7))) & 0xFu;
                    zlo[hh] = (0x6400u | z) * 0x00010001u;          // 1024 + z
                    zhi[hh] = (0x5400u | (z << 4)) * 0x00010001u;   // 64 + z
                    sc[hh] = __half2float(cur.sc[mt][hh]);
                }
                float c[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; nt++) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
                const uint32_t wa[4] = {cur.w[mt][0].x, cur.w[mt][0].y, cur.w[mt][0].z, cur.w[mt][0].w};
                const uint32_t wb[4] = {cur.w[mt][1].x, cur.w[mt][1].y, cur.w[mt][1].z, cur.w[mt][1].w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t da[4], db[4];
                    unpack8(wa[j], zlo[0], zhi[0], da);
                    unpack8(wb[j], zlo[1], zhi[1], db);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        mma_f16(c[nt], da[0], db[0], da[1], db[1], xp[nt][j][0], xp[nt][j][1]);
                        mma_f16(c[nt], da[2], db[2], da[3], db[3], xp[nt][j][2], xp[nt][j][3]);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    acc[mt][nt][0] = fmaf(sc[0], c[nt][0], acc[mt][nt][0]);
                    acc[mt][nt][1] = fmaf(sc[0], c[nt][1], acc[mt][nt][1]);
                    acc[mt][nt][2] = fmaf(sc[1], c[nt][2], acc[mt][nt][2]);
                    acc[mt][nt][3] = fmaf(sc[1], c[nt][3], acc[mt][nt][3]);
                }
            }
            prefetch(st[d]);   // the stage is spent: its next occupant, D steps ahead, leaves now
            if (++gi == gpw) {
                unit_end(u);
                gi = 0;
                u++;
            }
        }
    }
}

constexpr int kSms = 148;   // B200: one persistent CTA per SM (a smaller part would only leave CTAs queued behind the first wave)
constexpr size_t red_bytes(int MT, int NT) { return 2 * (size_t)warps_of(MT, NT) * MT * NT * 4 * 32 * sizeof(float); }

int fill(SkParams& p, const uint16_t* x, int M, int K) {
    if (!x || M < 1 || M > 16) return Q4_ERR_INVALID;
    if (K <= 0 || (K % 128)) return Q4_ERR_UNSUPPORTED_SIZE;
    p.x = reinterpret_cast<const __half*>(x);
    p.M = M;
    p.K = K;
    p.PW = q4_pw(K);
    p.PZ = q4_pz(K);
    p.G = q4_groups(K);
    return Q4_OK;
}

SkMat sk_mat(const q4_qweight* w, uint16_t* y, int ldy, int tile0) {
    SkMat m;
    m.w = w->weight;
    m.z = w->zeros;
    m.s = reinterpret_cast<const __half*>(w->scales);
    m.y = reinterpret_cast<__half*>(y);
    m.ldy = ldy;
    m.tile0 = tile0;
    return m;
}

template <int MT, int NT, bool SILU>
int launch_variant(const SkParams& p, cudaStream_t s) {
    constexpr size_t smem = red_bytes(MT, NT);
    static_assert(smem <= 48 * 1024, "the reduction buffers fit the default dynamic shared memory limit: no per-device opt-in is needed");
    const int units = SILU ? p.total_tiles : p.total_tiles / MT;
    Q4Launch L(dim3(units < kSms ? units : kSms), dim3(warps_of(MT, NT) * 32), smem, s);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_skinny_kernel<MT, NT, SILU>, p));
    return Q4_OK;
}

template <bool SILU>
int launch(const SkParams& p, cudaStream_t s) {
    const bool two = p.M > 8;
    if (SILU) return two ? launch_variant<2, 2, true>(p, s) : launch_variant<2, 1, true>(p, s);
    // Two tiles per unit halve the reads of x but double the grain the work is dealt in: take pairs when the most loaded
    // SM then carries no more features than with single tiles.
    const int t = p.total_tiles;
    const bool pair = (t % 2 == 0) && 2 * q4_div_up(t / 2, kSms) <= q4_div_up(t, kSms);
    if (pair) return two ? launch_variant<2, 2, false>(p, s) : launch_variant<2, 1, false>(p, s);
    return two ? launch_variant<1, 2, false>(p, s) : launch_variant<1, 1, false>(p, s);
}

}  // namespace

extern "C" int q4_matmul_q4_rows(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* w, int M, int inpSize, int opSize,
                                 const uint16_t* residual, float residual_scale) {
    SkParams p = {};
    if (int e = fill(p, x, M, inpSize)) return e;
    if (!y || !w) return Q4_ERR_INVALID;
    if (opSize <= 0 || (opSize % 16)) return Q4_ERR_UNSUPPORTED_SIZE;
    p.nmat = 1;
    p.m[0] = sk_mat(w, y, opSize, 0);
    p.total_tiles = opSize / 16;
    p.residual = reinterpret_cast<const __half*>(residual);
    p.rscale = residual_scale;
    return launch<false>(p, (cudaStream_t)stream);
}

extern "C" int q4_qkv_matmul_rows(void* stream, uint16_t* q, uint16_t* k, uint16_t* v, const uint16_t* x, const q4_qweight* qw,
                                  const q4_qweight* kw, const q4_qweight* vw, int M, int inpSize, int opSize, int kvSize) {
    SkParams p = {};
    if (int e = fill(p, x, M, inpSize)) return e;
    if (!q || !k || !v || !qw || !kw || !vw) return Q4_ERR_INVALID;
    if (opSize <= 0 || kvSize <= 0 || (opSize % 32) || (kvSize % 32)) return Q4_ERR_UNSUPPORTED_SIZE;   // a CTA's two tiles lie in one matrix
    p.nmat = 3;
    const int tq = opSize / 16, tkv = kvSize / 16;
    p.m[0] = sk_mat(qw, q, opSize, 0);
    p.m[1] = sk_mat(kw, k, kvSize, tq);
    p.m[2] = sk_mat(vw, v, kvSize, tq + tkv);
    p.total_tiles = tq + 2 * tkv;
    return launch<false>(p, (cudaStream_t)stream);
}

extern "C" int q4_ffn_silu_rows(void* stream, uint16_t* h, const uint16_t* x, const q4_qweight* gate_w, const q4_qweight* up_w, int M,
                                int inpSize, int opSize) {
    SkParams p = {};
    if (int e = fill(p, x, M, inpSize)) return e;
    if (!h || !gate_w || !up_w) return Q4_ERR_INVALID;
    if (opSize <= 0 || (opSize % 16)) return Q4_ERR_UNSUPPORTED_SIZE;
    p.nmat = 2;
    p.m[0] = sk_mat(gate_w, h, opSize, 0);
    p.m[1] = sk_mat(up_w, h, opSize, 0);
    p.total_tiles = opSize / 16;
    return launch<true>(p, (cudaStream_t)stream);
}
