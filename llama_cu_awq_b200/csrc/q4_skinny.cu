// AWQ W4 g128 dequantize-and-multiply for a handful of rows (1 <= M <= 16): the projections of batched decode.
//
// The reference has one sequence per process (RunState, common.h:62-78) and its mat_vec_kernel_int4 family
// (gpu_kernels.h:179-283) reads every weight once per token; with several sequences decoded together the weights are
// still read once per STEP, so the op stays bound by HBM as long as the per-weight work is small. That is what this
// kernel is built for; the tcgen05 GEMM (q4_gemm.cu) takes over from M > 16, where the contraction starts to matter.
//
// Work split: a CTA (8 warps) owns 16 * MT output features of one launch and the whole K axis; warp w takes the w-th
// eighth of the 128-input groups, and the eight partial tiles are summed in warp order through shared memory (fixed
// order: results are bit-reproducible). Inside a warp the product runs on mma.sync m16n8k16 (fp16 in, fp32 out) with
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
#define SK_WARPS 8
#endif
#ifndef SK_D11
#define SK_D11 4
#endif
#ifndef SK_D12
#define SK_D12 3
#endif
#ifndef SK_D2
#define SK_D2 2
#endif
#ifndef SK_MINB
#define SK_MINB 2
#endif
constexpr int kWarps = SK_WARPS;

// MT: 16-feature tiles per CTA (1 or 2); NT: 8-row batch tiles (1: M <= 8, 2: M <= 16); SILU: tile 0 = gate, tile 1 = up.
template <int MT, int NT, bool SILU>
__global__ void __launch_bounds__(kWarps * 32, (MT * NT == 4) ? 1 : SK_MINB) q4_skinny_kernel(const SkParams p) {
    __shared__ float red[kWarps][MT][NT][4][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;

    // the CTA's tiles: feature rows and their matrix
    const uint4* wrow[MT][2];
    const uint32_t* zrow[MT][2];
    const __half* srow[MT][2];
    int mat_of[MT], f0[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        int mi, tile;
        if (SILU) {
            mi = mt;
            tile = blockIdx.x;
        } else {
            tile = blockIdx.x * MT + mt;
            mi = 0;
            if (p.nmat > 1 && tile >= p.m[1].tile0) mi = 1;
            if (p.nmat > 2 && tile >= p.m[2].tile0) mi = 2;
            tile -= p.m[mi].tile0;
        }
        mat_of[mt] = mi;
        f0[mt] = tile * 16;
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            const size_t row = (size_t)f0[mt] + g + 8 * hh;
            wrow[mt][hh] = reinterpret_cast<const uint4*>(p.m[mi].w + row * p.PW) + t;
            zrow[mt][hh] = p.m[mi].z + row * p.PZ;
            srow[mt][hh] = p.m[mi].s + row * p.G;
        }
    }
    // this warp's groups
    const int g_begin = (int)((long long)p.G * warp / kWarps), g_end = (int)((long long)p.G * (warp + 1) / kWarps);

    float acc[MT][NT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[mt][nt][0] = acc[mt][nt][1] = acc[mt][nt][2] = acc[mt][nt][3] = 0.f;

    // A group's operands per thread: 16 bytes of packed weights, the zeros word and the scale for each of its 2 MT rows.
    // D groups are in flight ahead of the math (the loads of a warp's first D groups leave before anything else happens;
    // short K slices - 4 groups per warp at K = 4096 - are then covered whole).
    constexpr int D = (MT == 1) ? (NT == 1 ? SK_D11 : SK_D12) : SK_D2;
    struct Stage {
        uint4 w[MT][2];
        uint32_t zw[MT][2];
        __half sc[MT][2];
    };
    Stage st[D];
    auto load_stage = [&](Stage& d, int grp) {
        if (grp < g_end) {
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    d.w[mt][hh] = ldg_stream(wrow[mt][hh] + 4 * grp);
                    d.zw[mt][hh] = __ldg(zrow[mt][hh] + (grp >> 3));
                    d.sc[mt][hh] = __ldg(srow[mt][hh] + grp);
                }
        }
    };
#pragma unroll
    for (int d = 0; d < D; d++) load_stage(st[d], g_begin + d);
    griddep_wait();
    griddep_launch_dependents();

    const __half* xrow[NT];
    bool xok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        xok[nt] = g + 8 * nt < p.M;
        xrow[nt] = p.x + (size_t)(xok[nt] ? g + 8 * nt : 0) * p.K + 32 * t;
    }

    for (int base = g_begin; base < g_end; base += D) {
#pragma unroll
        for (int d = 0; d < D; d++) {
            const int grp = base + d;
            if (grp >= g_end) break;
            const Stage cur = st[d];
            load_stage(st[d], grp + D);
            // the batch rows' 32 inputs of this thread's quarter of the group, in the unpack's pairing
            uint32_t xp[NT][4][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (xok[nt]) xv = *reinterpret_cast<const uint4*>(xrow[nt] + 128 * grp + 8 * j);
                    permute_x8(xv, xp[nt][j]);
                }
            }
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
        }
    }

    // the eight K slices, summed in warp order
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) red[warp][mt][nt][e][lane] = acc[mt][nt][e];
    __syncthreads();
    // thread = (nt, e, lane) for all tiles: element (feature f0 + g + 8 (e >> 1), batch row 8 nt + 2 t + (e & 1))
    for (int i = threadIdx.x; i < NT * 4 * 32; i += kWarps * 32) {
        const int l = i & 31, e = (i >> 5) & 3, nt = i >> 7;
        const int row = 8 * nt + 2 * (l & 3) + (e & 1);
        float v[MT];
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) s += red[w][mt][nt][e][l];
            v[mt] = s;
        }
        if (row >= p.M) continue;
        if (SILU) {
            float val = v[0];
            val *= 1.0f / (1.0f + expf(-val));
            val *= v[MT - 1];
            p.m[0].y[(size_t)row * p.m[0].ldy + f0[0] + (l >> 2) + 8 * (e >> 1)] = __float2half(val);
        } else {
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const SkMat& mm = p.m[mat_of[mt]];
                const size_t at = (size_t)row * mm.ldy + f0[mt] + (l >> 2) + 8 * (e >> 1);
                float val = v[mt];
                if (p.residual) val += __half2float(p.residual[at]) * p.rscale;
                mm.y[at] = __float2half(val);
            }
        }
    }
}

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

template <bool SILU>
int launch(const SkParams& p, cudaStream_t s) {
    const bool two = p.M > 8;
    if (SILU) {
        Q4Launch L(dim3(p.total_tiles), dim3(kWarps * 32), 0, s);
        if (two) Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_skinny_kernel<2, 2, true>, p));
        else Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_skinny_kernel<2, 1, true>, p));
        return Q4_OK;
    }
    // two tiles per CTA halve the x traffic; one tile per CTA when that is what it takes to put two CTAs on every SM
    const bool pair = (p.total_tiles % 2 == 0) && p.total_tiles >= 4 * 148;
    Q4Launch L(dim3(pair ? p.total_tiles / 2 : p.total_tiles), dim3(kWarps * 32), 0, s);
    if (pair) {
        if (two) Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_skinny_kernel<2, 2, false>, p));
        else Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_skinny_kernel<2, 1, false>, p));
    } else {
        if (two) Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_skinny_kernel<1, 2, false>, p));
        else Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_skinny_kernel<1, 1, false>, p));
    }
    return Q4_OK;
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
