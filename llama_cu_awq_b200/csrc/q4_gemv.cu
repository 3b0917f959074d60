// AWQ W4 g128 dequantize-and-multiply GEMV kernels (batch 1) and their C-ABI launchers.
//
// Replaces mat_vec_kernel_int4 / qkv_matvec_kernel / ffn_matvec_silu_kernel of the reference
// (gpu_kernels.h:179-283) and their wrappers (llama2_q4.cu:367-404).
//
// Work split: a tile is 8 consecutive output columns of one matrix. Each thread owns 32-weight chunks of the
// K axis (one 128-bit load per output column per chunk, lanes adjacent -> 512 B coalesced per warp per column),
// keeps the matching 32 activations in registers and reuses them for all 8 columns. Nibbles are unpacked two at
// a time into half2 with one LOP3 each (magic-number trick), the zero point is folded into the same subtract,
// products are summed in short half2 chains (8 weights) that are flushed to fp32, and the group scale is
// applied in fp32. The 8 per-column partials are reduced across the warp with a transposing butterfly
// (9 shuffles instead of 40) and, when several warps share a tile, through shared memory.
// Weight loads of the first chunk are issued before griddepcontrol.wait, so under programmatic dependent
// launch they overlap the tail of the previous kernel (weights never depend on activations).
#include "q4_common.cuh"

namespace {

constexpr int kRows = 8;  // output columns per tile

struct GemvMat {
    const uint32_t* w;
    const uint32_t* z;
    const __half* s;
    __half* out;
    int n;       // output columns of this matrix
    int tile0;   // first tile index of this matrix in the launch
    int kv;      // 1: out += loff + *pos * n
};

struct GemvParams {
    const __half* x;
    int K, PW, PZ, G;
    int nmat;
    GemvMat m[3];
    int total_tiles;
    int accum;
    float gpu_count;
    long long loff;
    const int* pos;
};

__device__ __forceinline__ float silu_mul(float g, float u) {
    float val = g;
    val *= 1.0f / (1.0f + expf(-val));
    val *= u;
    return val;
}

// After the call, lane l holds in the return value the warp total of acc[(l>>2) & 7]
// (lanes 4r..4r+3 all hold column r).
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
    return a1;  // column index = (bit4?4:0) + (bit3?2:0) + (bit2?1:0) = (lane >> 2) & 7
}

// KW = warps that share one tile along K (1 or 4). Block = 128 threads.
// SILU: tile = 4 gate columns (acc 0..3) + the same 4 up columns (acc 4..7); m[0]=gate, m[1]=up.
template <int KW, bool SILU>
__global__ void __launch_bounds__(128) q4_gemv_kernel(const GemvParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile = (KW == 4) ? blockIdx.x : blockIdx.x * 4 + warp;
    const bool active = tile < p.total_tiles;  // warp-uniform

    int mi = 0;
    if (!SILU) {
        if (p.nmat > 1 && tile >= p.m[1].tile0) mi = 1;
        if (p.nmat > 2 && tile >= p.m[2].tile0) mi = 2;
    }
    const GemvMat& m = p.m[mi];
    const int row0 = SILU ? tile * 4 : (tile - m.tile0) * kRows;

    const uint32_t* wrow[kRows];
    const uint32_t* zrow[kRows];
    const __half* srow[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        const GemvMat& mm = SILU ? p.m[r >> 2] : m;
        const int row = SILU ? row0 + (r & 3) : row0 + r;
        wrow[r] = mm.w + (size_t)row * p.PW;
        zrow[r] = mm.z + (size_t)row * p.PZ;
        srow[r] = mm.s + (size_t)row * p.G;
    }

    const int nchunks = p.PW >> 2;
    const int kt = (KW == 4) ? threadIdx.x : lane;
    constexpr int kstride = KW * 32;

    float acc[kRows];
#pragma unroll
    for (int r = 0; r < kRows; r++) acc[r] = 0.f;

    uint4 wv[kRows];
    int c = kt;
    if (active && c < nchunks) {
#pragma unroll
        for (int r = 0; r < kRows; r++) wv[r] = ldg_stream(reinterpret_cast<const uint4*>(wrow[r]) + c);
    }
    griddep_wait();
    griddep_launch_dependents();
    if (active) {
        while (c < nchunks) {
            // activations of this chunk (zero beyond K so that padded weight words contribute nothing)
            uint32_t xp[4][4];
            const int k0 = c * 32;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint4 xv = make_uint4(0, 0, 0, 0);
                if (k0 + j * 8 < p.K) xv = *reinterpret_cast<const uint4*>(p.x + k0 + j * 8);
                permute_x8(xv, xp[j]);
            }
            const int g = c >> 2;
            uint4 cur[kRows];
#pragma unroll
            for (int r = 0; r < kRows; r++) cur[r] = wv[r];
            const int cn = c + kstride;
            if (cn < nchunks) {
#pragma unroll
                for (int r = 0; r < kRows; r++) wv[r] = ldg_stream(reinterpret_cast<const uint4*>(wrow[r]) + cn);
            }
#pragma unroll
            for (int r = 0; r < kRows; r++) {
                const uint32_t zw = __ldg(zrow[r] + (g >> 3));
                const uint32_t z = (zw >> (4 * (g & 7))) & 0xFu;
                const float sc = __half2float(__ldg(srow[r] + g));
                uint32_t zlo, zhi;
                zero_consts(z, zlo, zhi);
                const __half2 zero2 = u2h2(0u);
                // four products per half lane, then fp32: longer fp16 chains cost accuracy on long rows (K > 8192)
                const __half2 a0 = dot8(cur[r].x, xp[0], zlo, zhi, zero2);
                const __half2 a1 = dot8(cur[r].y, xp[1], zlo, zhi, zero2);
                const __half2 b0 = dot8(cur[r].z, xp[2], zlo, zhi, zero2);
                const __half2 b1 = dot8(cur[r].w, xp[3], zlo, zhi, zero2);
                acc[r] = fmaf(sc, (h2sum(a0) + h2sum(a1)) + (h2sum(b0) + h2sum(b1)), acc[r]);
            }
            c = cn;
        }
    }

    float tot = transpose_reduce8(acc, lane);
    if (KW == 4) {
        __shared__ float red[4][kRows];
        if ((lane & 3) == 0) red[warp][lane >> 2] = tot;
        __syncthreads();
        if (warp != 0) return;
        const int r = lane >> 2;
        tot = red[0][r] + red[1][r] + red[2][r] + red[3][r];
    }
    if (!active) return;

    if (SILU) {
        // lanes 4r..4r+3 hold column r: gate columns are r=0..3, up columns r=4..7
        const float up = __shfl_sync(0xffffffffu, tot, (lane + 16) & 31);
        if (lane < 16 && (lane & 3) == 0) {
            const int n = row0 + (lane >> 2);
            p.m[0].out[n] = __float2half(silu_mul(tot, up));
        }
    } else if ((lane & 3) == 0) {
        const int n = row0 + (lane >> 2);
        __half* out = m.out;
        if (m.kv) out += p.loff + (long long)(*p.pos) * m.n;
        float sum = tot;
        if (p.accum) sum += __half2float(out[n]) / p.gpu_count;
        out[n] = __float2half(sum);
    }
}

int check_sizes(int K, int N) { return ((K & 7) || (N & 7) || K <= 0 || N <= 0) ? Q4_ERR_UNSUPPORTED_SIZE : Q4_OK; }

void fill_dims(GemvParams& p, int K) {
    p.K = K;
    p.PW = q4_pw(K);
    p.PZ = q4_pz(K);
    p.G = q4_groups(K);
}

template <bool SILU>
int launch(const GemvParams& p, cudaStream_t s) {
    const int nchunks = p.PW / 4;
    if (nchunks > 64) {
        Q4Launch L(dim3(p.total_tiles), dim3(128), 0, s);
        Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_gemv_kernel<4, SILU>, p));
    } else {
        Q4Launch L(dim3(q4_div_up(p.total_tiles, 4)), dim3(128), 0, s);
        Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, q4_gemv_kernel<1, SILU>, p));
    }
    return Q4_OK;
}

GemvMat mat(const q4_qweight* w, uint16_t* out, int n, int tile0, int kv) {
    GemvMat m;
    m.w = w->weight;
    m.z = w->zeros;
    m.s = reinterpret_cast<const __half*>(w->scales);
    m.out = reinterpret_cast<__half*>(out);
    m.n = n;
    m.tile0 = tile0;
    m.kv = kv;
    return m;
}

}  // namespace

extern "C" int q4_matmul_q4(void* stream, uint16_t* xout, const uint16_t* x, const q4_qweight* w, int inpSize,
                            int opSize, int accum, int gpu_count, int loff, const int* pPos) {
    if (int e = check_sizes(inpSize, opSize)) return e;
    if (!xout || !x || !w || gpu_count < 1 || (loff != -1 && !pPos)) return Q4_ERR_INVALID;
    GemvParams p = {};
    fill_dims(p, inpSize);
    p.x = reinterpret_cast<const __half*>(x);
    p.nmat = 1;
    p.m[0] = mat(w, xout, opSize, 0, loff != -1);
    p.total_tiles = opSize / kRows;
    p.accum = accum != 0;
    p.gpu_count = (float)gpu_count;
    p.loff = loff == -1 ? 0 : loff;
    p.pos = pPos;
    return launch<false>(p, (cudaStream_t)stream);
}

extern "C" int q4_qkv_matvec(void* stream, uint16_t* q, uint16_t* key_cache, uint16_t* value_cache, const uint16_t* x,
                             const q4_qweight* qw, const q4_qweight* kw, const q4_qweight* vw, int inpSize, int opSize,
                             int kvSize, int loff, const int* pPos) {
    if (int e = check_sizes(inpSize, opSize)) return e;
    if (int e = check_sizes(inpSize, kvSize)) return e;
    if (!q || !key_cache || !value_cache || !x || !qw || !kw || !vw || !pPos || loff < 0) return Q4_ERR_INVALID;
    GemvParams p = {};
    fill_dims(p, inpSize);
    p.x = reinterpret_cast<const __half*>(x);
    p.nmat = 3;
    const int tq = opSize / kRows, tkv = kvSize / kRows;
    p.m[0] = mat(qw, q, opSize, 0, 0);
    p.m[1] = mat(kw, key_cache, kvSize, tq, 1);
    p.m[2] = mat(vw, value_cache, kvSize, tq + tkv, 1);
    p.total_tiles = tq + 2 * tkv;
    p.accum = 0;
    p.gpu_count = 1.f;
    p.loff = loff;
    p.pos = pPos;
    return launch<false>(p, (cudaStream_t)stream);
}

extern "C" int q4_ffn_matvec_silu(void* stream, uint16_t* xout, const uint16_t* x, const q4_qweight* gate_w,
                                  const q4_qweight* up_w, int inpSize, int opSize) {
    if (int e = check_sizes(inpSize, opSize)) return e;
    if (!xout || !x || !gate_w || !up_w) return Q4_ERR_INVALID;
    GemvParams p = {};
    fill_dims(p, inpSize);
    p.x = reinterpret_cast<const __half*>(x);
    p.nmat = 2;
    p.m[0] = mat(gate_w, xout, opSize, 0, 0);
    p.m[1] = mat(up_w, xout, opSize, 0, 0);
    p.total_tiles = opSize / 4;
    p.gpu_count = 1.f;
    return launch<true>(p, (cudaStream_t)stream);
}
