// Small per-token ops: RMSNorm, RoPE, embedding gather, greedy argmax hand-off, the fp16 classifier GEMV,
// and the dequantisation test hooks. Replaces rmsnorm_kernel, RoPERotation_kernel, copy_embedding_kernel,
// argmax_kernel and mat_vec_kernel of the reference (gpu_kernels.h:61-147,340-363,456-501).
#include <math_constants.h>
#include <stdio.h>

#include "q4_common.cuh"

static thread_local char g_last_error[256];
void q4_note_cuda_error(cudaError_t e, const char* file, int line) {
    snprintf(g_last_error, sizeof(g_last_error), "CUDA error in file '%s' in line %i : %s.", file, line, cudaGetErrorString(e));
    fprintf(stderr, "%s\n", g_last_error);
}

extern "C" const char* q4_status_string(int s) {
    switch (s) {
        case Q4_OK: return "ok";
        case Q4_ERR_UNSUPPORTED_SIZE: return "Unsupported matmul size";
        case Q4_ERR_CUDA: return "CUDA error";
        case Q4_ERR_IO: return "I/O error";
        case Q4_ERR_BAD_MODEL: return "bad model file";
        case Q4_ERR_INVALID: return "invalid argument";
        case Q4_ERR_TIMEOUT: return "device-side wait timed out";
        case Q4_ERR_LIMIT: return "size exceeds the entry point's capacity";
        default: return "unknown status";
    }
}
extern "C" int q4_abi_version(void) { return 1; }
extern "C" const char* q4_build_arch(void) { return "sm_100a"; }

namespace {

// Block-wide sum; every thread gets the total. blockDim.x multiple of 32, <= 1024.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    __syncthreads();
    return t;
}

// o = x * rsqrt(mean(x^2) + 1e-5) * w. Same arithmetic and rounding points as gpu_kernels.h:72-105
// (fp32 sum of squares, eps added after the mean, val * (ss * w), one fp16 rounding).
__global__ void __launch_bounds__(1024) rmsnorm_kernel(__half* o, const __half* x, const __half* w, int size) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch_dependents();
    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < size; i += blockDim.x * 8) {
        if (i + 8 <= size) {
            uint4 v = *reinterpret_cast<const uint4*>(x + i);
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 f = __half22float2(h[j]);
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
            }
        } else {
            for (int j = i; j < size; j++) { float f = __half2float(x[j]); ss = fmaf(f, f, ss); }
        }
    }
    ss = block_sum(ss, red);
    ss /= size;
    ss += 1e-5f;
    ss = 1.0f / sqrtf(ss);
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        float val = __half2float(x[i]);
        val *= ss * __half2float(w[i]);
        o[i] = __float2half(val);
    }
}

// RoPERotation_kernel (gpu_kernels.h:340-363): rotate-half RoPE of the query heads in place and of the key heads of cache
// row `pos`. A block takes kRopeHeadsPerBlock heads; the angles depend on the position only, so the block evaluates the
// head_size / 2 (cos, sin) pairs once into shared memory and every head of the block reuses them. head_size <= 512.
constexpr int kRopeHeadsPerBlock = 4;
__global__ void __launch_bounds__(256) rope_kernel(__half* q, __half* key_cache, int num_heads, int num_kv_heads, int head_size, const int* pPos,
                                                   long long loff, float theta) {
    griddep_wait();
    griddep_launch_dependents();
    __shared__ float2 table[256];
    const int pos = *pPos, pairs = head_size / 2;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) table[i] = rope_cos_sin(pos, i, head_size, theta);
    __syncthreads();
    __half* key_row = key_cache + loff + (long long)pos * num_kv_heads * head_size;
    const int first = blockIdx.x * kRopeHeadsPerBlock, last = min(first + kRopeHeadsPerBlock, num_heads);
    for (int e = threadIdx.x; e < (last - first) * pairs; e += blockDim.x) {
        const int head = first + e / pairs, i = e % pairs;
        __half* qh = q + (size_t)head * head_size;
        rope_rotate(qh + i, qh + i + pairs, qh + i, qh + i + pairs, table[i]);
        if (head < num_kv_heads) {
            __half* kh = key_row + (size_t)head * head_size;
            rope_rotate(kh + i, kh + i + pairs, kh + i, kh + i + pairs, table[i]);
        }
    }
}

// gpu_kernels.h:61-69. tokens[] lives in pinned host memory and is read through the mapping.
__global__ void embed_kernel(__half* x, const __half* __restrict__ table, int dim, const int* tokens, const int* pPos) {
    griddep_wait();
    griddep_launch_dependents();
    const int token = tokens[*pPos];
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)token * dim);
    uint4* dst = reinterpret_cast<uint4*>(x);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim / 8; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// Greedy hand-off: gpu_kernels.h:456-501. Ordered key = (value, lowest index).
__global__ void __launch_bounds__(1024) argmax_kernel(const __half* __restrict__ x, int size, int* result, volatile int* pPos,
                                                      int* pPosGpu, int write_token) {
    __shared__ float sval[32];
    __shared__ int sidx[32];
    griddep_wait();
    griddep_launch_dependents();
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = __half2float(x[i]);
        if (v > best) { best = v; bi = i; }
    }
    if (bi == 0x7fffffff && threadIdx.x < size) bi = threadIdx.x;  // all -inf / NaN column
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? sval[lane] : -CUDART_INF_F;
        bi = lane < nw ? sidx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            int token_pos = *pPos;
            token_pos++;
            if (write_token) result[token_pos] = (bi == 0x7fffffff) ? 0 : bi;
            *pPos = token_pos;
            *pPosGpu = token_pos;
        }
    }
}

// fp16 GEMV (classifier): out[d] = alpha * sum_n w[d][n] * x[n]. gpu_kernels.h:117-147.
// One warp per 2 output rows; each lane streams 16-byte pieces, 4 per row in flight.
constexpr int kF16Rows = 2;
__global__ void __launch_bounds__(256) matvec_f16_kernel(__half* out, const __half* x, const __half* __restrict__ w, int n, int d,
                                                         float alpha) {
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int row0 = warp_global * kF16Rows;
    const bool active = row0 < d;
    const int nvec = n >> 3;  // uint4 per row
    constexpr int U = 4;
    uint4 wv[kF16Rows][U];
    const uint4* wr[kF16Rows];
#pragma unroll
    for (int r = 0; r < kF16Rows; r++) wr[r] = reinterpret_cast<const uint4*>(w + (size_t)min(row0 + r, d - 1) * n);
    int c = lane;
    if (active) {
#pragma unroll
        for (int r = 0; r < kF16Rows; r++)
#pragma unroll
            for (int u = 0; u < U; u++)
                if (c + u * 32 < nvec) wv[r][u] = ldg_stream(wr[r] + c + u * 32);
    }
    griddep_wait();
    griddep_launch_dependents();
    if (!active) return;
    float acc[kF16Rows] = {0.f, 0.f};
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    while (c < nvec) {
        uint4 cur[kF16Rows][U];
#pragma unroll
        for (int r = 0; r < kF16Rows; r++)
#pragma unroll
            for (int u = 0; u < U; u++) cur[r][u] = wv[r][u];
        const int cn = c + U * 32;
#pragma unroll
        for (int r = 0; r < kF16Rows; r++)
#pragma unroll
            for (int u = 0; u < U; u++)
                if (cn + u * 32 < nvec) wv[r][u] = ldg_stream(wr[r] + cn + u * 32);
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (c + u * 32 < nvec) {
                const uint4 xq = xv[c + u * 32];
                const __half2* xh = reinterpret_cast<const __half2*>(&xq);
#pragma unroll
                for (int r = 0; r < kF16Rows; r++) {
                    const __half2* wh = reinterpret_cast<const __half2*>(&cur[r][u]);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 a = __half22float2(wh[j]), b = __half22float2(xh[j]);
                        acc[r] = fmaf(a.x, b.x, acc[r]);
                        acc[r] = fmaf(a.y, b.y, acc[r]);
                    }
                }
            }
        }
        c = cn;
    }
#pragma unroll
    for (int r = 0; r < kF16Rows; r++) {
        const float s = warp_sum(acc[r]) * alpha;
        if (lane == 0 && row0 + r < d) out[row0 + r] = __float2half(s);
    }
}

__global__ void dequant_kernel(float* out, const uint32_t* w, const uint32_t* z, const __half* s, int K, int N, int PW, int PZ, int G) {
    const size_t total = (size_t)N * K;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / K), k = (int)(i % K), g = k >> 7;
        const uint32_t q = (w[(size_t)n * PW + (k >> 3)] >> (4 * (k & 7))) & 0xFu;
        const uint32_t zz = (z[(size_t)n * PZ + (g >> 3)] >> (4 * (g & 7))) & 0xFu;
        out[i] = ((float)q - (float)zz) * __half2float(s[(size_t)n * G + g]);
    }
}

__global__ void unpack_kernel(uint8_t* q_out, uint8_t* z_out, const uint32_t* w, const uint32_t* z, int K, int N, int PW, int PZ, int G) {
    const size_t total = (size_t)N * K;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / K), k = (int)(i % K);
        q_out[i] = (uint8_t)((w[(size_t)n * PW + (k >> 3)] >> (4 * (k & 7))) & 0xFu);
        if (k < G) z_out[(size_t)n * G + k] = (uint8_t)((z[(size_t)n * PZ + (k >> 3)] >> (4 * (k & 7))) & 0xFu);
    }
}

}  // namespace

extern "C" int q4_rmsnorm(void* stream, uint16_t* o, const uint16_t* x, const uint16_t* weight, int size) {
    if (!o || !x || !weight || size <= 0) return Q4_ERR_INVALID;
    Q4Launch L(dim3(1), dim3(size >= 8192 ? 1024 : 512), 0, (cudaStream_t)stream);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, rmsnorm_kernel, (__half*)o, (const __half*)x, (const __half*)weight, size));
    return Q4_OK;
}

extern "C" int q4_rope(void* stream, uint16_t* q, uint16_t* k, int num_heads, int num_kv_heads, int head_size, const int* pPos,
                       int loff, float rope_theta) {
    if (!q || !k || !pPos || num_heads <= 0 || head_size <= 0 || (head_size & 1) || num_kv_heads > num_heads) return Q4_ERR_INVALID;
    if (head_size > 512) return Q4_ERR_UNSUPPORTED_SIZE;
    Q4Launch L(dim3(q4_div_up(num_heads, kRopeHeadsPerBlock)), dim3(256), 0, (cudaStream_t)stream);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, rope_kernel, (__half*)q, (__half*)k, num_heads, num_kv_heads, head_size, pPos, (long long)loff, rope_theta));
    return Q4_OK;
}

extern "C" int q4_embed(void* stream, uint16_t* x, const uint16_t* table, int dim, const int* tokens, const int* pPos) {
    if (!x || !table || !tokens || !pPos || dim <= 0 || (dim & 7)) return Q4_ERR_INVALID;
    Q4Launch L(dim3(q4_div_up(dim / 8, 256)), dim3(256), 0, (cudaStream_t)stream);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, embed_kernel, (__half*)x, (const __half*)table, dim, tokens, pPos));
    return Q4_OK;
}

extern "C" int q4_argmax(void* stream, const uint16_t* logits, int size, int* tokens_pinned, volatile int* pos_pinned, int* pos_dev,
                         int write_token) {
    if (!logits || !tokens_pinned || !pos_pinned || !pos_dev || size <= 0) return Q4_ERR_INVALID;
    Q4Launch L(dim3(1), dim3(1024), 0, (cudaStream_t)stream);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, argmax_kernel, (const __half*)logits, size, tokens_pinned, pos_pinned, pos_dev, write_token));
    return Q4_OK;
}

extern "C" int q4_matmul_f16(void* stream, uint16_t* xout, const uint16_t* x, const uint16_t* w, int n, int d, float alpha) {
    if ((n & 7) || (d & 7) || n <= 0 || d <= 0) return Q4_ERR_UNSUPPORTED_SIZE;
    if (!xout || !x || !w) return Q4_ERR_INVALID;
    const int rows_per_block = 8 * kF16Rows;
    Q4Launch L(dim3(q4_div_up(d, rows_per_block)), dim3(256), 0, (cudaStream_t)stream);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, matvec_f16_kernel, (__half*)xout, (const __half*)x, (const __half*)w, n, d, alpha));
    return Q4_OK;
}

extern "C" int q4_dequant(void* stream, float* out, const q4_qweight* w, int K, int N) {
    if (!out || !w || K <= 0 || N <= 0) return Q4_ERR_INVALID;
    dequant_kernel<<<1184, 256, 0, (cudaStream_t)stream>>>(out, w->weight, w->zeros, (const __half*)w->scales, K, N, q4_pw(K), q4_pz(K), q4_groups(K));
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}

extern "C" int q4_unpack_nibbles(void* stream, uint8_t* q_out, uint8_t* z_out, const q4_qweight* w, int K, int N) {
    if (!q_out || !z_out || !w || K <= 0 || N <= 0) return Q4_ERR_INVALID;
    unpack_kernel<<<1184, 256, 0, (cudaStream_t)stream>>>(q_out, z_out, w->weight, w->zeros, K, N, q4_pw(K), q4_pz(K), q4_groups(K));
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}
