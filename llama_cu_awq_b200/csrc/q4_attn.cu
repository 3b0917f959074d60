// fp16 attention of one query per head over the KV cache, split along the sequence so that every SM has work
// at any context length (the reference's three kernels give one head's AV product to 4 blocks only).
// Replaces MultiHeadAttention (llama2_q4.cu:410-427; mat_vec_kernel_simple, softmax_kernel, vec_mat_kernel at
// gpu_kernels.h:150-176,365-454,287-337).
//
// Pass 1: grid (splits, heads). A block takes positions [t0, t1) of one head. Eight lanes share a position
// (16 head dims each, two 128-bit loads of K and of V), so a warp covers 4 positions per step and a block of 4
// warps 16. Scores are rounded to fp16 like the reference's; the softmax runs online in fp32 (running max, sum
// and un-normalised V accumulator per lane group), merged across the block in shared memory and written to
// scratch as (max, sum, acc[head_size]).
// Pass 2: one block per head merges the splits and writes fp16.
// The sequence length comes from *pPos on the device; the grid does not depend on it.
#include <math_constants.h>

#include <stdio.h>

#include <mutex>

#include "q4_common.cuh"

namespace {

constexpr int kAttnThreads = 128;
constexpr int kGroups = kAttnThreads / 8;  // positions in flight per block
constexpr int kMaxHeadSize = 256;

int attn_splits(int num_heads) {
    int s = q4_div_up(2 * 148, num_heads);
    if (s < 1) s = 1;
    if (s > 32) s = 32;
    return s;
}

template <int HS>
__global__ void __launch_bounds__(kAttnThreads) attn_partial_kernel(float* scratch, const __half* q, const __half* kc, const __half* vc,
                                                                    int kv_mul, int kv_stride, const int* pPos) {
    constexpr int PER = HS / 8;      // head dims per lane
    constexpr int VEC = PER / 8;     // uint4 per lane per row
    __shared__ float sm_m[kGroups], sm_l[kGroups];
    __shared__ float sm_acc[kGroups][HS];

    const int h = blockIdx.y, split = blockIdx.x, nsplit = gridDim.x;
    const int lane8 = threadIdx.x & 7, grp = threadIdx.x >> 3;
    griddep_wait();
    griddep_launch_dependents();
    const int T = *pPos + 1;
    // split boundaries in units of kGroups positions
    const int units = (T + kGroups - 1) / kGroups;
    const int u0 = (int)((long long)units * split / nsplit), u1 = (int)((long long)units * (split + 1) / nsplit);
    const int t0 = u0 * kGroups, t1 = min(u1 * kGroups, T);

    float qf[PER];
    {
        const __half* qp = q + (size_t)h * HS + lane8 * PER;
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            uint4 u = *reinterpret_cast<const uint4*>(qp + v * 8);
            const __half2* hh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
            for (int j = 0; j < 4; j++) { float2 f = __half22float2(hh[j]); qf[v * 8 + 2 * j] = f.x; qf[v * 8 + 2 * j + 1] = f.y; }
        }
    }
    const float alpha = (float)(1.0 / sqrt((double)HS));
    const size_t head_off = (size_t)(h / kv_mul) * HS + lane8 * PER;

    float m = -CUDART_INF_F, l = 0.f;
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) acc[i] = 0.f;

    // the trip count is the same for every lane of the block (shuffles below use the full mask)
    for (int tb = t0; tb < t1; tb += kGroups) {
        const int t = tb + grp;
        const bool valid = t < t1;
        const __half* kr = kc + (size_t)(valid ? t : t0) * kv_stride + head_off;
        const __half* vr = vc + (size_t)(valid ? t : t0) * kv_stride + head_off;
        uint4 kv4[VEC], vv4[VEC];
#pragma unroll
        for (int v = 0; v < VEC; v++) { kv4[v] = *reinterpret_cast<const uint4*>(kr + v * 8); vv4[v] = *reinterpret_cast<const uint4*>(vr + v * 8); }
        float s = 0.f;
#pragma unroll
        for (int v = 0; v < VEC; v++) {
            const __half2* hh = reinterpret_cast<const __half2*>(&kv4[v]);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 f = __half22float2(hh[j]);
                s = fmaf(f.x, qf[v * 8 + 2 * j], s);
                s = fmaf(f.y, qf[v * 8 + 2 * j + 1], s);
            }
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (valid) {
            s = __half2float(__float2half(s * alpha));  // the reference stores scores as fp16 (gpu_kernels.h:171-175)
            const float mn = fmaxf(m, s);
            const float corr = expf(m - mn);            // 0 on the first position (m = -inf)
            const float p = expf(s - mn);
            l = l * corr + p;
#pragma unroll
            for (int v = 0; v < VEC; v++) {
                const __half2* hh = reinterpret_cast<const __half2*>(&vv4[v]);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    float2 f = __half22float2(hh[j]);
                    acc[v * 8 + 2 * j] = fmaf(p, f.x, acc[v * 8 + 2 * j] * corr);
                    acc[v * 8 + 2 * j + 1] = fmaf(p, f.y, acc[v * 8 + 2 * j + 1] * corr);
                }
            }
            m = mn;
        }
    }

    if (lane8 == 0) { sm_m[grp] = m; sm_l[grp] = l; }
#pragma unroll
    for (int i = 0; i < PER; i++) sm_acc[grp][lane8 * PER + i] = acc[i];
    __syncthreads();

    float M = -CUDART_INF_F;
#pragma unroll
    for (int g = 0; g < kGroups; g++) M = fmaxf(M, sm_m[g]);
    float* out = scratch + ((size_t)h * nsplit + split) * (HS + 2);
    if (threadIdx.x == 0) {
        float L = 0.f;
        for (int g = 0; g < kGroups; g++) L += (sm_m[g] == -CUDART_INF_F) ? 0.f : sm_l[g] * expf(sm_m[g] - M);
        out[0] = M;
        out[1] = L;
    }
    for (int d = threadIdx.x; d < HS; d += kAttnThreads) {
        float a = 0.f;
#pragma unroll
        for (int g = 0; g < kGroups; g++) a += (sm_m[g] == -CUDART_INF_F) ? 0.f : sm_acc[g][d] * expf(sm_m[g] - M);
        out[2 + d] = a;
    }
}

__global__ void attn_merge_kernel(__half* output, const float* scratch, int nsplit, int head_size) {
    griddep_wait();
    griddep_launch_dependents();
    const int h = blockIdx.x;
    const float* base = scratch + (size_t)h * nsplit * (head_size + 2);
    float M = -CUDART_INF_F;
    for (int s = 0; s < nsplit; s++) M = fmaxf(M, base[(size_t)s * (head_size + 2)]);
    float L = 0.f;
    for (int s = 0; s < nsplit; s++) {
        const float ms = base[(size_t)s * (head_size + 2)];
        if (ms != -CUDART_INF_F) L += base[(size_t)s * (head_size + 2) + 1] * expf(ms - M);
    }
    for (int d = threadIdx.x; d < head_size; d += blockDim.x) {
        float a = 0.f;
        for (int s = 0; s < nsplit; s++) {
            const float ms = base[(size_t)s * (head_size + 2)];
            if (ms != -CUDART_INF_F) a += base[(size_t)s * (head_size + 2) + 2 + d] * expf(ms - M);
        }
        output[(size_t)h * head_size + d] = __float2half(a / L);
    }
}

}  // namespace

extern "C" size_t q4_attention_scratch_bytes(int num_heads, int head_size) {
    if (num_heads <= 0 || head_size <= 0) return 0;
    return (size_t)num_heads * attn_splits(num_heads) * (head_size + 2) * sizeof(float);
}

// Launches the two passes with caller-owned scratch.
static int q4_attention_launch(cudaStream_t s, uint16_t* output, const uint16_t* q, const uint16_t* key_cache, const uint16_t* value_cache,
                        float* scratch, int num_heads, int head_size, int kv_mul, const int* pPos) {
    const int nsplit = attn_splits(num_heads);
    const int kv_stride = num_heads * head_size / kv_mul;
    Q4Launch L(dim3(nsplit, num_heads), dim3(kAttnThreads), 0, s);
    const __half* qh = (const __half*)q;
    const __half* kc = (const __half*)key_cache;
    const __half* vc = (const __half*)value_cache;
    switch (head_size) {
        case 64: Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, attn_partial_kernel<64>, scratch, qh, kc, vc, kv_mul, kv_stride, pPos)); break;
        case 128: Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, attn_partial_kernel<128>, scratch, qh, kc, vc, kv_mul, kv_stride, pPos)); break;
        case 256: Q4_CUDA_TRY(cudaLaunchKernelEx(&L.cfg, attn_partial_kernel<256>, scratch, qh, kc, vc, kv_mul, kv_stride, pPos)); break;
        default: return Q4_ERR_UNSUPPORTED_SIZE;
    }
    Q4Launch L2(dim3(num_heads), dim3(head_size < 128 ? 64 : 128), 0, s);
    Q4_CUDA_TRY(cudaLaunchKernelEx(&L2.cfg, attn_merge_kernel, (__half*)output, (const float*)scratch, nsplit, head_size));
    return Q4_OK;
}

extern "C" int q4_attention(void* stream, uint16_t* output, const uint16_t* q, const uint16_t* key_cache, const uint16_t* value_cache,
                            void* scratch, int num_heads, int head_size, int kv_mul, int max_seq_len, const int* pPos) {
    (void)max_seq_len;  // the reference sizes its grid with it (llama2_q4.cu:415); this grid is length-independent
    if (!output || !q || !key_cache || !value_cache || !scratch || !pPos || num_heads <= 0 || kv_mul <= 0 || num_heads % kv_mul)
        return Q4_ERR_INVALID;
    if (head_size > kMaxHeadSize) return Q4_ERR_UNSUPPORTED_SIZE;
    return q4_attention_launch((cudaStream_t)stream, output, q, key_cache, value_cache, (float*)scratch, num_heads, head_size, kv_mul, pPos);
}

// ------------------------------------------------------------------------------------------------------------
// Attention without a caller-provided scratch buffer.
//
// Some hosts of this library hand it nothing but the reference's own buffers and may not allocate device memory
// themselves: a serving process whose device memory is fully committed to weights and KV cache at start-up (the
// reference allocates everything once, in malloc_run_state), or a plugin that only receives raw pointers from
// the runtime that owns the memory. For them the split partial results live in a fixed array inside the
// library's own device image instead. Every GPU that loads the library carries the array until the process ends.
// ------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_attention_static_scratch[Q4_ATTENTION_STATIC_MAX_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
float* g_static_ptr[kMaxDevices];  // device address of the array, per device (the symbol itself is not an address on the host)

int static_scratch(float** out) {
    int dev = 0;
    Q4_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return Q4_ERR_LIMIT;
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        Q4_CUDA_TRY(cudaGetSymbolAddress(&p, g_attention_static_scratch));
        g_static_ptr[dev] = reinterpret_cast<float*>(p);
    }
    *out = g_static_ptr[dev];
    return Q4_OK;
}
}  // namespace

extern "C" int q4_attention_static(void* stream, uint16_t* output, const uint16_t* q, const uint16_t* key_cache,
                                   const uint16_t* value_cache, int num_heads, int head_size, int kv_mul, int max_seq_len, const int* pPos) {
    (void)max_seq_len;
    if (!output || !q || !key_cache || !value_cache || !pPos || num_heads <= 0 || kv_mul <= 0 || num_heads % kv_mul) return Q4_ERR_INVALID;
    if (head_size > kMaxHeadSize) return Q4_ERR_UNSUPPORTED_SIZE;
    if (q4_attention_scratch_bytes(num_heads, head_size) > (size_t)Q4_ATTENTION_STATIC_MAX_BYTES) {
        fprintf(stderr, "q4_attention_static: %d heads of size %d need %zu bytes of scratch, the built-in array holds %d\n", num_heads, head_size,
                q4_attention_scratch_bytes(num_heads, head_size), Q4_ATTENTION_STATIC_MAX_BYTES);
        return Q4_ERR_LIMIT;
    }
    float* scratch = nullptr;
    if (int e = static_scratch(&scratch)) return e;
    return q4_attention_launch((cudaStream_t)stream, output, q, key_cache, value_cache, scratch, num_heads, head_size, kv_mul, pPos);
}
