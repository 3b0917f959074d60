// Temperature / top-p sampling of the next token: the non-greedy branch of sample() (sampler.h:85-115) with its kernels
// softmax_logits_kernel and sample_top_p_kernel (gpu_kernels.h:507-592) and the radix sort / prefix sum between them.
//
// One launch of one CTA instead of four launches. Semantics kept from the reference:
//   val = fp16(logit / temperature); e = fp16(exp(val - max)); p = fp16(e / sum(exp, unrounded fp32)); (written back in place)
//   0 < topp < 1: order = p descending (equal p: lower index first, the radix sort is stable), threshold = coin * topp
//   otherwise   : order = index order, threshold = coin
//   token = first element in that order whose inclusive prefix sum of p reaches the threshold; the last one if none does.
// The reference accumulates the prefix sum in fp16 in whatever order the device-wide scan takes. Here the sum is EXACT:
// every fp16 probability is an integer multiple of 2^-24, so prefix sums are 64-bit integers and the result does not
// depend on any summation order. The sorted order is never materialised: two histogram passes over the fp16 bit pattern
// (high byte, then low byte) find the probability value at which the prefix crosses the threshold, and a count over the
// ties in index order finds the element.
#include <math_constants.h>

#include "q4_common.cuh"

namespace {

constexpr int kT = 1024;

__device__ __forceinline__ unsigned long long prob_units(unsigned short h) {   // fp16 in [0, 1] -> multiples of 2^-24
    const unsigned e = (h >> 10) & 31u, mnt = h & 1023u;
    return e == 0 ? (unsigned long long)mnt : (unsigned long long)(1024u + mnt) << (e - 1);
}

// Fixed-order block reductions (thread-strided partials, xor tree 16..1 inside a warp, the same tree over the 32 warp
// partials): the CPU oracle repeats exactly this order.
__device__ __forceinline__ float block_max(float v, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = sh[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = sh[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    __syncthreads();
    return r;
}

// Exclusive prefix over the threads' values (64-bit), Hillis-Steele in shared memory. Returns the exclusive prefix of
// this thread; *total gets the sum over the block.
__device__ __forceinline__ unsigned long long block_exclusive_scan(unsigned long long v, unsigned long long* sh, unsigned long long* total) {
    const int t = threadIdx.x;
    sh[t] = v;
    __syncthreads();
    for (int o = 1; o < kT; o <<= 1) {
        const unsigned long long add = t >= o ? sh[t - o] : 0ull;
        __syncthreads();
        sh[t] += add;
        __syncthreads();
    }
    const unsigned long long incl = sh[t];
    *total = sh[kT - 1];
    __syncthreads();
    return incl - v;
}

__global__ void __launch_bounds__(kT) sample_topp_kernel(__half* __restrict__ logits, int n, float temperature, float topp, float coin, int* result,
                                                        volatile int* pPos, int* pPosGpu) {
    __shared__ float shf[32];
    __shared__ unsigned long long sh64[kT];
    __shared__ unsigned long long hist[256];
    __shared__ int s_found;
    __shared__ unsigned s_last;
    __shared__ int s_bin;
    __shared__ unsigned long long s_before;
    const int t = threadIdx.x;

    // ---- softmax with temperature (softmax_logits_kernel) ----
    float mx = -CUDART_INF_F;
    for (int i = t; i < n; i += kT) {
        float val = __half2float(logits[i]);
        val /= temperature;
        const __half hv = __float2half(val);
        logits[i] = hv;
        mx = fmaxf(mx, __half2float(hv));
    }
    mx = block_max(mx, shf);
    float sum = 0.f;
    for (int i = t; i < n; i += kT) {
        const float v = expf(__half2float(logits[i]) - mx);
        logits[i] = __float2half(v);
        sum += v;
    }
    sum = block_sum(sum, shf);
    for (int i = t; i < n; i += kT) logits[i] = __float2half(__half2float(logits[i]) / sum);
    __syncthreads();

    const unsigned short* pb = reinterpret_cast<const unsigned short*>(logits);
    const bool sorted = topp > 0.f && topp < 1.f;
    const float threshold = sorted ? coin * topp : coin;
    // prefix >= threshold  <=>  integer prefix >= ceil(threshold * 2^24). A threshold <= 0 selects the first element of
    // the order whatever its probability (`prefix >= 0` holds at once): index 0 in index order; in sorted order the
    // largest probability, which is what need = 1 finds.
    const double td = ceil((double)threshold * 16777216.0);
    const bool take_first = !(threshold > 0.f);
    unsigned long long need = td <= 1.0 ? 1ull : (td >= 9.0e18 ? ~0ull : (unsigned long long)td);

    const int chunk = (n + kT - 1) / kT;
    const int i0 = min(n, t * chunk), i1 = min(n, i0 + chunk);
    if (t == 0) { s_found = 0x7fffffff; s_last = 0xFFFFFFFFu; }
    __syncthreads();
    int token = -1;

    if (!sorted) {
        // ---- index order: blocked exclusive scan, the owning thread walks its chunk ----
        unsigned long long local = 0;
        for (int i = i0; i < i1; i++) local += prob_units(pb[i]);
        unsigned long long total;
        const unsigned long long excl = block_exclusive_scan(local, sh64, &total);
        if (excl < need && excl + local >= need) {
            unsigned long long c = excl;
            for (int i = i0; i < i1; i++) {
                c += prob_units(pb[i]);
                if (c >= need) { atomicMin(&s_found, i); break; }
            }
        }
        __syncthreads();
        token = take_first ? 0 : (s_found == 0x7fffffff ? n - 1 : s_found);
    } else {
        // ---- descending probability: find the fp16 value at which the prefix crosses, high byte then low byte ----
        unsigned long long before = 0;
        int key = -1;
        for (int level = 0; level < 2; level++) {
            if (t < 256) hist[t] = 0;
            __syncthreads();
            for (int i = t; i < n; i += kT) {
                const unsigned short k = pb[i];
                if (level == 0) atomicAdd(&hist[k >> 8], prob_units(k));
                else if ((k >> 8) == key) atomicAdd(&hist[k & 255], prob_units(k));
            }
            __syncthreads();
            if (t == 0) {
                unsigned long long c = level == 0 ? 0ull : s_before;
                int found = -1;
                for (int b = 255; b >= 0; b--) {
                    if (hist[b] != 0 && c + hist[b] >= need) { found = b; break; }
                    c += hist[b];
                }
                s_bin = found;
                s_before = c;
            }
            __syncthreads();
            if (s_bin < 0) { key = -1; break; }
            key = level == 0 ? s_bin : (key << 8) | s_bin;
            before = s_before;
        }
        if (key < 0) {
            // the threshold is never reached: the last element of the order = lowest probability, highest index among equals
            unsigned best = 0xFFFFFFFFu;   // (key << 18 | ~index) minimised: lowest key (< 2^14), then highest index (n <= 2^18)
            for (int i = t; i < n; i += kT) best = min(best, ((unsigned)pb[i] << 18) | (unsigned)(0x3FFFF - i));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) best = min(best, __shfl_xor_sync(0xffffffffu, best, o));
            if ((t & 31) == 0) atomicMin(&s_last, best);
            __syncthreads();
            token = 0x3FFFF - (int)(s_last & 0x3FFFFu);
        } else {
            // the k-th element (index order) among those whose probability has exactly this bit pattern
            const unsigned long long pv = prob_units((unsigned short)key);
            const unsigned long long kth = (need - before + pv - 1) / pv;   // 1-based, >= 1
            unsigned long long cnt = 0;
            for (int i = i0; i < i1; i++) cnt += pb[i] == (unsigned short)key;
            unsigned long long total;
            const unsigned long long excl = block_exclusive_scan(cnt, sh64, &total);
            if (excl < kth && excl + cnt >= kth) {
                unsigned long long c = excl;
                for (int i = i0; i < i1; i++) {
                    if (pb[i] == (unsigned short)key && ++c == kth) { atomicMin(&s_found, i); break; }
                }
            }
            __syncthreads();
            token = s_found == 0x7fffffff ? n - 1 : s_found;
        }
    }
    if (t == 0) {   // hand-off as in sample_top_p_kernel (gpu_kernels.h:583-591)
        int token_pos = *pPos;
        token_pos++;
        result[token_pos] = token;
        *pPos = token_pos;
        *pPosGpu = token_pos;
    }
}

}  // namespace

// xorshift* of the reference (sampler.h:66-75): the host draws one coin per forward call.
extern "C" unsigned int q4_random_u32(unsigned long long* state) {
    *state ^= *state >> 12;
    *state ^= *state << 25;
    *state ^= *state >> 27;
    return (unsigned int)((*state * 0x2545F4914F6CDD1Dull) >> 32);
}
extern "C" float q4_random_f32(unsigned long long* state) { return (q4_random_u32(state) >> 8) / 16777216.0f; }

extern "C" int q4_sample_topp(void* stream, uint16_t* logits, int n, float temperature, float topp, float coin, int* tokens_pinned,
                              volatile int* pos_pinned, int* pos_dev) {
    if (!logits || !tokens_pinned || !pos_pinned || !pos_dev || n <= 0 || n > (1 << 18) || !(temperature > 0.f)) return Q4_ERR_INVALID;
    sample_topp_kernel<<<1, kT, 0, (cudaStream_t)stream>>>((__half*)logits, n, temperature, topp, coin, tokens_pinned, pos_pinned, pos_dev);
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}
