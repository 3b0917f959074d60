// Many rows through the network at once: prompt prefill (the rows are consecutive positions of one sequence) and batched
// decode (the rows are the current positions of several sequences). The reference has neither: it pushes a prompt
// through the batch-1 schedule token by token (llama2_q4.cu:710-735) and holds one sequence (RunState, common.h:62-78).
// The schedule per layer is run_llama_network's (llama2_q4.cu:444-524) with every op widened to rows:
//   RMSNorm -> Q, K, V (W4 dequant-GEMM on tcgen05, q4_gemm.cu) -> RoPE, K/V rows into the cache -> causal attention
//   -> O projection + residual [-> all-reduce] -> RMSNorm -> gate, up (GEMM) -> SiLU * up -> down + residual [-> all-reduce]
// with the rounding points of the batch-1 path (fp16 activations between ops, fp32 inside). A row is (sequence, position):
// the K/V cache row it writes and the range of cached positions it attends to follow from that pair, so one set of
// kernels serves both uses. The small row-wise kernels here are bandwidth-trivial next to the GEMMs and are kept simple.
#include <math_constants.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>

#include "q4_model.h"

namespace {

constexpr int kRowThreads = 256;

// Every kernel of this file starts with griddepcontrol.wait + launch_dependents, so it may be launched with programmatic
// stream serialisation: its successor (often a weight-streaming kernel whose first loads do not depend on it) then begins
// its prologue while this one runs, and waits for this one's completion before it touches anything produced here. The
// batched-decode step (a handful of rows, latency-bound small kernels) is launched that way. A prompt's rows are not:
// with hundreds of rows the overlap buys nothing measurable, and with the rotation and attention kernels launched that way
// two runs of the same 512-token prompt did not always give the same bits on this GPU and driver (about one run in ten
// differed in the last bits of a few logits; cause not found), so those launches keep plain stream order.
template <typename... KArgs, typename... Args>
cudaError_t launch_rows(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    Q4Launch L(grid, block, smem, s, overlap);
    return cudaLaunchKernelEx(&L.cfg, kernel, KArgs(args)...);
}

// ids of the rows' tokens: tok_base[seq * tok_stride + pos]
__global__ void embed_rows_kernel(__half* x, const __half* table, int dim, const int* tok_base, long long tok_stride, const int* row_seq, const int* row_pos,
                                  int vocab) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    const int m = blockIdx.x;
    int token = tok_base[(long long)row_seq[m] * tok_stride + row_pos[m]];
    if (token < 0 || token >= vocab) token = 0;   // (ids are validated on the host; a generated id is always in range)
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)token * dim);
    uint4* dst = reinterpret_cast<uint4*>(x + (size_t)m * dim);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
}

// rmsnorm_kernel (gpu_kernels.h:72-105) per row: o = x * (rsqrt(mean(x^2) + 1e-5) * w), fp32 inside, fp16 out.
// size % 8 == 0; a thread keeps up to four 8-element pieces of the row in registers between the two passes.
__device__ __forceinline__ float sumsq8(const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 f = __half22float2(h[j]);
        s += f.x * f.x + f.y * f.y;
    }
    return s;
}
__device__ __forceinline__ uint4 scale8(const uint4& v, const uint4& w, float r) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    const __half2* wh = reinterpret_cast<const __half2*>(&w);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 f = __half22float2(h[j]), g = __half22float2(wh[j]);
        oh[j] = __floats2half2_rn(f.x * (r * g.x), f.y * (r * g.y));
    }
    return o;
}
__global__ void __launch_bounds__(kRowThreads) rmsnorm_rows_kernel(__half* o, const __half* x, const __half* w, int size) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    __shared__ float red[kRowThreads / 32];
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)blockIdx.x * size);
    uint4* orow = reinterpret_cast<uint4*>(o + (size_t)blockIdx.x * size);
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    const int nvec = size / 8;
    constexpr int kKeep = 4;
    uint4 v[kKeep];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kKeep; c++) {
        const int i = threadIdx.x + c * kRowThreads;
        if (i < nvec) { v[c] = xr[i]; ss += sumsq8(v[c]); }
    }
    for (int i = threadIdx.x + kKeep * kRowThreads; i < nvec; i += kRowThreads) ss += sumsq8(xr[i]);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kRowThreads / 32; i++) tot += red[i];
    tot /= size;
    tot += 1e-5f;
    tot = 1.0f / sqrtf(tot);
#pragma unroll
    for (int c = 0; c < kKeep; c++) {
        const int i = threadIdx.x + c * kRowThreads;
        if (i < nvec) orow[i] = scale8(v[c], wv[i], tot);
    }
    for (int i = threadIdx.x + kKeep * kRowThreads; i < nvec; i += kRowThreads) orow[i] = scale8(xr[i], wv[i], tot);
}

// RoPERotation_kernel (gpu_kernels.h:340-363) per row, and the row's K and V into the cache: query heads are rotated in place,
// the key heads are rotated on their way into cache row `pos` of the row's sequence, the value heads are copied there.
// A block takes kRopeHeads heads (query heads first, then key/value heads) of one row: the head_size / 2 rotation angles
// depend on the position only and are computed once per block, in the reference's arithmetic (powf, cosf, sinf in fp32).
// head_size <= 256. grid (rows, ceil((heads + kv_heads) / kRopeHeads)), block 256.
constexpr int kRopeHeads = 4;
__global__ void __launch_bounds__(256) rope_store_rows_kernel(__half* q, const __half* k, const __half* v, int ldq, int ldkv, __half* kc, __half* vc, int n_heads,
                                                              int n_kv_heads, int head_size, const int* row_seq, const int* row_pos, long long seq_stride, long long loff,
                                                              float theta) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    __shared__ float2 table[128];
    const int m = blockIdx.x;
    const int pos = row_pos[m];
    const int half_hs = head_size / 2;
    for (int i = threadIdx.x; i < half_hs; i += blockDim.x) table[i] = rope_cos_sin(pos, i, head_size, theta);
    __syncthreads();
    __half* qr = q + (size_t)m * ldq;      // ldq, ldkv: halfs between rows of q and of k / v (they may be slices of one wider buffer)
    const size_t src0 = (size_t)m * ldkv;
    const size_t dst0 = (size_t)row_seq[m] * seq_stride + loff + (size_t)pos * n_kv_heads * head_size;
    const int h_first = blockIdx.y * kRopeHeads, h_end = min(h_first + kRopeHeads, n_heads + n_kv_heads);
    for (int e = threadIdx.x; e < (h_end - h_first) * half_hs; e += blockDim.x) {
        const int hh = h_first + e / half_hs, i = e % half_hs;
        if (hh < n_heads) {
            __half* p = qr + (size_t)hh * head_size;
            rope_rotate(p + i, p + i + half_hs, p + i, p + i + half_hs, table[i]);
        } else {
            const int h = hh - n_heads;
            const size_t src = src0 + (size_t)h * head_size, dst = dst0 + (size_t)h * head_size;
            rope_rotate(k + src + i, k + src + i + half_hs, kc + dst + i, kc + dst + i + half_hs, table[i]);
            vc[dst + i] = v[src + i];
            vc[dst + i + half_hs] = v[src + i + half_hs];
        }
    }
}

// MultiHeadAttention (llama2_q4.cu:410-427) for one (row, head): the query attends to cached positions 0 .. pos of its own
// sequence (its own K/V row was stored by the RoPE kernel before). Scores are rounded to fp16 as the reference stores them
// (gpu_kernels.h:171-175); the softmax runs online in fp32 over the keys a warp visits, the warps are merged at the end.
// A warp takes four keys per round (keys 4 (warp + 8 i) .. + 3) and issues their eight K/V loads together, so a round costs
// one memory latency, not eight. head_size 128: a lane holds four dims. grid (heads, rows), block 256.
constexpr int kAttWarps = 8, kAttKeys = 4;
__global__ void __launch_bounds__(kAttWarps * 32) attention_rows_kernel(__half* out, const __half* q, int ldq, const __half* kc, const __half* vc, int n_heads, int kv_mul,
                                                                       const int* row_seq, const int* row_pos, long long seq_stride, long long loff, int kv_n) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    constexpr int HS = 128;
    const int h = blockIdx.x, m = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int T = row_pos[m] + 1;
    const __half* kb = kc + (size_t)row_seq[m] * seq_stride + loff + (size_t)(h / kv_mul) * HS + lane * 4;
    const __half* vb = vc + (size_t)row_seq[m] * seq_stride + loff + (size_t)(h / kv_mul) * HS + lane * 4;
    float qf[4];
    {
        const uint2 qv = *reinterpret_cast<const uint2*>(q + (size_t)m * ldq + (size_t)h * HS + lane * 4);
        const __half2* qh = reinterpret_cast<const __half2*>(&qv);
        qf[0] = __low2float(qh[0]); qf[1] = __high2float(qh[0]); qf[2] = __low2float(qh[1]); qf[3] = __high2float(qh[1]);
    }
    const float alpha = (float)(1.0 / sqrt((double)HS));
    float mx = -CUDART_INF_F, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t0 = warp * kAttKeys; t0 < T; t0 += kAttWarps * kAttKeys) {
        uint2 kv[kAttKeys], vv[kAttKeys];
#pragma unroll
        for (int u = 0; u < kAttKeys; u++) {
            const int t = min(t0 + u, T - 1);   // a round's tail re-reads the last key; its weight is forced to zero below
            kv[u] = *reinterpret_cast<const uint2*>(kb + (size_t)t * kv_n);
            vv[u] = *reinterpret_cast<const uint2*>(vb + (size_t)t * kv_n);
        }
        float sc[kAttKeys];
#pragma unroll
        for (int u = 0; u < kAttKeys; u++) {
            const __half2* kh = reinterpret_cast<const __half2*>(&kv[u]);
            sc[u] = qf[0] * __low2float(kh[0]) + qf[1] * __high2float(kh[0]) + qf[2] * __low2float(kh[1]) + qf[3] * __high2float(kh[1]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < kAttKeys; u++) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
        float mn = mx;
#pragma unroll
        for (int u = 0; u < kAttKeys; u++) {
            sc[u] = t0 + u < T ? __half2float(__float2half(sc[u] * alpha)) : -CUDART_INF_F;
            mn = fmaxf(mn, sc[u]);
        }
        const float corr = expf(mx - mn);   // key t0 itself is always valid, so mn is finite
        l *= corr;
#pragma unroll
        for (int j = 0; j < 4; j++) acc[j] *= corr;
#pragma unroll
        for (int u = 0; u < kAttKeys; u++) {
            const float pr = expf(sc[u] - mn);
            const __half2* vh = reinterpret_cast<const __half2*>(&vv[u]);
            l += pr;
            acc[0] += pr * __low2float(vh[0]);
            acc[1] += pr * __high2float(vh[0]);
            acc[2] += pr * __low2float(vh[1]);
            acc[3] += pr * __high2float(vh[1]);
        }
        mx = mn;
    }
    __shared__ float s_m[kAttWarps], s_l[kAttWarps], s_acc[kAttWarps][HS];
    if (lane == 0) { s_m[warp] = mx; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < 4; j++) s_acc[warp][lane * 4 + j] = acc[j];
    __syncthreads();
    if (threadIdx.x < HS) {
        float M = -CUDART_INF_F;
        for (int w = 0; w < kAttWarps; w++) M = fmaxf(M, s_m[w]);
        float a = 0.f, L = 0.f;
        for (int w = 0; w < kAttWarps; w++) {
            if (s_m[w] != -CUDART_INF_F) {
                const float e = expf(s_m[w] - M);
                a += s_acc[w][threadIdx.x] * e;
                L += s_l[w] * e;
            }
        }
        out[((size_t)m * n_heads + h) * HS + threadIdx.x] = __float2half(L > 0.f ? a / L : 0.f);
    }
}

// ---- causal attention of a prompt (rows = consecutive positions of one sequence) on the tensor cores ----
// The (row, head) kernel above re-reads the whole K/V history once per row; for a prompt that is rows^2 / 2 cache rows per
// head. Here a CTA takes 64 consecutive rows of one head (a warp: 16 of them) and walks the keys in chunks of 64 staged in
// shared memory, so a cache row is read once per 64 query rows. S = Q K^T and O += P V run as mma.sync m16n8k16 (fp16 in,
// fp32 out); the scores are scaled and rounded to fp16 exactly where MultiHeadAttention stores them (gpu_kernels.h:171-175),
// the softmax is the online form in fp32, P is rounded to fp16 for the second product (the reference's att buffer is fp16
// too). head_size 128. Keys beyond the last row's position are zero-filled in shared memory and masked.
constexpr int kAtRows = 64, kAtKeys = 64, kAtLd = 136;   // 136 halfs = 272 B between rows: conflict-free fragment loads

__device__ __forceinline__ void mma_f16(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// grid (heads, ceil(n / 64)), block 128. kc / vc point at this layer's cache rows of the sequence (position 0).
__global__ void __launch_bounds__(128) attention_prefill_kernel(__half* out, const __half* q, int ldq, const __half* kc, const __half* vc, int n_heads, int kv_mul,
                                                                int n, int pos0, int kv_n) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    constexpr int HS = 128;
    __shared__ __align__(16) __half sK[kAtKeys][kAtLd];
    __shared__ __align__(16) __half sV[kAtKeys][kAtLd];
    const int h = blockIdx.x, m0 = blockIdx.y * kAtRows;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row_a = m0 + warp * 16 + g, row_b = row_a + 8;          // this thread's two query rows
    const int last_pos = pos0 + n - 1;                                // newest cache row that is valid
    const int pos_a = min(pos0 + row_a, last_pos), pos_b = min(pos0 + row_b, last_pos);
    const int warp_last = min(pos0 + m0 + warp * 16 + 15, last_pos);  // newest key any row of this warp attends to
    const int cta_last = min(pos0 + m0 + kAtRows - 1, last_pos);
    const size_t head_off = (size_t)(h / kv_mul) * HS;

    // Q fragments: 8 k-steps of 16 dims; rows past the prompt read as zero
    uint32_t qa[8][4];
    {
        const __half* qa_p = q + (size_t)row_a * ldq + (size_t)h * HS;
        const __half* qb_p = q + (size_t)row_b * ldq + (size_t)h * HS;
#pragma unroll
        for (int s = 0; s < 8; s++) {
            qa[s][0] = row_a < n ? *reinterpret_cast<const uint32_t*>(qa_p + 16 * s + 2 * t) : 0u;
            qa[s][1] = row_b < n ? *reinterpret_cast<const uint32_t*>(qb_p + 16 * s + 2 * t) : 0u;
            qa[s][2] = row_a < n ? *reinterpret_cast<const uint32_t*>(qa_p + 16 * s + 2 * t + 8) : 0u;
            qa[s][3] = row_b < n ? *reinterpret_cast<const uint32_t*>(qb_p + 16 * s + 2 * t + 8) : 0u;
        }
    }
    const float alpha = (float)(1.0 / sqrt((double)HS));
    float o[16][4];
#pragma unroll
    for (int d = 0; d < 16; d++) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float mx_a = -CUDART_INF_F, mx_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;

    for (int t0 = 0; t0 <= cta_last; t0 += kAtKeys) {
        __syncthreads();   // the previous chunk is consumed
        for (int i = threadIdx.x; i < kAtKeys * (HS / 8); i += 128) {
            const int r = i >> 4, c = (i & 15) * 8, key = t0 + r;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (key <= cta_last) {
                kv = *reinterpret_cast<const uint4*>(kc + (size_t)key * kv_n + head_off + c);
                vv = *reinterpret_cast<const uint4*>(vc + (size_t)key * kv_n + head_off + c);
            }
            *reinterpret_cast<uint4*>(&sK[r][c]) = kv;
            *reinterpret_cast<uint4*>(&sV[r][c]) = vv;
        }
        __syncthreads();
        if (t0 > warp_last) continue;   // warp-uniform: nothing of this chunk is visible to the warp's rows

        // S = Q K^T for 16 rows x 64 keys
        float sc[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&sK[8 * j + g][16 * s + 2 * t]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&sK[8 * j + g][16 * s + 2 * t + 8]);
                mma_f16(sc[j], qa[s], b0, b1);
            }
        }
        // scale, round to fp16 as the reference stores the scores, mask, chunk maxima
        float cm_a = -CUDART_INF_F, cm_b = -CUDART_INF_F;
#pragma unroll
        for (int j = 0; j < 8; j++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = t0 + 8 * j + 2 * t + (e & 1);
                const int pos = (e < 2) ? pos_a : pos_b;
                float v = __half2float(__float2half(sc[j][e] * alpha));
                v = key <= pos ? v : -CUDART_INF_F;
                sc[j][e] = v;
                if (e < 2) cm_a = fmaxf(cm_a, v); else cm_b = fmaxf(cm_b, v);
            }
        }
        cm_a = fmaxf(cm_a, __shfl_xor_sync(0xffffffffu, cm_a, 1));
        cm_a = fmaxf(cm_a, __shfl_xor_sync(0xffffffffu, cm_a, 2));
        cm_b = fmaxf(cm_b, __shfl_xor_sync(0xffffffffu, cm_b, 1));
        cm_b = fmaxf(cm_b, __shfl_xor_sync(0xffffffffu, cm_b, 2));
        // key 0 is visible to every row, so after the first chunk the running maxima are finite
        const float nm_a = fmaxf(mx_a, cm_a), nm_b = fmaxf(mx_b, cm_b);
        const float corr_a = __expf(mx_a - nm_a), corr_b = __expf(mx_b - nm_b);
        mx_a = nm_a; mx_b = nm_b;
        float sum_a = 0.f, sum_b = 0.f;
        uint32_t pa[4][4];   // P as A fragments: k-step jj covers keys 16 jj .. 16 jj + 15
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const __half2 p01 = __floats2half2_rn(__expf(sc[j][0] - nm_a), __expf(sc[j][1] - nm_a));
            const __half2 p23 = __floats2half2_rn(__expf(sc[j][2] - nm_b), __expf(sc[j][3] - nm_b));
            sum_a += __low2float(p01) + __high2float(p01);
            sum_b += __low2float(p23) + __high2float(p23);
            pa[j >> 1][(j & 1) * 2 + 0] = *reinterpret_cast<const uint32_t*>(&p01);
            pa[j >> 1][(j & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&p23);
        }
        l_a = l_a * corr_a + sum_a;
        l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int d = 0; d < 16; d++) { o[d][0] *= corr_a; o[d][1] *= corr_a; o[d][2] *= corr_b; o[d][3] *= corr_b; }
        // O += P V: V fragments through ldmatrix.trans (V is [key][dim]; the product wants keys along k)
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
#pragma unroll
            for (int d = 0; d < 16; d += 2) {
                uint32_t v0, v1, v2, v3;
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&sV[16 * jj + (lane & 15)][8 * d + 8 * (lane >> 4)]);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(addr));
                mma_f16(o[d], pa[jj], v0, v1);
                mma_f16(o[d + 1], pa[jj], v2, v3);
            }
        }
    }
    // the quad's partial row sums, then O / l
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
#pragma unroll
    for (int d = 0; d < 16; d++) {
        if (row_a < n) *reinterpret_cast<uint32_t*>(out + ((size_t)row_a * n_heads + h) * HS + 8 * d + 2 * t) = pack_h2(o[d][0] * inv_a, o[d][1] * inv_a);
        if (row_b < n) *reinterpret_cast<uint32_t*>(out + ((size_t)row_b * n_heads + h) * HS + 8 * d + 2 * t) = pack_h2(o[d][2] * inv_b, o[d][3] * inv_b);
    }
}

// ffn_matvec_silu's epilogue (gpu_kernels.h:278-281) on the result of the fused gate|up GEMM: row m of gu holds the hid gate
// values and then the hid up values; h[m][j] = silu(gate) * up in fp32, fp16 out. hid % 8 == 0.
__global__ void silu_mul_rows_kernel(__half* h, const __half* gu, int hid, int rows) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    const int per_row = hid / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < (size_t)rows * per_row; i += (size_t)gridDim.x * blockDim.x) {
        const size_t m = i / per_row, j = i - m * per_row;
        const uint4 gv = reinterpret_cast<const uint4*>(gu + m * 2 * hid)[j], uv = reinterpret_cast<const uint4*>(gu + m * 2 * hid + hid)[j];
        const __half2* gh = reinterpret_cast<const __half2*>(&gv);
        const __half2* uh = reinterpret_cast<const __half2*>(&uv);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const float2 g = __half22float2(gh[jj]), u = __half22float2(uh[jj]);
            float a = g.x, b = g.y;
            a *= 1.0f / (1.0f + expf(-a));
            b *= 1.0f / (1.0f + expf(-b));
            oh[jj] = __floats2half2_rn(a * u.x, b * u.y);
        }
        reinterpret_cast<uint4*>(h + m * hid)[j] = o;
    }
}

// x = y + x * scale: the residual of matmul(QWeight)'s accum form (gpu_kernels.h:237-238) applied to a GEMM result that
// was written without it (the GEMM's own residual epilogue reads x element by element behind the tile's fp32 sums, which
// costs more than this pass over two small matrices). fp32 inside, rounded once. n % 8 == 0.
__global__ void add_residual_rows_kernel(__half* x, const __half* y, float scale, size_t n) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n / 8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 xv = reinterpret_cast<const uint4*>(x)[i], yv = reinterpret_cast<const uint4*>(y)[i];
        const __half2* xh = reinterpret_cast<const __half2*>(&xv);
        const __half2* yh = reinterpret_cast<const __half2*>(&yv);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 a = __half22float2(xh[j]), b = __half22float2(yh[j]);
            oh[j] = __floats2half2_rn(b.x + a.x * scale, b.y + a.y * scale);
        }
        reinterpret_cast<uint4*>(x)[i] = o;
    }
}

// both position words (device, pinned host) to `pos`, in stream order
__global__ void set_pos_kernel(int* pos_dev, volatile int* pos_pinned, int pos) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    *pos_dev = pos;
    *pos_pinned = pos;
}

__global__ void iota_rows_kernel(int* row_seq, int* row_pos, int n, int seq, int pos0, int step_seq) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        row_seq[i] = seq + i * step_seq;
        if (row_pos) row_pos[i] = pos0 + i;
    }
}

// mat_vec_kernel (gpu_kernels.h:117-147) for B rows of x at once: a warp takes one classifier row and B dot products, so the
// classifier is read once per step, not once per sequence. x rows sit in shared memory. B <= 16.
__global__ void __launch_bounds__(256) matvec_f16_rows_kernel(__half* y, const __half* x, const __half* w, int n, int d, int B, int y_stride) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    extern __shared__ __align__(16) __half sx[];
    for (int i = threadIdx.x; i < B * n / 8; i += blockDim.x) reinterpret_cast<uint4*>(sx)[i] = reinterpret_cast<const uint4*>(x)[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int row = blockIdx.x * 8 + warp; row < d; row += gridDim.x * 8) {
        float acc[16];
#pragma unroll
        for (int b = 0; b < 16; b++) acc[b] = 0.f;
        const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)row * n);
        for (int i = lane; i < n / 8; i += 32) {
            const uint4 wv = ldg_stream(wr + i);
            const __half2* wh = reinterpret_cast<const __half2*>(&wv);
#pragma unroll
            for (int b = 0; b < 16; b++) {
                if (b < B) {
                    const uint4 xv = reinterpret_cast<const uint4*>(sx + (size_t)b * n)[i];
                    const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 a = __half22float2(wh[j]), c = __half22float2(xh[j]);
                        acc[b] = fmaf(a.x, c.x, acc[b]);
                        acc[b] = fmaf(a.y, c.y, acc[b]);
                    }
                }
            }
        }
#pragma unroll
        for (int b = 0; b < 16; b++) {
            if (b < B) {
                const float v = warp_sum(acc[b]);
                if (lane == 0) y[(size_t)b * y_stride + row] = __float2half(v);
            }
        }
    }
}

// The same product on mma.sync m16n8k16 when the shapes allow (n % 32 == 0, d % 16 == 0): a warp takes 16 classifier rows
// and the whole of n. The k index of an MMA is only a summation label, so thread (g, t) feeds the eight consecutive
// weights it loaded with one 16-byte load (rows g and g + 8, inputs 32 c + 8 t ..) as A and the same eight inputs of batch
// row g as B - no shuffles, no shared memory; fp32 accumulation over the whole row as mat_vec_kernel does.
template <int NT>
__global__ void __launch_bounds__(256) classifier_rows_kernel(__half* y, const __half* x, const __half* w, int n, int d, int B, int y_stride) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x * 8 + warp;
    if (tile * 16 >= d) return;
    const uint4* wa = reinterpret_cast<const uint4*>(w + (size_t)(tile * 16 + g) * n) + t;
    const uint4* wb = reinterpret_cast<const uint4*>(w + (size_t)(tile * 16 + g + 8) * n) + t;
    const uint4* xr[NT];
    bool ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        ok[nt] = g + 8 * nt < B;
        xr[nt] = reinterpret_cast<const uint4*>(x + (size_t)(ok[nt] ? g + 8 * nt : 0) * n) + t;
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    const int chunks = n / 32;
    constexpr int U = 4;
    for (int c0 = 0; c0 < chunks; c0 += U) {
        uint4 a[U], b[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (c0 + u < chunks) { a[u] = ldg_stream(wa + 4 * (c0 + u)); b[u] = ldg_stream(wb + 4 * (c0 + u)); }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (c0 + u < chunks) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (ok[nt]) xv = xr[nt][4 * (c0 + u)];
                    const uint32_t A0[4] = {a[u].x, b[u].x, a[u].y, b[u].y}, A1[4] = {a[u].z, b[u].z, a[u].w, b[u].w};
                    mma_f16(acc[nt], A0, xv.x, xv.y);
                    mma_f16(acc[nt], A1, xv.z, xv.w);
                }
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = 8 * nt + 2 * t + (e & 1);
            if (row < B) y[(size_t)row * y_stride + tile * 16 + g + 8 * (e >> 1)] = __float2half(acc[nt][e]);
        }
}

// argmax per row (lowest index among equal maxima, like q4_argmax) and the hand-off of batched decode: the id becomes
// the sequence's next token when that position is past its prompt, and the sequence moves on by one position.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const __half* logits, int vocab, int* tokens, long long tok_stride, int* pos, int n_prompt) {
    griddep_wait();   // launched with programmatic stream serialisation: wait for the producer, then let the consumer's prologue start
    griddep_launch_dependents();
    __shared__ float sval[32];
    __shared__ int sidx[32];
    const int s = blockIdx.x;
    const __half* x = logits + (size_t)s * vocab;
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    const int nvec = (vocab % 8 == 0) ? vocab / 8 : 0;   // rows of a multiple of 8 halfs start 16-byte aligned
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        const uint4 v = reinterpret_cast<const uint4*>(x)[i];
        const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float f = __half2float(h[j]);
            if (f > best) { best = f; bi = i * 8 + j; }
        }
    }
    for (int i = nvec * 8 + threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = __half2float(x[i]);
        if (v > best) { best = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sval[threadIdx.x >> 5] = best; sidx[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (sval[w] > best || (sval[w] == best && sidx[w] < bi)) { best = sval[w]; bi = sidx[w]; }
        const int p = pos[s];
        if (p + 1 >= n_prompt) tokens[(long long)s * tok_stride + p + 1] = bi == 0x7fffffff ? 0 : bi;
        pos[s] = p + 1;
    }
}

}  // namespace

// ------------------------------------------------------------------------------------------------------------
// row buffers and the interleaved weight copies the GEMM prefers (built on first use)
// ------------------------------------------------------------------------------------------------------------
struct q4_rows {
    int cap = 0;   // rows the buffers hold
    __half *X = nullptr, *XB = nullptr, *Q = nullptr, *K = nullptr, *V = nullptr, *ATT = nullptr, *G = nullptr;
    __half *QKV = nullptr, *GU = nullptr;   // GEMM path: [rows][q_n + 2 kv_n] and [rows][2 hid], written by one GEMM each
    int *row_seq = nullptr, *row_pos = nullptr;
    void* ws = nullptr;
    size_t ws_bytes = 0;
    // GEMM path, per layer four matrices: q|k|v and gate|up stacked along the output axis (one launch each), o, down.
    // Interleaved copy of the packed words, and for the stacked ones a copy of zeros and scales in the same order.
    struct GemmMat { uint32_t* wi; q4_qweight w; int K, N; };
    std::vector<GemmMat> gm;     // [layer * 4 + {0 qkv, 1 o, 2 gate|up, 3 down}]
    std::vector<void*> allocs;
};

static int rows_alloc(q4_rows* r, void** p, size_t bytes) {
    Q4_CUDA_TRY(cudaMalloc(p, bytes));
    r->allocs.push_back(*p);
    return Q4_OK;
}

void q4_rows_free(q4_model* m) {
    if (!m->rows) return;
    for (void* p : m->rows->allocs) cudaFree(p);
    delete m->rows;
    m->rows = nullptr;
}

// Status word of the GEMM workspace (Q4_ERR_TIMEOUT after a bounded device-side wait ran out); the device is idle.
int q4_rows_status(q4_model* m) {
    if (!m->rows || !m->rows->ws) return Q4_OK;
    int st[2] = {0, 0};
    Q4_CUDA_TRY(cudaMemcpy(st, m->rows->ws, sizeof(st), cudaMemcpyDeviceToHost));
    if (st[0]) fprintf(stderr, "q4 prefill / batch path: a bounded device-side wait of the GEMM ran out (status %d, location 0x%x)\n", st[0], st[1]);
    return st[0];
}

// More than this many rows go through the tcgen05 GEMM, fewer through the mma.sync kernels that stream the packed weights.
constexpr int kSkinnyRows = 16;

// Buffers for up to `rows` rows (grown on demand) and, once and only when the GEMM will be used, the interleaved weight copies.
static int rows_prepare(q4_model* m, int rows) {
    if (m->column || m->head_size != 128 || (m->cfg.dim % 128) || (m->o_kc % 128) || (m->h_kc % 128)) return Q4_ERR_UNSUPPORTED_SIZE;
    if (!m->rows) m->rows = new q4_rows();
    q4_rows* r = m->rows;
    const q4_config& c = m->cfg;
    int e;
#define RTRY(expr) do { e = (expr); if (e != Q4_OK) return e; } while (0)
    if (r->gm.empty() && rows > kSkinnyRows) {
        r->gm.assign((size_t)c.n_layers * 4, q4_rows::GemmMat{});
        for (int l = 0; l < c.n_layers; l++) {
            const DevLayer& L = m->layers[l];
            const DevQW* groups[4][3] = {{&L.q, &L.k, &L.v}, {&L.o, nullptr, nullptr}, {&L.gate, &L.up, nullptr}, {&L.down, nullptr, nullptr}};
            for (int i = 0; i < 4; i++) {
                q4_rows::GemmMat& gmat = r->gm[(size_t)l * 4 + i];
                const int K = groups[i][0]->K;
                int N = 0, parts = 0;
                for (int j = 0; j < 3 && groups[i][j]; j++) { N += groups[i][j]->N; parts++; }
                gmat.K = K;
                gmat.N = N;
                RTRY(rows_alloc(r, (void**)&gmat.wi, (size_t)N * q4_pw(K) * 4));
                uint32_t* zeros = nullptr;
                uint16_t* scales = nullptr;
                if (parts > 1) {
                    RTRY(rows_alloc(r, (void**)&zeros, (size_t)N * q4_pz(K) * 4));
                    RTRY(rows_alloc(r, (void**)&scales, (size_t)N * q4_groups(K) * 2));
                }
                size_t row0 = 0;
                for (int j = 0; j < parts; j++) {
                    const DevQW* q = groups[i][j];
                    RTRY(q4_gemm_interleave_weights(nullptr, gmat.wi + row0 * q4_pw(K), q->w.weight, K, q->N));
                    if (parts > 1) {
                        Q4_CUDA_TRY(cudaMemcpy(zeros + row0 * q4_pz(K), q->w.zeros, (size_t)q->N * q4_pz(K) * 4, cudaMemcpyDeviceToDevice));
                        Q4_CUDA_TRY(cudaMemcpy(scales + row0 * q4_groups(K), q->w.scales, (size_t)q->N * q4_groups(K) * 2, cudaMemcpyDeviceToDevice));
                    }
                    row0 += q->N;
                }
                gmat.w.weight = gmat.wi;   // (the GEMM reads the interleaved words; this field only has to be non-null)
                gmat.w.zeros = parts > 1 ? zeros : groups[i][0]->w.zeros;
                gmat.w.scales = parts > 1 ? scales : groups[i][0]->w.scales;
            }
        }
        Q4_CUDA_TRY(cudaDeviceSynchronize());
    }
    if (rows > r->cap) {
        const int cap = (rows + 63) / 64 * 64;
        const size_t dim = c.dim, hk = m->h_kc;
        RTRY(rows_alloc(r, (void**)&r->X, 2 * cap * dim));
        RTRY(rows_alloc(r, (void**)&r->XB, 2 * cap * dim));
        RTRY(rows_alloc(r, (void**)&r->Q, 2 * (size_t)cap * m->q_n));
        RTRY(rows_alloc(r, (void**)&r->K, 2 * (size_t)cap * m->kv_n));
        RTRY(rows_alloc(r, (void**)&r->V, 2 * (size_t)cap * m->kv_n));
        RTRY(rows_alloc(r, (void**)&r->ATT, 2 * (size_t)cap * m->q_n));
        RTRY(rows_alloc(r, (void**)&r->G, 2 * cap * hk));
        if (cap > kSkinnyRows) {
            RTRY(rows_alloc(r, (void**)&r->QKV, 2 * (size_t)cap * (m->q_n + 2 * m->kv_n)));
            RTRY(rows_alloc(r, (void**)&r->GU, 2 * cap * 2 * hk));
        }
        RTRY(rows_alloc(r, (void**)&r->row_seq, sizeof(int) * cap));
        RTRY(rows_alloc(r, (void**)&r->row_pos, sizeof(int) * cap));
        size_t ws = 0;
        const int shapes[4][2] = {{c.dim, m->q_n + 2 * m->kv_n}, {m->o_kc, c.dim}, {c.dim, 2 * m->h_kc}, {m->h_kc, c.dim}};
        for (auto& s : shapes)
            for (int mm : {1, 16, 17, 64, 65, cap}) ws = std::max(ws, q4_matmul_q4_batched_workspace_bytes(std::min(mm, cap), s[0], s[1]));
        RTRY(rows_alloc(r, &r->ws, ws));
        Q4_CUDA_TRY(cudaMemset(r->ws, 0, ws));
        r->ws_bytes = ws;
        r->cap = cap;
    }
#undef RTRY
    return Q4_OK;
}

// Sum of the ranks' partial [count] vectors: NCCL when it is attached, the communicator's choice says so (large messages)
// and the caller allows it (a prompt's rows); else the one-shot peer push in pieces its inbox holds (always for the
// batched-decode step, which is replayed from a CUDA graph and keeps to kernels of this library).
static int rows_all_reduce(q4_model* m, cudaStream_t s, __half* buf, size_t count, bool allow_nccl) {
    if (m->g == 1) return Q4_OK;
    for (size_t at = 0; at < count;) {
        const bool nccl = allow_nccl && q4_comm_prefers_nccl(m->comm, (int)std::min<size_t>(count - at, (size_t)1 << 30));
        const size_t n = nccl ? count - at : std::min<size_t>(count - at, (size_t)Q4_COMM_MAX_HALFS);
        if (int e = nccl ? q4_all_reduce(m->comm, s, (uint16_t*)(buf + at), (int)n) : q4_all_reduce_peer_push(m->comm, s, (uint16_t*)(buf + at), (int)n)) return e;
        at += n;
    }
    return Q4_OK;
}

// All layers for `n` rows whose embeddings are in r->X; K/V rows go to (kc, vc) with `seq_stride` halfs between sequences.
// pos0 >= 0: the rows are positions pos0 .. pos0 + n - 1 of one sequence (prompt); -1: one row per sequence (batched decode).
static int rows_layers(q4_model* m, cudaStream_t s, int n, __half* kc, __half* vc, long long seq_stride, int pos0) {
    q4_rows* r = m->rows;
    const q4_config& c = m->cfg;
    const int g = m->g, dim = c.dim, hs = m->head_size;
    const int heads = c.n_heads / g, kv_heads = c.n_kv_heads / g;
    int e;
#define OP(expr) do { e = (expr); if (e != Q4_OK) return e; } while (0)
    auto gemm = [&](__half* y, const __half* x, int l, int mat) {   // mat: 0 q|k|v, 1 o, 2 gate|up, 3 down
        const q4_rows::GemmMat& gmat = r->gm[(size_t)l * 4 + mat];
        return q4_matmul_q4_batched(s, (uint16_t*)y, (const uint16_t*)x, &gmat.w, gmat.wi, n, gmat.K, gmat.N, r->ws, r->ws_bytes);
    };
    // q, k, v of the rows: three buffers (few-rows kernels) or three slices of the fused GEMM's output
    const int nqkv = m->q_n + 2 * m->kv_n;
    const bool skinny = n <= kSkinnyRows;
    const bool overlap = pos0 < 0;   // batched decode: programmatic dependent launches (see launch_rows)
    for (int l = 0; l < c.n_layers; l++) {
        const DevLayer& L = m->layers[l];
        const long long loff = (long long)l * c.seq_len * m->kv_n;
        launch_rows(overlap, rmsnorm_rows_kernel, dim3(n), dim3(kRowThreads), 0, s, r->XB, r->X, (const __half*)L.rms_att, dim);
        if (skinny) {
            OP(q4_qkv_matmul_rows(s, (uint16_t*)r->Q, (uint16_t*)r->K, (uint16_t*)r->V, (const uint16_t*)r->XB, &L.q.w, &L.k.w, &L.v.w, n, dim, m->q_n, m->kv_n));
        } else {
            OP(gemm(r->QKV, r->XB, l, 0));
        }
        __half* qp = skinny ? r->Q : r->QKV;
        const __half* kp = skinny ? r->K : r->QKV + m->q_n;
        const __half* vp = skinny ? r->V : r->QKV + m->q_n + m->kv_n;
        const int ldq = skinny ? m->q_n : nqkv, ldkv = skinny ? m->kv_n : nqkv;
        launch_rows(overlap, rope_store_rows_kernel, dim3(n, q4_div_up(heads + kv_heads, kRopeHeads)), dim3(256), 0, s, qp, kp, vp, ldq, ldkv, kc, vc, heads, kv_heads, hs,
                    r->row_seq, r->row_pos, seq_stride, loff, c.rope_theta);
        if (pos0 >= 0 && !skinny)
            launch_rows(overlap, attention_prefill_kernel, dim3(heads, q4_div_up(n, kAtRows)), dim3(128), 0, s, r->ATT, (const __half*)qp, ldq, kc + loff, vc + loff, heads,
                        m->kv_mul, n, pos0, m->kv_n);
        else
            launch_rows(overlap, attention_rows_kernel, dim3(heads, n), dim3(kAttWarps * 32), 0, s, r->ATT, (const __half*)qp, ldq, kc, vc, heads, m->kv_mul, r->row_seq,
                        r->row_pos, seq_stride, loff, m->kv_n);
        // x = o_proj(att) + x / g, summed over the ranks (gpu_kernels.h:237-238, llama2_q4.cu:472-476)
        if (skinny) OP(q4_matmul_q4_rows(s, (uint16_t*)r->X, (const uint16_t*)r->ATT, &L.o.w, n, m->o_kc, dim, (const uint16_t*)r->X, 1.0f / g));
        else {   // the normalised rows in XB are spent: the projection lands there, then x = projection + x / g
            OP(gemm(r->XB, r->ATT, l, 1));
            launch_rows(overlap, add_residual_rows_kernel, dim3(148 * 4), dim3(256), 0, s, r->X, (const __half*)r->XB, 1.0f / g, (size_t)n * dim);
        }
        OP(rows_all_reduce(m, s, r->X, (size_t)n * dim, pos0 >= 0));
        launch_rows(overlap, rmsnorm_rows_kernel, dim3(n), dim3(kRowThreads), 0, s, r->XB, r->X, (const __half*)L.rms_ffn, dim);
        if (skinny) {
            // gate and up stay in fp32 until silu(gate) * up, as in ffn_matvec_silu_kernel (gpu_kernels.h:278-281)
            OP(q4_ffn_silu_rows(s, (uint16_t*)r->G, (const uint16_t*)r->XB, &L.gate.w, &L.up.w, n, dim, m->h_kc));
            OP(q4_matmul_q4_rows(s, (uint16_t*)r->X, (const uint16_t*)r->G, &L.down.w, n, m->h_kc, dim, (const uint16_t*)r->X, 1.0f / g));
        } else {
            OP(gemm(r->GU, r->XB, l, 2));
            launch_rows(overlap, silu_mul_rows_kernel, dim3(148 * 4), dim3(256), 0, s, r->G, (const __half*)r->GU, m->h_kc, n);
            OP(gemm(r->XB, r->G, l, 3));
            launch_rows(overlap, add_residual_rows_kernel, dim3(148 * 4), dim3(256), 0, s, r->X, (const __half*)r->XB, 1.0f / g, (size_t)n * dim);
        }
        OP(rows_all_reduce(m, s, r->X, (size_t)n * dim, pos0 >= 0));
    }
    Q4_CUDA_TRY(cudaGetLastError());
#undef OP
    return Q4_OK;
}

// ------------------------------------------------------------------------------------------------------------
// prefill
// ------------------------------------------------------------------------------------------------------------
extern "C" int q4_model_prefill(q4_model* m, void* stream, int n_tokens, int gen_token) {
    if (!m || n_tokens < 1) return Q4_ERR_INVALID;
    const q4_config& c = m->cfg;
    const int pos0 = m->host_pos;
    if (pos0 + n_tokens > c.seq_len || pos0 + n_tokens >= Q4_MAX_SEQ_LEN) return Q4_ERR_LIMIT;
    if (int e = rows_prepare(m, n_tokens)) return e;
    q4_rows* r = m->rows;
    cudaStream_t s = (cudaStream_t)stream;
    const int n = n_tokens;
    const bool overlap = false;
    launch_rows(overlap, iota_rows_kernel, dim3(q4_div_up(n, 256)), dim3(256), 0, s, r->row_seq, r->row_pos, n, 0, pos0, 0);
    launch_rows(overlap, embed_rows_kernel, dim3(n), dim3(kRowThreads), 0, s, r->X, (const __half*)m->emb, c.dim, (const int*)m->shared->tokens, 0, r->row_seq, r->row_pos, c.vocab_size);
    if (int e = rows_layers(m, s, n, (__half*)m->kc, (__half*)m->vc, 0, pos0)) return e;
    // the last row goes on through the batch-1 tail (llama2_q4.cu:528-537, sampler.h:77-84): final norm, classifier,
    // [all-gather], hand-off; the position words are moved to that row first, the hand-off then steps them past it
    Q4_CUDA_TRY(cudaMemcpyAsync(m->x, r->X + (size_t)(n - 1) * c.dim, 2 * (size_t)c.dim, cudaMemcpyDeviceToDevice, s));
    launch_rows(overlap, set_pos_kernel, dim3(1), dim3(1), 0, s, m->pos, &m->shared->pos, pos0 + n - 1);
    int e;
    if ((e = q4_rmsnorm(s, m->x, m->x, m->rms_final, c.dim)) != Q4_OK) return e;
    if ((e = q4_matmul_f16(s, m->logits + (size_t)m->rank * m->v_n, m->x, m->wcls, c.dim, m->v_n, 1.0f)) != Q4_OK) return e;
    if (m->g > 1 && (e = q4_all_gather(m->comm, s, m->logits + (size_t)m->rank * m->v_n, m->logits, m->v_n)) != Q4_OK) return e;
    if ((e = q4_argmax(s, m->logits, c.vocab_size, (int*)m->shared->tokens, &m->shared->pos, m->pos, gen_token != 0)) != Q4_OK) return e;
    // sample() draws one coin per position, used or not (sampler.h:79): keep the generator where n token steps leave it
    for (int i = 0; i < n; i++) (void)q4_random_f32(&m->rng_state);
    m->host_pos = pos0 + n;
    return Q4_OK;
}

// ------------------------------------------------------------------------------------------------------------
// batched decode: several sequences, one position each per step
// ------------------------------------------------------------------------------------------------------------
struct q4_batch {
    q4_model* m;
    int n_seq, n_prompt, max_len;
    __half *kc = nullptr, *vc = nullptr, *logits = nullptr, *xf = nullptr, *part = nullptr;
    int *tokens = nullptr, *pos = nullptr;
    long long seq_stride;
    int steps = 0;
    // A step is the same work every time (positions and ids live in device memory), so it is captured once as a CUDA
    // graph and replayed: ~260 launches per step on a 32-layer model would otherwise be issued one by one.
    cudaGraphExec_t step_graph = nullptr;
    bool use_graph = true;
};

extern "C" int q4_batch_free(q4_batch* b) {
    if (!b) return Q4_OK;
    if (b->step_graph) cudaGraphExecDestroy(b->step_graph);
    cudaFree(b->kc); cudaFree(b->vc); cudaFree(b->logits); cudaFree(b->xf); cudaFree(b->part); cudaFree(b->tokens); cudaFree(b->pos);
    delete b;
    return Q4_OK;
}

extern "C" int q4_batch_create(q4_batch** out, q4_model* m, int n_seq) {
    if (!out || !m || n_seq < 1 || n_seq > 16) return Q4_ERR_INVALID;
    if (int e = rows_prepare(m, n_seq)) return e;
    const q4_config& c = m->cfg;
    if (2 * (size_t)n_seq * c.dim > 200 * 1024 && !(c.dim % 32 == 0 && m->v_n % 16 == 0)) return Q4_ERR_UNSUPPORTED_SIZE;   // the plain classifier keeps the rows in shared memory
    Q4_CUDA_TRY(cudaFuncSetAttribute(matvec_f16_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::min<size_t>(2 * (size_t)n_seq * c.dim, 200 * 1024)));
    q4_batch* b = new q4_batch();
    b->m = m;
    b->n_seq = n_seq;
    b->n_prompt = 0;
    b->max_len = c.seq_len;
    b->seq_stride = (long long)c.n_layers * c.seq_len * m->kv_n;
    const size_t kv_bytes = 2 * (size_t)n_seq * b->seq_stride;
    cudaError_t e = cudaMalloc((void**)&b->kc, kv_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&b->vc, kv_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&b->logits, 2 * (size_t)n_seq * c.vocab_size);
    if (e == cudaSuccess) e = cudaMalloc((void**)&b->xf, 2 * (size_t)n_seq * c.dim);
    if (e == cudaSuccess) e = cudaMalloc((void**)&b->part, 2 * (size_t)n_seq * m->v_n);
    if (e == cudaSuccess) e = cudaMalloc((void**)&b->tokens, sizeof(int) * (size_t)n_seq * (c.seq_len + 1));
    if (e == cudaSuccess) e = cudaMalloc((void**)&b->pos, sizeof(int) * n_seq);
    if (e == cudaSuccess) e = cudaMemset(b->kc, 0, kv_bytes);
    if (e == cudaSuccess) e = cudaMemset(b->vc, 0, kv_bytes);
    if (e != cudaSuccess) { q4_note_cuda_error(e, __FILE__, __LINE__); q4_batch_free(b); return Q4_ERR_CUDA; }
    *out = b;
    return Q4_OK;
}

// prompts: [n_seq][n_prompt] token ids; all sequences start at position 0
extern "C" int q4_batch_reset(q4_batch* b, const int* prompts, int n_prompt) {
    if (!b || !prompts || n_prompt < 1 || n_prompt > b->max_len) return Q4_ERR_INVALID;
    for (int i = 0; i < b->n_seq * n_prompt; i++)
        if (prompts[i] < 0 || prompts[i] >= b->m->cfg.vocab_size) return Q4_ERR_INVALID;
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    Q4_CUDA_TRY(cudaMemset(b->tokens, 0, sizeof(int) * (size_t)b->n_seq * (b->max_len + 1)));
    Q4_CUDA_TRY(cudaMemcpy2D(b->tokens, sizeof(int) * (b->max_len + 1), prompts, sizeof(int) * n_prompt, sizeof(int) * n_prompt, b->n_seq, cudaMemcpyHostToDevice));
    Q4_CUDA_TRY(cudaMemset(b->pos, 0, sizeof(int) * b->n_seq));
    if (b->step_graph && n_prompt != b->n_prompt) {   // the prompt length is an argument of the captured hand-off kernel
        cudaGraphExecDestroy(b->step_graph);
        b->step_graph = nullptr;
    }
    b->n_prompt = n_prompt;
    b->steps = 0;
    return Q4_OK;
}

static int batch_step(q4_batch* b, cudaStream_t s);

// One position of every sequence: embedding .. logits .. greedy hand-off per sequence. Asynchronous on `stream`.
extern "C" int q4_batch_forward(q4_batch* b, void* stream) {
    if (!b || b->n_prompt < 1) return Q4_ERR_INVALID;
    if (b->steps >= b->max_len) return Q4_ERR_LIMIT;
    cudaStream_t s = (cudaStream_t)stream;
    if (!b->use_graph) {
        if (int e = batch_step(b, s)) return e;
    } else {
        if (!b->step_graph) {
            cudaGraph_t graph = nullptr;
            Q4_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            const int e = batch_step(b, s);
            const cudaError_t ce = cudaStreamEndCapture(s, &graph);
            if (e != Q4_OK) { if (graph) cudaGraphDestroy(graph); return e; }
            Q4_CUDA_TRY(ce);
            Q4_CUDA_TRY(cudaGraphInstantiate(&b->step_graph, graph, 0));
            Q4_CUDA_TRY(cudaGraphDestroy(graph));
        }
        Q4_CUDA_TRY(cudaGraphLaunch(b->step_graph, s));
    }
    b->steps++;
    return Q4_OK;
}

static int batch_step(q4_batch* b, cudaStream_t s) {
    q4_model* m = b->m;
    q4_rows* r = m->rows;
    const q4_config& c = m->cfg;
    const int n = b->n_seq;
    const bool overlap = true;
    launch_rows(overlap, iota_rows_kernel, dim3(1), dim3(32), 0, s, r->row_seq, nullptr, n, 0, 0, 1);
    Q4_CUDA_TRY(cudaMemcpyAsync(r->row_pos, b->pos, sizeof(int) * n, cudaMemcpyDeviceToDevice, s));
    launch_rows(overlap, embed_rows_kernel, dim3(n), dim3(kRowThreads), 0, s, r->X, (const __half*)m->emb, c.dim, b->tokens, b->max_len + 1, r->row_seq, r->row_pos, c.vocab_size);
    if (int e = rows_layers(m, s, n, b->kc, b->vc, b->seq_stride, -1)) return e;
    launch_rows(overlap, rmsnorm_rows_kernel, dim3(n), dim3(kRowThreads), 0, s, b->xf, r->X, (const __half*)m->rms_final, c.dim);
    const size_t smem = 2 * (size_t)n * c.dim;
    __half* cls_out = m->g == 1 ? b->logits : b->part;   // TP: every rank computes its vocabulary slice of every row; the slices are gathered row by row
    const int cls_stride = m->g == 1 ? c.vocab_size : m->v_n;
    if (c.dim % 32 == 0 && m->v_n % 16 == 0) {
        if (n <= 8) launch_rows(overlap, classifier_rows_kernel<1>, dim3(q4_div_up(m->v_n / 16, 8)), dim3(256), 0, s, cls_out, b->xf, (const __half*)m->wcls, c.dim, m->v_n, n, cls_stride);
        else launch_rows(overlap, classifier_rows_kernel<2>, dim3(q4_div_up(m->v_n / 16, 8)), dim3(256), 0, s, cls_out, b->xf, (const __half*)m->wcls, c.dim, m->v_n, n, cls_stride);
    } else {
        launch_rows(overlap, matvec_f16_rows_kernel, dim3(148 * 2), dim3(256), smem, s, cls_out, b->xf, (const __half*)m->wcls, c.dim, m->v_n, n, cls_stride);
    }
    if (m->g > 1) {
        for (int i = 0; i < n; i++)
            if (int e = q4_all_gather(m->comm, s, (const uint16_t*)(b->part + (size_t)i * m->v_n), (uint16_t*)(b->logits + (size_t)i * c.vocab_size), m->v_n)) return e;
    }
    launch_rows(overlap, argmax_rows_kernel, dim3(n), dim3(1024), 0, s, b->logits, c.vocab_size, b->tokens, b->max_len + 1, b->pos, b->n_prompt);
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}

extern "C" const uint16_t* q4_batch_logits(const q4_batch* b) { return b ? (const uint16_t*)b->logits : nullptr; }

// tokens[s][0 .. len) of every sequence (synchronises the device)
extern "C" int q4_batch_read_tokens(const q4_batch* b, int* out, int len) {
    if (!b || !out || len < 1 || len > b->max_len + 1) return Q4_ERR_INVALID;
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    Q4_CUDA_TRY(cudaMemcpy2D(out, sizeof(int) * len, b->tokens, sizeof(int) * (b->max_len + 1), sizeof(int) * len, b->n_seq, cudaMemcpyDeviceToHost));
    return Q4_OK;
}
