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

// ids of the rows' tokens: tok_base[seq * tok_stride + pos]
__global__ void embed_rows_kernel(__half* x, const __half* table, int dim, const int* tok_base, long long tok_stride, const int* row_seq, const int* row_pos,
                                  int vocab) {
    const int m = blockIdx.x;
    int token = tok_base[(long long)row_seq[m] * tok_stride + row_pos[m]];
    if (token < 0 || token >= vocab) token = 0;   // (ids are validated on the host; a generated id is always in range)
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)token * dim);
    uint4* dst = reinterpret_cast<uint4*>(x + (size_t)m * dim);
    for (int i = threadIdx.x; i < dim / 8; i += blockDim.x) dst[i] = src[i];
}

// rmsnorm_kernel (gpu_kernels.h:72-105) per row: o = x * (rsqrt(mean(x^2) + 1e-5) * w), fp32 inside, fp16 out
__global__ void rmsnorm_rows_kernel(__half* o, const __half* x, const __half* w, int size) {
    __shared__ float red[kRowThreads / 32];
    const __half* xr = x + (size_t)blockIdx.x * size;
    __half* orow = o + (size_t)blockIdx.x * size;
    float ss = 0.f;
    for (int i = threadIdx.x; i < size; i += blockDim.x) {
        const float v = __half2float(xr[i]);
        ss += v * v;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < kRowThreads / 32; i++) tot += red[i];
    tot /= size;
    tot += 1e-5f;
    tot = 1.0f / sqrtf(tot);
    for (int i = threadIdx.x; i < size; i += blockDim.x) orow[i] = __float2half(__half2float(xr[i]) * (tot * __half2float(w[i])));
}

// RoPERotation_kernel (gpu_kernels.h:340-363) per row, and the row's K and V into the cache: query heads are rotated in place,
// the key heads are rotated on their way into cache row `pos` of the row's sequence, the value heads are copied there.
// grid (rows, heads + kv_heads), block head_size / 2.
__global__ void rope_store_rows_kernel(__half* q, const __half* k, const __half* v, __half* kc, __half* vc, int n_heads, int n_kv_heads, int head_size,
                                       const int* row_seq, const int* row_pos, long long seq_stride, long long loff, float theta) {
    const int m = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
    const int pos = row_pos[m];
    const int head_dim = (i * 2) % head_size;
    const float freq = 1.0f / powf(theta, head_dim / (float)head_size);
    const float val = pos * freq;
    const float fcr = cosf(val), fci = sinf(val);
    const int half_hs = head_size / 2;
    if (h < n_heads) {
        __half* qr = q + (size_t)m * n_heads * head_size + (size_t)h * head_size;
        const float q0 = __half2float(qr[i]), q1 = __half2float(qr[i + half_hs]);
        qr[i] = __float2half(q0 * fcr - q1 * fci);
        qr[i + half_hs] = __float2half(q0 * fci + q1 * fcr);
    } else {
        const int kh = h - n_heads;
        const size_t src = (size_t)m * n_kv_heads * head_size + (size_t)kh * head_size;
        const size_t dst = (size_t)row_seq[m] * seq_stride + loff + (size_t)pos * n_kv_heads * head_size + (size_t)kh * head_size;
        const float k0 = __half2float(k[src + i]), k1 = __half2float(k[src + i + half_hs]);
        kc[dst + i] = __float2half(k0 * fcr - k1 * fci);
        kc[dst + i + half_hs] = __float2half(k0 * fci + k1 * fcr);
        vc[dst + i] = v[src + i];
        vc[dst + i + half_hs] = v[src + i + half_hs];
    }
}

// MultiHeadAttention (llama2_q4.cu:410-427) for one (row, head): the query attends to cached positions 0 .. pos of its own
// sequence (its own K/V row was stored by the RoPE kernel before). Scores are rounded to fp16 as the reference stores them
// (gpu_kernels.h:171-175); the softmax runs online in fp32 over the keys a warp visits (keys warp, warp + 4, ...), the four
// warps are merged at the end. head_size 128: a lane holds four dims. grid (heads, rows), block 128.
__global__ void __launch_bounds__(128) attention_rows_kernel(__half* out, const __half* q, const __half* kc, const __half* vc, int n_heads, int kv_mul,
                                                             const int* row_seq, const int* row_pos, long long seq_stride, long long loff, int kv_n) {
    constexpr int HS = 128;
    const int h = blockIdx.x, m = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int T = row_pos[m] + 1;
    const __half* kb = kc + (size_t)row_seq[m] * seq_stride + loff + (size_t)(h / kv_mul) * HS + lane * 4;
    const __half* vb = vc + (size_t)row_seq[m] * seq_stride + loff + (size_t)(h / kv_mul) * HS + lane * 4;
    float qf[4];
    {
        const uint2 qv = *reinterpret_cast<const uint2*>(q + ((size_t)m * n_heads + h) * HS + lane * 4);
        const __half2* qh = reinterpret_cast<const __half2*>(&qv);
        qf[0] = __low2float(qh[0]); qf[1] = __high2float(qh[0]); qf[2] = __low2float(qh[1]); qf[3] = __high2float(qh[1]);
    }
    const float alpha = (float)(1.0 / sqrt((double)HS));
    float mx = -CUDART_INF_F, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = warp; t < T; t += 4) {
        const uint2 kv = *reinterpret_cast<const uint2*>(kb + (size_t)t * kv_n);
        const uint2 vv = *reinterpret_cast<const uint2*>(vb + (size_t)t * kv_n);
        const __half2* kh = reinterpret_cast<const __half2*>(&kv);
        float sc = qf[0] * __low2float(kh[0]) + qf[1] * __high2float(kh[0]) + qf[2] * __low2float(kh[1]) + qf[3] * __high2float(kh[1]);
        sc = warp_sum(sc);
        sc = __half2float(__float2half(sc * alpha));
        const float mn = fmaxf(mx, sc);
        const float corr = expf(mx - mn), pr = expf(sc - mn);
        const __half2* vh = reinterpret_cast<const __half2*>(&vv);
        l = l * corr + pr;
        acc[0] = acc[0] * corr + pr * __low2float(vh[0]);
        acc[1] = acc[1] * corr + pr * __high2float(vh[0]);
        acc[2] = acc[2] * corr + pr * __low2float(vh[1]);
        acc[3] = acc[3] * corr + pr * __high2float(vh[1]);
        mx = mn;
    }
    __shared__ float s_m[4], s_l[4], s_acc[4][HS];
    if (lane == 0) { s_m[warp] = mx; s_l[warp] = l; }
#pragma unroll
    for (int j = 0; j < 4; j++) s_acc[warp][lane * 4 + j] = acc[j];
    __syncthreads();
    if (threadIdx.x < HS) {
        float M = -CUDART_INF_F;
        for (int w = 0; w < 4; w++) M = fmaxf(M, s_m[w]);
        float a = 0.f, L = 0.f;
        for (int w = 0; w < 4; w++) {
            if (s_m[w] != -CUDART_INF_F) {
                const float e = expf(s_m[w] - M);
                a += s_acc[w][threadIdx.x] * e;
                L += s_l[w] * e;
            }
        }
        out[((size_t)m * n_heads + h) * HS + threadIdx.x] = __float2half(L > 0.f ? a / L : 0.f);
    }
}

// ffn_matvec_silu's epilogue (gpu_kernels.h:278-281) on two GEMM results: h = silu(gate) * up in fp32, fp16 out
__global__ void silu_mul_rows_kernel(__half* h, const __half* gate, const __half* up, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float val = __half2float(gate[i]);
        val *= 1.0f / (1.0f + expf(-val));
        val *= __half2float(up[i]);
        h[i] = __float2half(val);
    }
}

// both position words (device, pinned host) to `pos`, in stream order
__global__ void set_pos_kernel(int* pos_dev, volatile int* pos_pinned, int pos) {
    *pos_dev = pos;
    *pos_pinned = pos;
}

__global__ void iota_rows_kernel(int* row_seq, int* row_pos, int n, int seq, int pos0, int step_seq) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        row_seq[i] = seq + i * step_seq;
        if (row_pos) row_pos[i] = pos0 + i;
    }
}

// mat_vec_kernel (gpu_kernels.h:117-147) for B rows of x at once: a warp takes one classifier row and B dot products, so the
// classifier is read once per step, not once per sequence. x rows sit in shared memory. B <= 16.
__global__ void __launch_bounds__(256) matvec_f16_rows_kernel(__half* y, const __half* x, const __half* w, int n, int d, int B, int y_stride) {
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

// argmax per row (lowest index among equal maxima, like q4_argmax) and the hand-off of batched decode: the id becomes
// the sequence's next token when that position is past its prompt, and the sequence moves on by one position.
__global__ void __launch_bounds__(256) argmax_rows_kernel(const __half* logits, int vocab, int* tokens, long long tok_stride, int* pos, int n_prompt) {
    __shared__ float sval[8];
    __shared__ int sidx[8];
    const int s = blockIdx.x;
    const __half* x = logits + (size_t)s * vocab;
    float best = -CUDART_INF_F;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
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
        for (int w = 1; w < 8; w++)
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
    __half *X = nullptr, *XB = nullptr, *Q = nullptr, *K = nullptr, *V = nullptr, *ATT = nullptr, *G = nullptr, *U = nullptr;
    int *row_seq = nullptr, *row_pos = nullptr;
    void* ws = nullptr;
    size_t ws_bytes = 0;
    std::vector<uint32_t*> wi;   // [layer * 7 + matrix] interleaved copy of the packed weights (q k v o gate up down)
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

static const DevQW* layer_mats(const DevLayer& L, int i) {
    const DevQW* a[7] = {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down};
    return a[i];
}

// Buffers for up to `rows` rows (grown on demand) and, once, the interleaved weight copies.
static int rows_prepare(q4_model* m, int rows) {
    if (m->column || m->head_size != 128 || (m->cfg.dim % 128) || (m->o_kc % 128) || (m->h_kc % 128)) return Q4_ERR_UNSUPPORTED_SIZE;
    if (!m->rows) m->rows = new q4_rows();
    q4_rows* r = m->rows;
    const q4_config& c = m->cfg;
    int e;
#define RTRY(expr) do { e = (expr); if (e != Q4_OK) return e; } while (0)
    if (r->wi.empty()) {
        r->wi.assign((size_t)c.n_layers * 7, nullptr);
        for (int l = 0; l < c.n_layers; l++)
            for (int i = 0; i < 7; i++) {
                const DevQW* q = layer_mats(m->layers[l], i);
                uint32_t* d = nullptr;
                RTRY(rows_alloc(r, (void**)&d, (size_t)q->N * q4_pw(q->K) * 4));
                RTRY(q4_gemm_interleave_weights(nullptr, d, q->w.weight, q->K, q->N));
                r->wi[(size_t)l * 7 + i] = d;
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
        RTRY(rows_alloc(r, (void**)&r->U, 2 * cap * hk));
        RTRY(rows_alloc(r, (void**)&r->row_seq, sizeof(int) * cap));
        RTRY(rows_alloc(r, (void**)&r->row_pos, sizeof(int) * cap));
        size_t ws = 0;
        const int shapes[5][2] = {{c.dim, m->q_n}, {c.dim, m->kv_n}, {m->o_kc, c.dim}, {c.dim, m->h_kc}, {m->h_kc, c.dim}};
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

// Sum of the ranks' partial [count] vectors: NCCL when it is attached and the communicator's choice says so (large messages),
// else the one-shot peer push in pieces its inbox holds.
static int rows_all_reduce(q4_model* m, cudaStream_t s, __half* buf, size_t count) {
    if (m->g == 1) return Q4_OK;
    for (size_t at = 0; at < count;) {
        const size_t n = q4_comm_prefers_nccl(m->comm, (int)std::min<size_t>(count - at, (size_t)1 << 30)) ? count - at : std::min<size_t>(count - at, (size_t)Q4_COMM_MAX_HALFS);
        if (int e = q4_all_reduce(m->comm, s, (uint16_t*)(buf + at), (int)n)) return e;
        at += n;
    }
    return Q4_OK;
}

// All layers for `n` rows whose embeddings are in r->X; K/V rows go to (kc, vc) with `seq_stride` halfs between sequences.
static int rows_layers(q4_model* m, cudaStream_t s, int n, __half* kc, __half* vc, long long seq_stride) {
    q4_rows* r = m->rows;
    const q4_config& c = m->cfg;
    const int g = m->g, dim = c.dim, hs = m->head_size;
    const int heads = c.n_heads / g, kv_heads = c.n_kv_heads / g;
    int e;
#define OP(expr) do { e = (expr); if (e != Q4_OK) return e; } while (0)
    auto gemm = [&](__half* y, const __half* x, int l, int mat, const __half* resid, float rs) {
        const DevQW* q = layer_mats(m->layers[l], mat);
        return q4_matmul_q4_batched_residual(s, (uint16_t*)y, (const uint16_t*)x, &q->w, r->wi[(size_t)l * 7 + mat], n, q->K, q->N, (const uint16_t*)resid, rs,
                                             r->ws, r->ws_bytes);
    };
    for (int l = 0; l < c.n_layers; l++) {
        const DevLayer& L = m->layers[l];
        const long long loff = (long long)l * c.seq_len * m->kv_n;
        rmsnorm_rows_kernel<<<n, kRowThreads, 0, s>>>(r->XB, r->X, (const __half*)L.rms_att, dim);
        OP(gemm(r->Q, r->XB, l, 0, nullptr, 0.f));
        OP(gemm(r->K, r->XB, l, 1, nullptr, 0.f));
        OP(gemm(r->V, r->XB, l, 2, nullptr, 0.f));
        rope_store_rows_kernel<<<dim3(n, heads + kv_heads), hs / 2, 0, s>>>(r->Q, r->K, r->V, kc, vc, heads, kv_heads, hs, r->row_seq, r->row_pos, seq_stride,
                                                                              loff, c.rope_theta);
        attention_rows_kernel<<<dim3(heads, n), 128, 0, s>>>(r->ATT, r->Q, kc, vc, heads, m->kv_mul, r->row_seq, r->row_pos, seq_stride, loff, m->kv_n);
        // x = o_proj(att) + x / g, summed over the ranks (gpu_kernels.h:237-238, llama2_q4.cu:472-476)
        OP(gemm(r->X, r->ATT, l, 3, r->X, 1.0f / g));
        OP(rows_all_reduce(m, s, r->X, (size_t)n * dim));
        rmsnorm_rows_kernel<<<n, kRowThreads, 0, s>>>(r->XB, r->X, (const __half*)L.rms_ffn, dim);
        OP(gemm(r->G, r->XB, l, 4, nullptr, 0.f));
        OP(gemm(r->U, r->XB, l, 5, nullptr, 0.f));
        silu_mul_rows_kernel<<<148 * 4, 256, 0, s>>>(r->G, r->G, r->U, (size_t)n * m->h_kc);
        OP(gemm(r->X, r->G, l, 6, r->X, 1.0f / g));
        OP(rows_all_reduce(m, s, r->X, (size_t)n * dim));
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
    iota_rows_kernel<<<q4_div_up(n, 256), 256, 0, s>>>(r->row_seq, r->row_pos, n, 0, pos0, 0);
    embed_rows_kernel<<<n, kRowThreads, 0, s>>>(r->X, (const __half*)m->emb, c.dim, (const int*)m->shared->tokens, 0, r->row_seq, r->row_pos, c.vocab_size);
    if (int e = rows_layers(m, s, n, (__half*)m->kc, (__half*)m->vc, 0)) return e;
    // the last row goes on through the batch-1 tail (llama2_q4.cu:528-537, sampler.h:77-84): final norm, classifier,
    // [all-gather], hand-off; the position words are moved to that row first, the hand-off then steps them past it
    Q4_CUDA_TRY(cudaMemcpyAsync(m->x, r->X + (size_t)(n - 1) * c.dim, 2 * (size_t)c.dim, cudaMemcpyDeviceToDevice, s));
    set_pos_kernel<<<1, 1, 0, s>>>(m->pos, &m->shared->pos, pos0 + n - 1);
    int e;
    if ((e = q4_rmsnorm(s, m->x, m->x, m->rms_final, c.dim)) != Q4_OK) return e;
    if ((e = q4_matmul_f16(s, m->logits + (size_t)m->rank * m->v_n, m->x, m->wcls, c.dim, m->v_n, 1.0f)) != Q4_OK) return e;
    if (m->g > 1 && (e = q4_all_gather(m->comm, s, m->logits + (size_t)m->rank * m->v_n, m->logits, m->v_n)) != Q4_OK) return e;
    if ((e = q4_argmax(s, m->logits, c.vocab_size, (int*)m->shared->tokens, &m->shared->pos, m->pos, gen_token != 0)) != Q4_OK) return e;
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
};

extern "C" int q4_batch_free(q4_batch* b) {
    if (!b) return Q4_OK;
    cudaFree(b->kc); cudaFree(b->vc); cudaFree(b->logits); cudaFree(b->xf); cudaFree(b->part); cudaFree(b->tokens); cudaFree(b->pos);
    delete b;
    return Q4_OK;
}

extern "C" int q4_batch_create(q4_batch** out, q4_model* m, int n_seq) {
    if (!out || !m || n_seq < 1 || n_seq > 16) return Q4_ERR_INVALID;
    if (int e = rows_prepare(m, n_seq)) return e;
    const q4_config& c = m->cfg;
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
    b->n_prompt = n_prompt;
    b->steps = 0;
    return Q4_OK;
}

// One position of every sequence: embedding .. logits .. greedy hand-off per sequence. Asynchronous on `stream`.
extern "C" int q4_batch_forward(q4_batch* b, void* stream) {
    if (!b || b->n_prompt < 1) return Q4_ERR_INVALID;
    if (b->steps >= b->max_len) return Q4_ERR_LIMIT;
    q4_model* m = b->m;
    q4_rows* r = m->rows;
    const q4_config& c = m->cfg;
    cudaStream_t s = (cudaStream_t)stream;
    const int n = b->n_seq;
    iota_rows_kernel<<<1, 32, 0, s>>>(r->row_seq, nullptr, n, 0, 0, 1);
    Q4_CUDA_TRY(cudaMemcpyAsync(r->row_pos, b->pos, sizeof(int) * n, cudaMemcpyDeviceToDevice, s));
    embed_rows_kernel<<<n, kRowThreads, 0, s>>>(r->X, (const __half*)m->emb, c.dim, b->tokens, b->max_len + 1, r->row_seq, r->row_pos, c.vocab_size);
    if (int e = rows_layers(m, s, n, b->kc, b->vc, b->seq_stride)) return e;
    rmsnorm_rows_kernel<<<n, kRowThreads, 0, s>>>(b->xf, r->X, (const __half*)m->rms_final, c.dim);
    const size_t smem = 2 * (size_t)n * c.dim;
    Q4_CUDA_TRY(cudaFuncSetAttribute(matvec_f16_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (m->g == 1) {
        matvec_f16_rows_kernel<<<148 * 2, 256, smem, s>>>(b->logits, b->xf, (const __half*)m->wcls, c.dim, m->v_n, n, c.vocab_size);
    } else {   // every rank computes its vocabulary slice of every row; the slices are gathered row by row
        matvec_f16_rows_kernel<<<148 * 2, 256, smem, s>>>(b->part, b->xf, (const __half*)m->wcls, c.dim, m->v_n, n, m->v_n);
        for (int i = 0; i < n; i++)
            if (int e = q4_all_gather(m->comm, s, (const uint16_t*)(b->part + (size_t)i * m->v_n), (uint16_t*)(b->logits + (size_t)i * c.vocab_size), m->v_n)) return e;
    }
    argmax_rows_kernel<<<n, 256, 0, s>>>(b->logits, c.vocab_size, b->tokens, b->max_len + 1, b->pos, b->n_prompt);
    Q4_CUDA_TRY(cudaGetLastError());
    b->steps++;
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
