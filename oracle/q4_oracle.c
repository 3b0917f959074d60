/*
 * CPU restatement of the llama_cu_awq bs=1 decode arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA path and the
 * timed CPU baseline. Nothing in the shipped library links, loads or calls it.
 *
 * Every function cites the reference lines whose arithmetic it restates
 * (paths are relative to the llama_cu_awq project root). Two accumulation
 * orders are offered for the dot products:
 *   order = 0  "fast"  : plain k-ascending fp32 loop, OpenMP over outputs
 *   order = 1  "warp"  : the reference's order - lane-sequential fmaf over the
 *                        lane's elements, then the 1,2,4,8,16 shuffle-down tree
 *                        of cub::WarpReduce (only lane 0's value is kept)
 *
 * Pinning: the packed layout accessors are checked byte-for-byte against files
 * written by the reference's own weight_packer (tests/golden), and the "warp"
 * order is compared bit-for-bit with the reference's CUDA kernels on a GPU box
 * (oracle/ref_harness.cu). The reference ships no golden vectors of its own.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef uint16_t f16;

/* ---- fp16 <-> fp32, round to nearest even (what __float2half_rn / (half) do) ---- */
float q4o_h2f(f16 h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

f16 q4o_f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) { /* inf / nan */
        return (f16)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0));
    }
    if (ax >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (f16)(sign | 0x7C00u);
    }
    if (ax < 0x33000001u) { /* below half of the smallest subnormal (2^-25) -> 0 */
        return (f16)sign;
    }
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t half_ulp = 1u << (shift - 1);
    if (rem > half_ulp || (rem == half_ulp && (q & 1))) q++;
    return (f16)(sign | (base + q)); /* mantissa carry rolls into the exponent */
}

static inline int div_up(int a, int b) { return (a - 1) / b + 1; }

/* Packed heights. llama2_q4.cu:106-112 (weights, padded to 4 words) and :121-129. */
int q4o_packed_wt_height(int K) { return div_up(K, 32) * 4; }
int q4o_groups(int K) { return div_up(K, 128); }
int q4o_packed_zeros_height(int K) { return div_up(div_up(K, 128), 8); }

/* Nibble accessors. Little-endian nibbles, K-contiguous per output column:
 * weight_packer.cpp:116-124 (pack), gpu_kernels.h:203-208 (unpack), :185,192 (zeros). */
static inline uint32_t nib(const uint32_t *row, int i) { return (row[i >> 3] >> (4 * (i & 7))) & 0xFu; }

int q4o_q(const uint32_t *weight, int K, int n, int k) { return (int)nib(weight + (size_t)n * q4o_packed_wt_height(K), k); }
int q4o_z(const uint32_t *zeros, int K, int n, int g) { return (int)nib(zeros + (size_t)n * q4o_packed_zeros_height(K), g); }

/* Unpacked nibbles, one byte each, [N][K] and [N][G]. */
void q4o_unpack(uint8_t *q_out, uint8_t *z_out, const uint32_t *weight, const uint32_t *zeros, int K, int N) {
    int PW = q4o_packed_wt_height(K), PZ = q4o_packed_zeros_height(K), G = q4o_groups(K);
    for (int n = 0; n < N; n++) {
        for (int k = 0; k < K; k++) q_out[(size_t)n * K + k] = (uint8_t)nib(weight + (size_t)n * PW, k);
        for (int g = 0; g < G; g++) z_out[(size_t)n * G + g] = (uint8_t)nib(zeros + (size_t)n * PZ, g);
    }
}

/* Dequantised weights w(n,k) = (float(q) - float(z)) * float(s). gpu_kernels.h:192-193,204-205. */
void q4o_dequant(float *out, const uint32_t *weight, const uint32_t *zeros, const f16 *scales, int K, int N) {
    int PW = q4o_packed_wt_height(K), PZ = q4o_packed_zeros_height(K), G = q4o_groups(K);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const uint32_t *wr = weight + (size_t)n * PW;
        const uint32_t *zr = zeros + (size_t)n * PZ;
        for (int k = 0; k < K; k++) {
            int g = k >> 7;
            float qz = (float)nib(zr, g);
            float s = q4o_h2f(scales[(size_t)n * G + g]);
            out[(size_t)n * K + k] = ((float)nib(wr, k) - qz) * s;
        }
    }
}

/* shuffle-down tree of cub::WarpReduce<float>::Sum (offsets 1,2,4,8,16); lane 0 holds the result.
 * gpu_kernels.h:140-142,169-171,213-215,331-333. */
static float warp_tree(float v[32]) {
    for (int off = 1; off < 32; off <<= 1)
        for (int l = 0; l + off < 32; l++) v[l] = v[l] + v[l + off];
    return v[0];
}

/* One output column of the W4 g128 dot product. gpu_kernels.h:179-218 (get_mat_vec_int4). */
static float dot_q4(const f16 *x, const uint32_t *wr, const uint32_t *zr, const f16 *sr, int K, int order) {
    int PW = q4o_packed_wt_height(K);
    if (order == 1) {
        float lane[32];
        for (int t = 0; t < 32; t++) {
            float sum = 0.f;
            for (int ygq = 0; ygq * 128 + t * 4 < PW; ygq++) {
                uint32_t zw = zr[ygq];
                const uint32_t *w4 = wr + ygq * 128 + t * 4;
                int group_y = ygq * 8 + t / 4;
                float qz = (float)((zw >> (4 * (t / 4))) & 0xFu);
                float scale = q4o_h2f(sr[group_y]);
                int y_base = ygq * 1024 + t * 32;
                for (int qi = 0; qi < 4; qi++) {
                    int ys = y_base + qi * 8;
                    if (ys < K) {
                        uint32_t p = w4[qi];
                        for (int i = 0; i < 8; i++) {
                            float w = ((float)(p & 0xFu) - qz) * scale;
                            sum = fmaf(w, q4o_h2f(x[ys + i]), sum);
                            p >>= 4;
                        }
                    }
                }
            }
            lane[t] = sum;
        }
        return warp_tree(lane);
    }
    float sum = 0.f;
    int G = q4o_groups(K);
    for (int g = 0; g < G; g++) {
        float qz = (float)nib(zr, g);
        float scale = q4o_h2f(sr[g]);
        int k1 = (g + 1) * 128 < K ? (g + 1) * 128 : K;
        for (int k = g * 128; k < k1; k++) {
            float w = ((float)nib(wr, k) - qz) * scale;
            sum += w * q4o_h2f(x[k]);
        }
    }
    return sum;
}

/* y = W·x with optional fused residual y += y_old / gpu_count. gpu_kernels.h:221-248 (mat_vec_int4,
 * mat_vec_kernel_int4); host wrapper llama2_q4.cu:367-376. Output rounded to fp16. */
void q4o_matvec(f16 *y, const f16 *x, const uint32_t *weight, const uint32_t *zeros, const f16 *scales,
                int K, int N, int accum, int gpu_count, int order) {
    int PW = q4o_packed_wt_height(K), PZ = q4o_packed_zeros_height(K), G = q4o_groups(K);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        float sum = dot_q4(x, weight + (size_t)n * PW, zeros + (size_t)n * PZ, scales + (size_t)n * G, K, order);
        if (accum) sum += q4o_h2f(y[n]) / (float)gpu_count;
        y[n] = q4o_f2h(sum);
    }
}

/* fp32 (unrounded) variant used to compare the CUDA kernels with the exact sum. */
void q4o_matvec_f32(float *y, const f16 *x, const uint32_t *weight, const uint32_t *zeros, const f16 *scales, int K, int N) {
    int PW = q4o_packed_wt_height(K), PZ = q4o_packed_zeros_height(K), G = q4o_groups(K);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const uint32_t *wr = weight + (size_t)n * PW, *zr = zeros + (size_t)n * PZ;
        const f16 *sr = scales + (size_t)n * G;
        double sum = 0.0;
        for (int k = 0; k < K; k++) {
            int g = k >> 7;
            double w = ((double)nib(wr, k) - (double)nib(zr, g)) * (double)q4o_h2f(sr[g]);
            sum += w * (double)q4o_h2f(x[k]);
        }
        y[n] = (float)sum;
    }
}

/* h = silu(Wg·x) * (Wu·x). gpu_kernels.h:264-283 (ffn_matvec_silu_kernel); llama2_q4.cu:393-404. */
void q4o_ffn_silu(f16 *h, const f16 *x, const uint32_t *gw, const uint32_t *gz, const f16 *gs,
                  const uint32_t *uw, const uint32_t *uz, const f16 *us, int K, int N, int order) {
    int PW = q4o_packed_wt_height(K), PZ = q4o_packed_zeros_height(K), G = q4o_groups(K);
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        float g = dot_q4(x, gw + (size_t)n * PW, gz + (size_t)n * PZ, gs + (size_t)n * G, K, order);
        float u = dot_q4(x, uw + (size_t)n * PW, uz + (size_t)n * PZ, us + (size_t)n * G, K, order);
        float val = g;
        val *= 1.0f / (1.0f + expf(-val));
        val *= u;
        h[n] = q4o_f2h(val);
    }
}

/* fp16 GEMV (classifier). gpu_kernels.h:117-147 (mat_vec_kernel); llama2_q4.cu:357-365. */
void q4o_matvec_f16(f16 *y, const f16 *x, const f16 *W, int K, int N, float alpha, int order) {
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        const f16 *wr = W + (size_t)n * K;
        float sum;
        if (order == 1) {
            float lane[32];
            int serial = div_up(div_up(K, 32), 8);
            for (int t = 0; t < 32; t++) {
                float s = 0.f;
                for (int i = 0; i < serial; i++) {
                    int j = (i * 32 + t) * 8;
                    if (j < K)
                        for (int e = 0; e < 8; e++) s = fmaf(q4o_h2f(wr[j + e]), q4o_h2f(x[j + e]), s);
                }
                lane[t] = s;
            }
            sum = warp_tree(lane);
        } else {
            sum = 0.f;
            for (int k = 0; k < K; k++) sum += q4o_h2f(wr[k]) * q4o_h2f(x[k]);
        }
        sum *= alpha;
        y[n] = q4o_f2h(sum);
    }
}

/* RMSNorm, eps 1e-5 added after the mean. gpu_kernels.h:72-105; llama2_q4.cu:347-350.
 * Summation order follows the kernel: thread t of 1024 sums x[t], x[t+1024], ...; warps are
 * tree-reduced and the 32 warp totals are added in warp order. */
void q4o_rmsnorm(f16 *o, const f16 *x, const f16 *w, int size) {
    float part[1024];
    for (int t = 0; t < 1024; t++) {
        float ss = 0.f;
        for (int i = t; i < size; i += 1024) {
            float v = q4o_h2f(x[i]);
            ss = fmaf(v, v, ss);
        }
        part[t] = ss;
    }
    float total = 0.f;
    for (int wp = 0; wp < 32; wp++) {
        float s = warp_tree(part + wp * 32);
        total = (wp == 0) ? s : total + s;
    }
    float ss = total / (float)size;
    ss += 1e-5f;
    ss = 1.0f / sqrtf(ss);
    for (int i = 0; i < size; i++) {
        float val = q4o_h2f(x[i]);
        val *= ss * q4o_h2f(w[i]);
        o[i] = q4o_f2h(val);
    }
}

/* rotate-half RoPE on q (n_heads) and on the K row (first n_kv_heads). gpu_kernels.h:340-363. */
void q4o_rope(f16 *q, f16 *k_row, int n_heads, int n_kv_heads, int head_size, int pos, float theta) {
    int half_hs = head_size / 2;
    for (int h = 0; h < n_heads; h++) {
        for (int i = 0; i < half_hs; i++) {
            int head_dim = (i * 2) % head_size;
            float freq = 1.0f / powf(theta, (float)head_dim / (float)head_size);
            float val = (float)pos * freq;
            float fcr = cosf(val), fci = sinf(val);
            f16 *v = q + (size_t)h * head_size;
            float q0 = q4o_h2f(v[i]), q1 = q4o_h2f(v[i + half_hs]);
            v[i] = q4o_f2h(q0 * fcr - q1 * fci);
            v[i + half_hs] = q4o_f2h(q0 * fci + q1 * fcr);
            if (h < n_kv_heads) {
                f16 *kk = k_row + (size_t)h * head_size;
                float k0 = q4o_h2f(kk[i]), k1 = q4o_h2f(kk[i + half_hs]);
                kk[i] = q4o_f2h(k0 * fcr - k1 * fci);
                kk[i + half_hs] = q4o_f2h(k0 * fci + k1 * fcr);
            }
        }
    }
}

/* Attention of one query over positions 0..pos. Scores and probabilities are rounded to fp16 as
 * the reference does. llama2_q4.cu:410-427; gpu_kernels.h:150-176 (scores), :365-409 (softmax),
 * :287-337 (weighted sum of V). kcache/vcache point at the layer; row stride kv_stride halfs. */
void q4o_attention(f16 *out, const f16 *q, const f16 *kcache, const f16 *vcache, int n_heads, int head_size,
                   int kv_mul, int kv_stride, int pos) {
    int T = pos + 1;
    float alpha = (float)(1.0 / sqrt((double)head_size));
#pragma omp parallel
    {
        float *att = (float *)malloc(sizeof(float) * (size_t)T);
        f16 *p16 = (f16 *)malloc(sizeof(f16) * (size_t)T);
#pragma omp for schedule(static)
        for (int h = 0; h < n_heads; h++) {
            const f16 *qh = q + (size_t)h * head_size;
            int kvh = h / kv_mul;
            for (int t = 0; t < T; t++) {
                const f16 *kr = kcache + (size_t)t * kv_stride + (size_t)kvh * head_size;
                float lane[32];
                for (int l = 0; l < 32; l++) {
                    float s = 0.f;
                    for (int j = l; j < head_size; j += 32) s = fmaf(q4o_h2f(kr[j]), q4o_h2f(qh[j]), s);
                    lane[l] = s;
                }
                float sc = warp_tree(lane) * alpha;
                att[t] = q4o_h2f(q4o_f2h(sc));
            }
            float mx = att[0];
            for (int t = 1; t < T; t++) if (att[t] > mx) mx = att[t];
            float sum = 0.f;
            for (int t = 0; t < T; t++) { att[t] = expf(att[t] - mx); sum += att[t]; }
            for (int t = 0; t < T; t++) p16[t] = q4o_f2h(att[t] / sum);
            for (int n = 0; n < head_size; n++) {
                float acc = 0.f;
                for (int t = 0; t < T; t++)
                    acc += q4o_h2f(vcache[(size_t)t * kv_stride + (size_t)kvh * head_size + n]) * q4o_h2f(p16[t]);
                out[(size_t)h * head_size + n] = q4o_f2h(acc);
            }
        }
        free(att);
        free(p16);
    }
}

/* Greedy argmax over fp16 logits, lowest index among equals. gpu_kernels.h:456-501; sampler.h:77-84. */
int q4o_argmax(const f16 *x, int n) {
    int best = 0;
    float bv = q4o_h2f(x[0]);
    for (int i = 1; i < n; i++) {
        float v = q4o_h2f(x[i]);
        if (v > bv) { bv = v; best = i; }
    }
    return best;
}

/* xorshift* generator and coin of the sampler. sampler.h:66-75. */
unsigned int q4o_random_u32(unsigned long long *state) {
    *state ^= *state >> 12;
    *state ^= *state << 25;
    *state ^= *state >> 27;
    return (unsigned int)((*state * 0x2545F4914F6CDD1Dull) >> 32);
}
float q4o_random_f32(unsigned long long *state) { return (q4o_random_u32(state) >> 8) / 16777216.0f; }

static unsigned long long q4o_prob_units(f16 h) { /* fp16 in [0,1] as a multiple of 2^-24 */
    unsigned e = (h >> 10) & 31u, mnt = h & 1023u;
    return e == 0 ? (unsigned long long)mnt : (unsigned long long)(1024u + mnt) << (e - 1);
}

/* Butterfly sum over 32 values, pairs (l, l^16), (l, l^8) ... (l, l^1): the order of a warp's xor-shuffle reduction. */
static float q4o_butterfly32(float *v) {
    for (int o = 16; o > 0; o >>= 1) {
        float t[32];
        for (int l = 0; l < 32; l++) t[l] = v[l] + v[l ^ o];
        for (int l = 0; l < 32; l++) v[l] = t[l];
    }
    return v[0];
}

/* Non-greedy branch of sample(): sampler.h:85-115; softmax_logits_kernel gpu_kernels.h:507-556 (temperature, fp16
 * rounding after the division, after exp and after the normalisation; the sum is taken over the unrounded exps);
 * order and threshold sampler.h:92-104 (stable descending sort when 0 < topp < 1, threshold coin*topp; index order and
 * threshold coin otherwise); selection sample_top_p_kernel gpu_kernels.h:561-592 (first position whose inclusive prefix
 * sum >= threshold, else the last position). logits are replaced by the probabilities, as in the reference.
 * Two choices where the reference leaves the order open: the sum of exps is taken per 1024-strided lane, then by
 * butterfly over 32 lanes and over 32 warps (the CUDA kernel's order); the prefix sum is exact integer arithmetic on
 * multiples of 2^-24 (the reference's device-wide scan accumulates in fp16 in an unspecified order). */
int q4o_sample_topp(f16 *logits, int n, float temperature, float topp, float coin) {
    float mx = -INFINITY;
    for (int i = 0; i < n; i++) {
        float val = q4o_h2f(logits[i]);
        val /= temperature;
        logits[i] = q4o_f2h(val);
        if (q4o_h2f(logits[i]) > mx) mx = q4o_h2f(logits[i]);
    }
    float part[1024];
    for (int t = 0; t < 1024; t++) part[t] = 0.f;
    for (int i = 0; i < n; i++) {
        float v = expf(q4o_h2f(logits[i]) - mx);
        logits[i] = q4o_f2h(v);
        part[i & 1023] += v; /* lane t sums i = t, t+1024, ... in order */
    }
    float wsum[32];
    for (int w = 0; w < 32; w++) wsum[w] = q4o_butterfly32(part + 32 * w);
    const float sum = q4o_butterfly32(wsum);
    for (int i = 0; i < n; i++) logits[i] = q4o_f2h(q4o_h2f(logits[i]) / sum);

    const int sorted = topp > 0.f && topp < 1.f;
    const float threshold = sorted ? coin * topp : coin;
    double td = ceil((double)threshold * 16777216.0);
    unsigned long long need = td <= 1.0 ? 1ull : (td >= 9.0e18 ? ~0ull : (unsigned long long)td);
    if (!sorted) {
        if (!(threshold > 0.f)) return 0; /* prefix >= 0 holds at the first element whatever its probability */
        unsigned long long c = 0;
        for (int i = 0; i < n; i++) {
            c += q4o_prob_units(logits[i]);
            if (c >= need) return i;
        }
        return n - 1;
    }
    /* stable descending order by probability: counting sort on the fp16 bit pattern (non-negative values) */
    int *order = (int *)malloc(sizeof(int) * (size_t)n);
    int *start = (int *)calloc(65537, sizeof(int));
    for (int i = 0; i < n; i++) start[65535 - logits[i]]++;
    int acc = 0;
    for (int k = 0; k < 65536; k++) { int c = start[k]; start[k] = acc; acc += c; }
    for (int i = 0; i < n; i++) order[start[65535 - logits[i]]++] = i;
    unsigned long long c = 0;
    int res = order[n - 1];
    for (int t = 0; t < n; t++) {
        c += q4o_prob_units(logits[order[t]]);
        if (c >= need) { res = order[t]; break; }
    }
    free(order);
    free(start);
    return res;
}

/* ------------------------------------------------------------------------------------------
 * Whole model on the packed file image (tensor order: weight_packer.cpp:256-291 written,
 * llama2_q4.cu:220-246 read). The image is the file's bytes in memory.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    int dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_theta;
} q4o_config; /* common.h:15-24 */

typedef struct { const uint32_t *w, *z; const f16 *s; } q4o_qw;
typedef struct { q4o_qw q, k, v, o, up, gate, down; const f16 *rms_att, *rms_ffn; } q4o_layer;

typedef struct {
    q4o_config cfg;
    const f16 *emb, *wcls, *rms_final;
    q4o_layer *layers;
    /* run state, common.h:62-78 */
    f16 *x, *xb, *hb, *q, *logits, *kc, *vc;
} q4o_model;

size_t q4o_qweight_bytes(int K, int N) {
    return (size_t)N * ((size_t)q4o_packed_wt_height(K) * 4 + (size_t)q4o_packed_zeros_height(K) * 4 + (size_t)q4o_groups(K) * 2);
}

size_t q4o_file_bytes(const q4o_config *c) {
    int kv_dim = c->dim * c->n_kv_heads / c->n_heads;
    size_t per_layer = 2 * q4o_qweight_bytes(c->dim, c->dim) + 2 * q4o_qweight_bytes(c->dim, kv_dim) +
                       2 * q4o_qweight_bytes(c->dim, c->hidden_dim) + q4o_qweight_bytes(c->hidden_dim, c->dim) +
                       4 * (size_t)c->dim;
    return 32 + 4 * (size_t)c->vocab_size * c->dim + 2 * (size_t)c->dim + per_layer * c->n_layers;
}

static const uint8_t *take_q(const uint8_t *p, q4o_qw *w, int K, int N) {
    w->w = (const uint32_t *)p; p += (size_t)N * q4o_packed_wt_height(K) * 4;
    w->z = (const uint32_t *)p; p += (size_t)N * q4o_packed_zeros_height(K) * 4;
    w->s = (const f16 *)p;      p += (size_t)N * q4o_groups(K) * 2;
    return p;
}

q4o_model *q4o_model_open(const uint8_t *image, size_t bytes) {
    if (bytes < 32) return NULL;
    q4o_model *m = (q4o_model *)calloc(1, sizeof(q4o_model));
    memcpy(&m->cfg, image, 32);
    const q4o_config *c = &m->cfg;
    if (c->dim <= 0 || c->n_heads <= 0 || c->n_layers <= 0 || q4o_file_bytes(c) != bytes) { free(m); return NULL; }
    int kv_dim = c->dim * c->n_kv_heads / c->n_heads;
    const uint8_t *p = image + 32;
    m->emb = (const f16 *)p;  p += 2 * (size_t)c->vocab_size * c->dim;
    m->wcls = (const f16 *)p; p += 2 * (size_t)c->vocab_size * c->dim;
    m->rms_final = (const f16 *)p; p += 2 * (size_t)c->dim;
    m->layers = (q4o_layer *)calloc((size_t)c->n_layers, sizeof(q4o_layer));
    for (int l = 0; l < c->n_layers; l++) {
        q4o_layer *L = &m->layers[l];
        p = take_q(p, &L->q, c->dim, c->dim);
        p = take_q(p, &L->k, c->dim, kv_dim);
        p = take_q(p, &L->v, c->dim, kv_dim);
        p = take_q(p, &L->o, c->dim, c->dim);
        p = take_q(p, &L->up, c->dim, c->hidden_dim);   /* up precedes gate in the file */
        p = take_q(p, &L->gate, c->dim, c->hidden_dim);
        p = take_q(p, &L->down, c->hidden_dim, c->dim);
        L->rms_att = (const f16 *)p; p += 2 * (size_t)c->dim;
        L->rms_ffn = (const f16 *)p; p += 2 * (size_t)c->dim;
    }
    m->x = (f16 *)calloc((size_t)c->dim, 2);
    m->xb = (f16 *)calloc((size_t)c->dim, 2);
    m->q = (f16 *)calloc((size_t)c->dim, 2);
    m->hb = (f16 *)calloc((size_t)c->hidden_dim, 2);
    m->logits = (f16 *)calloc((size_t)c->vocab_size, 2);
    m->kc = (f16 *)calloc((size_t)c->n_layers * c->seq_len * kv_dim, 2);
    m->vc = (f16 *)calloc((size_t)c->n_layers * c->seq_len * kv_dim, 2);
    return m;
}

void q4o_model_close(q4o_model *m) {
    if (!m) return;
    free(m->layers); free(m->x); free(m->xb); free(m->q); free(m->hb); free(m->logits); free(m->kc); free(m->vc);
    free(m);
}

const f16 *q4o_model_logits(const q4o_model *m) { return m->logits; }
const f16 *q4o_model_x(const q4o_model *m) { return m->x; }

/* One token at position pos, single GPU math (gpu_count = 1). llama2_q4.cu:430-538. Returns argmax. */
int q4o_model_forward(q4o_model *m, int token, int pos, int order) {
    const q4o_config *c = &m->cfg;
    int dim = c->dim, hid = c->hidden_dim;
    int hs = dim / c->n_heads;
    int kv_dim = dim * c->n_kv_heads / c->n_heads;
    int kv_mul = c->n_heads / c->n_kv_heads;
    memcpy(m->x, m->emb + (size_t)token * dim, 2 * (size_t)dim); /* gpu_kernels.h:61-69 */
    for (int l = 0; l < c->n_layers; l++) {
        const q4o_layer *L = &m->layers[l];
        size_t loff = (size_t)l * c->seq_len * kv_dim;
        f16 *krow = m->kc + loff + (size_t)pos * kv_dim;
        f16 *vrow = m->vc + loff + (size_t)pos * kv_dim;
        q4o_rmsnorm(m->xb, m->x, L->rms_att, dim);
        q4o_matvec(m->q, m->xb, L->q.w, L->q.z, L->q.s, dim, dim, 0, 1, order);
        q4o_matvec(krow, m->xb, L->k.w, L->k.z, L->k.s, dim, kv_dim, 0, 1, order);
        q4o_matvec(vrow, m->xb, L->v.w, L->v.z, L->v.s, dim, kv_dim, 0, 1, order);
        q4o_rope(m->q, krow, c->n_heads, c->n_kv_heads, hs, pos, c->rope_theta);
        q4o_attention(m->xb, m->q, m->kc + loff, m->vc + loff, c->n_heads, hs, kv_mul, kv_dim, pos);
        q4o_matvec(m->x, m->xb, L->o.w, L->o.z, L->o.s, dim, dim, 1, 1, order);
        q4o_rmsnorm(m->xb, m->x, L->rms_ffn, dim);
        q4o_ffn_silu(m->hb, m->xb, L->gate.w, L->gate.z, L->gate.s, L->up.w, L->up.z, L->up.s, dim, hid, order);
        q4o_matvec(m->x, m->hb, L->down.w, L->down.z, L->down.s, hid, dim, 1, 1, order);
    }
    q4o_rmsnorm(m->x, m->x, m->rms_final, dim);
    q4o_matvec_f16(m->logits, m->x, m->wcls, dim, c->vocab_size, 1.0f, order);
    return q4o_argmax(m->logits, c->vocab_size);
}

/* Sum of g partial fp16 vectors the way cuda_comm.h:193-219 does on rank `rank`:
 * start from the rank's own vector, add peers in ascending rank order with fp16 adds. */
void q4o_allreduce_ref_order(f16 *out, const f16 *parts, int g, int rank, int count) {
    for (int i = 0; i < count; i++) {
        f16 acc = parts[(size_t)rank * count + i];
        for (int r = 0; r < g; r++) {
            if (r == rank) continue;
            acc = q4o_f2h(q4o_h2f(acc) + q4o_h2f(parts[(size_t)r * count + i]));
        }
        out[i] = acc;
    }
}

int q4o_num_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
