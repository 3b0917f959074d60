// Shared device helpers for the sm_100a decode kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/q4b200.h"

#define Q4_CUDA_TRY(call)                                   \
    do {                                                    \
        cudaError_t e__ = (call);                           \
        if (e__ != cudaSuccess) { q4_note_cuda_error(e__, __FILE__, __LINE__); return Q4_ERR_CUDA; } \
    } while (0)

void q4_note_cuda_error(cudaError_t e, const char* file, int line);

static inline int q4_div_up(int a, int b) { return (a - 1) / b + 1; }
static inline int q4_pw(int K) { return q4_div_up(K, 32) * 4; }              // words per weight row
static inline int q4_groups(int K) { return q4_div_up(K, 128); }             // scales per row
static inline int q4_pz(int K) { return q4_div_up(q4_div_up(K, 128), 8); }   // words per zeros row

// Launch attribute helper: programmatic dependent launch lets the next kernel's blocks start (and stream
// their weights) while the previous kernel drains; the kernel calls griddep_wait() before touching anything
// the previous kernel produced.
struct Q4Launch {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    Q4Launch(dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl = true) {
        cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
};

#ifdef __CUDACC__

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Streaming 128-bit load for weights: read once per token, keep them out of L1.
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

__device__ __forceinline__ __half2 u2h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t h22u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// x pairs as the nibble unpack produces them: a word holds q0..q7; the 0x000F000F mask yields (q0,q4),
// the 0x00F000F0 mask (q1,q5), and after >>8 (q2,q6), (q3,q7). xp[0..3] = (x0,x4),(x1,x5),(x2,x6),(x3,x7).
__device__ __forceinline__ void permute_x8(const uint4& xv, uint32_t xp[4]) {
    xp[0] = prmt(xv.x, xv.z, 0x5410);
    xp[1] = prmt(xv.x, xv.z, 0x7632);
    xp[2] = prmt(xv.y, xv.w, 0x5410);
    xp[3] = prmt(xv.y, xv.w, 0x7632);
}

// Zero-point constants for one group: zlo = (1024+z, 1024+z), zhi = (-(64+z), -(64+z)) as half2 bits.
__device__ __forceinline__ void zero_consts(uint32_t z, uint32_t& zlo, uint32_t& zhi) {
    zlo = (0x6400u | z) * 0x00010001u;
    zhi = (0xD400u | (z << 4)) * 0x00010001u;
}

// Dot product of 8 nibbles (one packed word) minus zero point with 8 activations, as a half2 pair of partial
// sums (4 products per half). (w & 0x000F000F) | 0x6400 is the half 1024+q, so subtracting 1024+z gives q-z
// exactly; (w & 0x00F000F0) | 0x6400 is 1024+16q, and fma(., 1/16, -(64+z)) gives q-z exactly.
__device__ __forceinline__ __half2 dot8(uint32_t w, const uint32_t xp[4], uint32_t zlo, uint32_t zhi, __half2 acc) {
    const __half2 sixteenth = u2h2(0x2C002C00u);
    __half2 d0 = __hsub2(u2h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), u2h2(zlo));
    __half2 d1 = __hfma2(u2h2(lop3_and_or(w, 0x00F000F0u, 0x64006400u)), sixteenth, u2h2(zhi));
    w >>= 8;
    __half2 d2 = __hsub2(u2h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), u2h2(zlo));
    __half2 d3 = __hfma2(u2h2(lop3_and_or(w, 0x00F000F0u, 0x64006400u)), sixteenth, u2h2(zhi));
    acc = __hfma2(d0, u2h2(xp[0]), acc);
    acc = __hfma2(d1, u2h2(xp[1]), acc);
    acc = __hfma2(d2, u2h2(xp[2]), acc);
    acc = __hfma2(d3, u2h2(xp[3]), acc);
    return acc;
}

__device__ __forceinline__ float h2sum(__half2 h) {
    float2 f = __half22float2(h);
    return f.x + f.y;
}

// Rotation of pair `pair` (elements pair and pair + head_size / 2) of a head at position `pos`: angle =
// pos / theta^(2 pair / head_size), evaluated in fp32 with powf, cosf and sinf exactly as RoPERotation_kernel evaluates it
// (gpu_kernels.h:346-350), so that rotated values round as the reference's do. Returns (cos, sin).
__device__ __forceinline__ float2 rope_cos_sin(int pos, int pair, int head_size, float theta) {
    const int even_dim = (2 * pair) % head_size;
    const float inv_wavelength = 1.0f / powf(theta, even_dim / (float)head_size);
    const float angle = pos * inv_wavelength;
    return make_float2(cosf(angle), sinf(angle));
}
// (lo, hi) <- (lo cos - hi sin, lo sin + hi cos), fp32 inside, each rounded to fp16 once
__device__ __forceinline__ void rope_rotate(const __half* src_lo, const __half* src_hi, __half* dst_lo, __half* dst_hi, float2 cs) {
    const float a = __half2float(*src_lo), b = __half2float(*src_hi);
    *dst_lo = __float2half(a * cs.x - b * cs.y);
    *dst_hi = __float2half(a * cs.y + b * cs.x);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

#endif  // __CUDACC__
