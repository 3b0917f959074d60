// Counter-based synthetic model generator on the device: every tensor element is a function of (seed, tensor id,
// logical element index), so a rank fills exactly its own shard without any file and all ranks / tensor-parallel
// degrees hold shards of one and the same model (a 70B model would otherwise need a 36 GB file read through host
// memory, as build_transformer does, llama2_q4.cu:645-646). Stand-in for real AWQ checkpoints, which need a network
// to fetch. Value distributions: packed weight words uniform (nibbles uniform on 0..15), zero points uniform on
// 0..15, scales fp16 of U[0.002, 0.02), embeddings and classifier fp16 of 0.02 * (sum of twelve uniforms - 6), i.e.
// normal to a very good approximation, using integer arithmetic and one multiply only, so that a host twin of the
// generator (synth.py) reproduces every bit.
#include "q4_model.h"

namespace {

__host__ __device__ __forceinline__ unsigned long long synth_hash(unsigned long long seed, unsigned long long tid, unsigned long long idx) {
    unsigned long long z = seed + tid * 0x9E3779B97F4A7C15ULL + idx * 0xD1B54A32D192ED03ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

// dst[n][j], j < pw_local: word (n0 + n, j0 + j) of the logical matrix; words past the shard's inputs are zero
__global__ void synth_words_kernel(uint32_t* dst, long long total, int pw_local, int valid_words, unsigned long long seed, int tid, long long n0,
                                   int pw_full, int j0) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / pw_local;
        const int j = (int)(i - n * pw_local);
        dst[i] = j < valid_words ? (uint32_t)synth_hash(seed, tid, (unsigned long long)((n0 + n) * pw_full + j0 + j)) : 0u;
    }
}

// zero points, re-packed for the shard: nibble g of row n = zero point of logical group g0 + g; unused nibbles are zero
__global__ void synth_zeros_kernel(uint32_t* dst, long long total, int pz_local, int groups_local, unsigned long long seed, int tid, long long n0,
                                   int groups_full, int g0) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / pz_local;
        const int jz = (int)(i - n * pz_local);
        uint32_t w = 0;
        for (int k = 0; k < 8; k++) {
            const int g = jz * 8 + k;
            if (g < groups_local) w |= (uint32_t)(synth_hash(seed, tid, (unsigned long long)((n0 + n) * groups_full + g0 + g)) & 15u) << (4 * k);
        }
        dst[i] = w;
    }
}

__global__ void synth_scales_kernel(__half* dst, long long total, int groups_local, unsigned long long seed, int tid, long long n0, int groups_full,
                                    int g0) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / groups_local;
        const int g = (int)(i - n * groups_local);
        const unsigned u = (unsigned)(synth_hash(seed, tid, (unsigned long long)((n0 + n) * groups_full + g0 + g)) >> 40);   // 24 bits
        // separate multiply and add (no contraction to an FMA): the host twin rounds twice as well
        dst[i] = __float2half_rn(__fadd_rn(0.002f, __fmul_rn(0.018f, (float)u * (1.0f / 16777216.0f))));
    }
}

__global__ void synth_normal_kernel(__half* dst, long long total, long long idx0, unsigned long long seed, int tid) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        int s = 0;
        for (int k = 0; k < 3; k++) {
            const unsigned long long h = synth_hash(seed, tid, (unsigned long long)((idx0 + i) * 4 + k));
            s += (int)(h & 0xFFFFu) + (int)((h >> 16) & 0xFFFFu) + (int)((h >> 32) & 0xFFFFu) + (int)(h >> 48);
        }
        dst[i] = __float2half_rn(__fmul_rn((float)(s - 393210), 0.02f / 65536.0f));
    }
}

__global__ void synth_const_kernel(uint16_t* dst, int n, uint16_t v) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = v;
}

int blocks_for(long long total) { return (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16); }

}  // namespace

int q4_synth_qweight(uint32_t* w, uint32_t* z, uint16_t* s, int K_full, int K, int k_begin, int N, int n_begin, unsigned long long seed, int tid) {
    const int pw = q4_pw(K), pz = q4_pz(K), gg = q4_groups(K);
    const long long nw = (long long)N * pw, nz = (long long)N * pz, ns = (long long)N * gg;
    synth_words_kernel<<<blocks_for(nw), 256>>>(w, nw, pw, (K + 7) / 8, seed, tid, n_begin, q4_pw(K_full), k_begin / 8);
    synth_zeros_kernel<<<blocks_for(nz), 256>>>(z, nz, pz, gg, seed, tid + 1, n_begin, q4_groups(K_full), k_begin / 128);
    synth_scales_kernel<<<blocks_for(ns), 256>>>((__half*)s, ns, gg, seed, tid + 2, n_begin, q4_groups(K_full), k_begin / 128);
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}

int q4_synth_normal(uint16_t* dst, long long count, long long idx0, unsigned long long seed, int tid) {
    synth_normal_kernel<<<blocks_for(count), 256>>>((__half*)dst, count, idx0, seed, tid);
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}

int q4_synth_const(uint16_t* dst, int n, uint16_t value) {
    synth_const_kernel<<<blocks_for(n), 256>>>(dst, n, value);
    Q4_CUDA_TRY(cudaGetLastError());
    return Q4_OK;
}
