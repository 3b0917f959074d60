// Internal model structures shared by the host code (q4_model.cu) and the fused decode kernel (q4_fused.cu).
#pragma once
#include <vector>

#include "q4_common.cuh"
#include "q4_comm_internal.h"

struct DevQW {
    q4_qweight w;
    int K, N;  // local (shard) dims
};

struct DevLayer {
    DevQW q, k, v, o, gate, up, down;
    uint16_t *rms_att, *rms_ffn;
};

static inline size_t qw_bytes(int K, int N) { return (size_t)N * ((size_t)q4_pw(K) * 4 + (size_t)q4_pz(K) * 4 + (size_t)q4_groups(K) * 2); }
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct q4_fused;  // state of the fused (persistent-kernel) path, q4_fused.cu
struct q4_rows;   // row buffers of the prefill / batched-decode path, q4_batch.cu

struct q4_model {
    q4_config cfg;
    int rank, g, tp_mode;
    q4_comm* comm;
    // shard geometry
    int head_size, kv_dim, kv_mul;
    int q_n, kv_n;            // local q / kv outputs
    int o_kb, o_kc;           // local slice of the attention output vector (inputs of o_proj)
    int h_kb, h_kc;           // local slice of the hidden vector (outputs of gate/up, inputs of down)
    int v_n;                  // local classifier rows
    bool column;              // -x column (llama2_q4.cu:479-493, 510-524): every matrix split by output columns, four all-gathers per layer
    // device memory
    char* arena;
    size_t arena_bytes;
    uint16_t *emb, *wcls, *rms_final;
    std::vector<DevLayer> layers;
    uint16_t *x, *xb, *hb, *q, *logits, *kc, *vc;
    float* attn_scratch;
    int* pos;
    q4_shared_data* shared;
    cudaGraphExec_t graph[3];   // prompt phase, generating (argmax), generating without the hand-off (a sampler follows)
    bool graph_ready[3];
    // sampler state (sampler.h:10-19): temperature 0 = greedy
    float temperature, topp;
    unsigned long long rng_state;
    q4_fused* fused;
    q4_rows* rows;
    int host_pos;               // forward calls since the last reset + the reset's position (bounds the K/V row written)
};

// q4_fused.cu
int q4_fused_prepare(q4_model* m);                              // builds the stream-layout weights and the phase table (lazy)
int q4_fused_forward(q4_model* m, cudaStream_t s, int gen_token, int no_handoff);
void q4_fused_reset(q4_model* m);                               // re-arms barrier counters (after q4_model_reset)
void q4_fused_free(q4_model* m);
int q4_fused_status(q4_model* m);
void q4_rows_free(q4_model* m);   // q4_batch.cu
int q4_rows_status(q4_model* m);
void q4_fused_set_wait_limit(q4_model* m, unsigned long long ns);   // device-side wait limit of the fused kernel (0 = default)

// q4_synth.cu: counter-based synthetic tensors generated on the device, shard by shard (see q4_model_create_synthetic)
int q4_synth_qweight(uint32_t* w, uint32_t* z, uint16_t* s, int K_full, int K, int k_begin, int N, int n_begin, unsigned long long seed, int tid);
int q4_synth_normal(uint16_t* dst, long long count, long long idx0, unsigned long long seed, int tid);
int q4_synth_const(uint16_t* dst, int n, uint16_t value);
