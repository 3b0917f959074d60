/*
 * q4b200 - C ABI of the B200 (sm_100a) decode path for AWQ W4 g128 Llama-2 models in the
 * llama_cu_awq packed file format.
 *
 * Every entry point replaces one host wrapper of the reference program (cited per function as
 * file:line within the llama_cu_awq project). Conventions:
 *   - plain pointers and sizes only; `stream` is a cudaStream_t passed as void*;
 *   - fp16 data is passed as uint16_t* (IEEE binary16 bits);
 *   - all data pointers are device pointers of the current device unless a comment says
 *     "pinned host"; the caller owns every buffer;
 *   - calls are asynchronous on `stream`; nothing is allocated by the per-token entry points;
 *   - the return value is a status code (Q4_OK = 0). The reference prints a message and calls
 *     exit() where these functions return Q4_ERR_UNSUPPORTED_SIZE / Q4_ERR_CUDA;
 *   - the token position is never passed by value on the per-token path: kernels read it from
 *     device memory (`pPos`), as the reference's kernels do, so that a captured CUDA graph
 *     can be replayed for every token.
 * There is no CPU fallback: without a CUDA device every compute entry point returns Q4_ERR_CUDA.
 */
#ifndef Q4B200_H
#define Q4B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define Q4_OK 0
#define Q4_ERR_UNSUPPORTED_SIZE 1 /* reference: "Unsupported matmul size. Exiting" (llama2_q4.cu:358,368,379,394) */
#define Q4_ERR_CUDA 2             /* reference: CUDA_CHECK -> exit (llama2_q4.cu:35-43) */
#define Q4_ERR_IO 3               /* reference: "Couldn't open file" / "error reading weights" -> exit (llama2_q4.cu:203-208,629-631) */
#define Q4_ERR_BAD_MODEL 4        /* header or file length inconsistent */
#define Q4_ERR_INVALID 5          /* bad argument */
#define Q4_ERR_TIMEOUT 6          /* a bounded device-side wait (peer flag) ran out */
#define Q4_ERR_LIMIT 7            /* request exceeds a fixed capacity of the entry point */

#define Q4_GROUP_SIZE 128 /* llama2_q4.cu:31, weight_packer.cpp:7 */
#define Q4_MAX_GPUS 8     /* cuda_comm.h:16 */
#define Q4_MAX_SEQ_LEN (128 * 1024) /* common.h:13 */

/* Model-config header: the first 32 bytes of the packed file. common.h:15-24, weight_packer.cpp:9-18. */
typedef struct {
    int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_theta;
} q4_config;

/* One quantized matrix, K inputs x N outputs, K-contiguous per output. common.h:26-30.
 *   weight u32[N][4*ceil(K/32)]  nibble i of word j holds q(n, 8j+i)
 *   zeros  u32[N][ceil(ceil(K/128)/8)]
 *   scales f16[N][ceil(K/128)] */
typedef struct {
    const uint32_t* weight;
    const uint32_t* zeros;
    const uint16_t* scales;
} q4_qweight;

/* CPU<->GPU mailbox in pinned host memory. common.h:57-60. */
typedef struct {
    volatile int32_t pos;
    int32_t tokens[Q4_MAX_SEQ_LEN];
} q4_shared_data;

const char* q4_status_string(int status);
/* Library/ABI version and the SM architecture the kernels were built for ("sm_100a"). */
int q4_abi_version(void);
const char* q4_build_arch(void);

/* ---------------------------------------------------------------------------------------------
 * Per-op entry points: the op-wrapper boundary of llama2_q4.cu:347-427 and sampler.h:77-84.
 * ------------------------------------------------------------------------------------------- */

/* rmsnorm(): llama2_q4.cu:347-350, kernel gpu_kernels.h:72-105. o = x * rsqrt(mean(x^2) + 1e-5) * weight. */
int q4_rmsnorm(void* stream, uint16_t* o, const uint16_t* x, const uint16_t* weight, int size);

/* matmul(QWeight): llama2_q4.cu:367-376, kernels gpu_kernels.h:179-248.
 * xout[n] = sum_k (q(n,k) - z(n,k/128)) * s(n,k/128) * x[k]; when accum != 0 the old xout[n] / gpu_count
 * is added first (fused residual); when loff != -1 the result is written at xout + loff + (*pPos) * opSize
 * (KV-cache row). inpSize and opSize must be multiples of 8. */
int q4_matmul_q4(void* stream, uint16_t* xout, const uint16_t* x, const q4_qweight* w, int inpSize, int opSize,
                 int accum, int gpu_count, int loff, const int* pPos);

/* qkv_matvec(): llama2_q4.cu:378-391, kernel gpu_kernels.h:250-262. Three projections of the same x in one
 * launch; K and V land in cache row *pPos at offset loff. Unlike the reference, kvSize may differ from opSize
 * (grouped-query models; the reference issues three matmul() calls there, llama2_q4.cu:457-459). */
int q4_qkv_matvec(void* stream, uint16_t* q, uint16_t* key_cache, uint16_t* value_cache, const uint16_t* x,
                  const q4_qweight* qw, const q4_qweight* kw, const q4_qweight* vw, int inpSize, int opSize,
                  int kvSize, int loff, const int* pPos);

/* ffn_matvec_silu(): llama2_q4.cu:393-404, kernel gpu_kernels.h:264-283. xout = silu(gate·x) * (up·x). */
int q4_ffn_matvec_silu(void* stream, uint16_t* xout, const uint16_t* x, const q4_qweight* gate_w,
                       const q4_qweight* up_w, int inpSize, int opSize);

/* RoPERotation(): llama2_q4.cu:406-408, kernel gpu_kernels.h:340-363. Rotates q (num_heads heads) and the K row
 * just written at k + loff + (*pPos) * num_kv_heads * head_size (first num_kv_heads heads), in place. */
int q4_rope(void* stream, uint16_t* q, uint16_t* k, int num_heads, int num_kv_heads, int head_size, const int* pPos,
            int loff, float rope_theta);

/* MultiHeadAttention(): llama2_q4.cu:410-427, kernels gpu_kernels.h:150-176,365-454,287-337.
 * One query per head over cache rows 0..*pPos; key_cache/value_cache already point at the layer; the row
 * stride is num_heads*head_size/kv_mul halfs. `scratch` replaces the reference's `att` buffer and must hold
 * q4_attention_scratch_bytes(num_heads, head_size) bytes; it carries the per-split partial results. */
size_t q4_attention_scratch_bytes(int num_heads, int head_size);
int q4_attention(void* stream, uint16_t* output, const uint16_t* q, const uint16_t* key_cache,
                 const uint16_t* value_cache, void* scratch, int num_heads, int head_size, int kv_mul, int max_seq_len,
                 const int* pPos);

/* Same computation as q4_attention for callers that cannot provide the scratch buffer because they may not
 * allocate device memory: hosts whose device memory is completely handed out at start-up, or plugins that only
 * receive the owning runtime's pointers. No counterpart in the reference (its `att` buffer is allocated by
 * malloc_run_state). The partial results go to an array of Q4_ATTENTION_STATIC_MAX_BYTES that is part of the
 * library's device image (every GPU that loads the library holds it until the process exits); shapes that need
 * more (q4_attention_scratch_bytes) are refused with Q4_ERR_LIMIT. The call allocates and frees nothing.
 * The first call on each device looks the array's device address up (cudaGetSymbolAddress); make that first call
 * outside of any stream capture. All calls share the one array: two calls that overlap on the GPU (different
 * streams) race; calls on one stream are safe. Nothing has to be cleared between calls: each call overwrites
 * every word it later reads. The array's address is remembered per CUDA device ordinal of the calling thread's
 * current device, which must be the device `stream` belongs to; the remembered address does not survive
 * cudaDeviceReset() (do not call this entry point again in a process that has reset the device). */
#define Q4_ATTENTION_STATIC_MAX_BYTES (256 * 1024)
int q4_attention_static(void* stream, uint16_t* output, const uint16_t* q, const uint16_t* key_cache,
                        const uint16_t* value_cache, int num_heads, int head_size, int kv_mul, int max_seq_len,
                        const int* pPos);

/* Batched form of matmul(QWeight) for prompt (prefill) and multi-sequence batches: Y[M][opSize] = X[M][inpSize] * deq(W),
 * row m being what q4_matmul_q4 computes for x = X[m] (accum = 0). The reference has no such path: it pushes a prompt
 * through the batch-1 kernel token by token (llama2_q4.cu:710-735); this is the dense contraction on the tensor cores
 * (tcgen05.mma with TMEM accumulators, operands staged by TMA). inpSize must be a multiple of 128, opSize of 8; x, y
 * row-major fp16, 16-byte aligned. `weight_interleaved` is either NULL (the packed words of `w` are used as they lie in
 * the file) or a copy of w->weight made by q4_gemm_interleave_weights, which saves the kernel four byte permutes per
 * packed word. `workspace` (device memory, 16-byte aligned, q4_matmul_q4_batched_workspace_bytes(M, inpSize, opSize) bytes,
 * caller-owned, not shared between calls that overlap on the GPU) holds a status word, tile counters and the fp32
 * partial sums of the K split; zero it once before the first call (and again after a reported time-out). Asynchronous on `stream`; q4_matmul_q4_batched_status synchronises the stream and returns
 * Q4_OK or the Q4_ERR_TIMEOUT a bounded device-side wait recorded. */
size_t q4_matmul_q4_batched_workspace_bytes(int M, int inpSize, int opSize);
int q4_gemm_interleave_weights(void* stream, uint32_t* dst, const uint32_t* weight, int inpSize, int opSize);
int q4_matmul_q4_batched(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* w, const uint32_t* weight_interleaved,
                         int M, int inpSize, int opSize, void* workspace, size_t workspace_bytes);
/* The same with the fused residual of matmul(QWeight)'s accum form (gpu_kernels.h:237-238) for every row:
 * y = product + residual * residual_scale, rounded to fp16 once; residual is [M][opSize] and may be y itself. */
int q4_matmul_q4_batched_residual(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* w,
                                  const uint32_t* weight_interleaved, int M, int inpSize, int opSize, const uint16_t* residual,
                                  float residual_scale, void* workspace, size_t workspace_bytes);
int q4_matmul_q4_batched_status(void* stream, const void* workspace);

/* The same products for a handful of rows (1 <= M <= 16): the projections of batched decode, where every sequence adds one
 * row and the weights are still read once per step. HBM-bound like the batch-1 kernels they widen (mat_vec_kernel_int4,
 * qkv_matvec_kernel, ffn_matvec_silu_kernel: gpu_kernels.h:179-283), so no tcgen05 tiles here: packed words straight from
 * global memory into mma.sync fragments, fp32 accumulation, group scale applied in fp32, no workspace, results
 * bit-reproducible. x is [M][inpSize], every y [M][its opSize], row-major fp16; inpSize a multiple of 128.
 *   q4_matmul_q4_rows : y = x * deq(w) [+ residual * residual_scale when residual is not NULL; residual may be y]; opSize % 16 == 0
 *   q4_qkv_matmul_rows: q, k, v from one read of x (opSize, kvSize multiples of 32)
 *   q4_ffn_silu_rows  : h = silu(x * deq(gate)) * (x * deq(up)), gate and up kept in fp32 until the product; opSize % 16 == 0 */
int q4_matmul_q4_rows(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* w, int M, int inpSize, int opSize,
                      const uint16_t* residual, float residual_scale);
int q4_qkv_matmul_rows(void* stream, uint16_t* q, uint16_t* k, uint16_t* v, const uint16_t* x, const q4_qweight* qw,
                       const q4_qweight* kw, const q4_qweight* vw, int M, int inpSize, int opSize, int kvSize);
int q4_ffn_silu_rows(void* stream, uint16_t* h, const uint16_t* x, const q4_qweight* gate_w, const q4_qweight* up_w, int M,
                     int inpSize, int opSize);
/* Measurement hook: q4_matmul_q4_batched over `nmat` distinct weight matrices of one shape (interleaved[i] may be NULL
 * or the array itself NULL), captured as one CUDA graph and replayed `reps` times between two events on `stream`. */
int q4_time_matmul_q4_batched(void* stream, uint16_t* y, const uint16_t* x, const q4_qweight* mats,
                              const uint32_t* const* interleaved, int nmat, int M, int inpSize, int opSize, void* workspace,
                              size_t workspace_bytes, int reps, double* us_per_launch);

/* matmul(half*): llama2_q4.cu:357-365, kernel gpu_kernels.h:117-147. fp16 GEMV used for the classifier:
 * xout[d] = alpha * sum_n w[d][n] * x[n]. n and d must be multiples of 8. */
int q4_matmul_f16(void* stream, uint16_t* xout, const uint16_t* x, const uint16_t* w, int n, int d, float alpha);

/* Embedding row gather: copy_embedding_kernel launch at llama2_q4.cu:441 (gpu_kernels.h:61-69).
 * `tokens` is the pinned-host token array; the row of tokens[*pPos] is copied to x. */
int q4_embed(void* stream, uint16_t* x, const uint16_t* table, int dim, const int* tokens, const int* pPos);

/* Greedy branch of sample(): sampler.h:77-84, kernel gpu_kernels.h:456-501. Writes argmax(logits) to
 * tokens_pinned[*pos_pinned + 1] when write_token != 0 and increments both position counters. Among equal
 * maxima the lowest index wins (the reference leaves that case to a race). */
int q4_argmax(void* stream, const uint16_t* logits, int size, int* tokens_pinned, volatile int* pos_pinned,
              int* pos_dev, int write_token);

/* Non-greedy branch of sample(): sampler.h:85-115 with softmax_logits_kernel / sample_top_p_kernel
 * (gpu_kernels.h:507-592) and the sort and prefix sum between them, as ONE launch. logits[0..n) are replaced by the
 * fp16 probabilities softmax(logits / temperature) as the reference does; the token is the first element, in
 * descending-probability order (0 < topp < 1, threshold coin * topp) or in index order (otherwise, threshold coin),
 * whose inclusive prefix sum reaches the threshold. The prefix sum is exact (integer multiples of 2^-24), where the
 * reference's runs in fp16. Writes tokens_pinned[*pos_pinned + 1] and increments both position words, like q4_argmax
 * with write_token = 1. temperature must be > 0 (the reference takes the greedy branch at 0); n <= 262144. */
int q4_sample_topp(void* stream, uint16_t* logits, int n, float temperature, float topp, float coin, int* tokens_pinned,
                   volatile int* pos_pinned, int* pos_dev);

/* The reference's xorshift* generator (sampler.h:66-75): one coin is drawn per sample() call, greedy or not. Host only. */
unsigned int q4_random_u32(unsigned long long* state);
float q4_random_f32(unsigned long long* state);

/* Test hook without a twin in the reference: dequantised weights w(n,k) as fp32 [N][K]
 * (the values gpu_kernels.h:204-205 computes on the fly), and raw nibbles as bytes. */
int q4_dequant(void* stream, float* out, const q4_qweight* w, int K, int N);
int q4_unpack_nibbles(void* stream, uint8_t* q_out, uint8_t* z_out, const q4_qweight* w, int K, int N);

/* ---------------------------------------------------------------------------------------------
 * Collectives: cuda_comm.h:80-300 (NCCL-shaped, as in the reference). One communicator per GPU.
 * Ranks may be threads of one process (the reference's model: peer pointers are exchanged through the
 * shared q4_comm_id) or separate processes (handles exchanged by the caller, q4_comm_export/_import).
 * ------------------------------------------------------------------------------------------- */
typedef struct q4_comm q4_comm;
typedef struct q4_comm_id q4_comm_id;

/* cudaCommGetUniqueId / cudaCommIdDestroy: cuda_comm.h:80-89,288-300. In-process rendezvous object. */
int q4_comm_id_create(q4_comm_id** id, int gpu_count);
int q4_comm_id_destroy(q4_comm_id* id);
/* cudaCommInitRank: cuda_comm.h:91-141. Thread-per-GPU flavour; call with device `rank`'s context current. */
int q4_comm_init_rank(q4_comm** comm, int gpu_count, q4_comm_id* id, int rank);
/* Process-per-GPU flavour: create the local inbox, export its 64-byte IPC handle, import every peer's. */
int q4_comm_create_local(q4_comm** comm, int gpu_count, int rank);
int q4_comm_export(q4_comm* comm, uint8_t handle[64]);
int q4_comm_import(q4_comm* comm, int peer, const uint8_t handle[64]);
/* cudaAllReduce (fp16 sum, in place): cuda_comm.h:160-224; call sites llama2_q4.cu:474-476,505-507.
 * One-shot push over NVLink: every rank stores its vector into every peer's inbox and sums the gpu_count
 * inbox slots in rank order in fp32, so all ranks obtain identical bits. count <= Q4_COMM_MAX_HALFS; vectors above
 * 64 KB are moved by four CTAs, each with its own part, flags and call counter. */
#define Q4_COMM_MAX_HALFS 131072
int q4_all_reduce(q4_comm* comm, void* stream, uint16_t* buf, int count);
/* cudaAllGather (fp16): cuda_comm.h:227-275; call site llama2_q4.cu:534-536. recv holds gpu_count*sendcount;
 * sendcount <= Q4_COMM_MAX_GATHER_HALFS. */
#define Q4_COMM_MAX_GATHER_HALFS 32768
int q4_all_gather(q4_comm* comm, void* stream, const uint16_t* send, uint16_t* recv, int sendcount);
/* Device-side wait status: 0, or Q4_ERR_TIMEOUT after a peer flag did not arrive within the bound. */
int q4_comm_status(q4_comm* comm);
/* Bound of the collectives' wait for the peers' flags, in nanoseconds of the device's global timer (default two
 * seconds; 0 restores it), and re-arming after a recorded timeout (every rank of the group must call it before
 * the next collective). */
int q4_comm_set_wait_limit_ns(q4_comm* comm, unsigned long long ns);
int q4_comm_reset(q4_comm* comm);
/* NCCL as the alternative transport of q4_all_reduce / q4_all_gather: the reference's -DENABLE_NCCL build
 * (CMakeLists.txt:14-43; ncclGetUniqueId / ncclCommInitRank at llama2_q4.cu:638-640,688-689, ncclAllReduce /
 * ncclAllGather at :474,505,534). libnccl.so.2 is opened at run time; without it q4_comm_nccl_available() is 0 and
 * the other calls return Q4_ERR_UNSUPPORTED_SIZE. One rank creates the id, the caller distributes its 128 bytes,
 * then every rank calls q4_comm_nccl_init (collective) on its communicator. The backend chooses the transport per
 * call: P2P (default) = one-shot peer push; NCCL; AUTO = by message size from the measured latency table (peer push
 * up to 32 KB on two GPUs and up to 128 KB on more, NCCL above). */
typedef struct { char internal[128]; } q4_nccl_id; /* same size and meaning as ncclUniqueId */
#define Q4_COMM_BACKEND_P2P 0
#define Q4_COMM_BACKEND_NCCL 1
#define Q4_COMM_BACKEND_AUTO 2
int q4_comm_nccl_available(void);
int q4_comm_nccl_unique_id(q4_nccl_id* id);
int q4_comm_nccl_init(q4_comm* comm, const q4_nccl_id* id);
int q4_comm_set_backend(q4_comm* comm, int backend);
/* cudaCommDestroy: cuda_comm.h:278-286. */
int q4_comm_destroy(q4_comm* comm);

/* ---------------------------------------------------------------------------------------------
 * Model level: build_transformer (llama2_q4.cu:625-659), run_transformer (:541-601),
 * generate_thread (:683-757).
 * ------------------------------------------------------------------------------------------- */
typedef struct q4_model q4_model;

#define Q4_TP_NONE 0   /* llama2_q4.cu:45-50 */
#define Q4_TP_COLUMN 1 /* every matrix split by output columns, four all-gathers per layer (llama2_q4.cu:479-493, 510-524);
                          served by forward paths 0 and 1 */
#define Q4_TP_HYBRID 2 /* Megatron: column split for q/k/v/gate/up, row split for o/down, two all-reduces per layer; all paths */

/* Reads the packed file (header + tensors in the order of weight_packer.cpp:256-291), keeps this rank's shard
 * on the current device (Megatron split of llama2_q4.cu:299-332, with row splits moved to 128-input group
 * boundaries) and allocates the run state (llama2_q4.cu:62-91). comm may be NULL when gpu_count == 1. */
int q4_model_load(q4_model** model, const char* path, int rank, int gpu_count, int tp_mode, q4_comm* comm);
/* The same model object without a file: a synthetic model of the given configuration, generated on the device
 * shard by shard from (seed, tensor, element index) - what stands in for real checkpoints in benchmarks of models
 * whose file would be tens of gigabytes (the reference reads the whole file through host memory,
 * llama2_q4.cu:645-646; it has no counterpart of this call). All ranks and all tensor-parallel degrees obtain shards
 * of one and the same logical model; llama_cu_awq_b200/synth.py writes the identical model as a packed file. */
int q4_model_create_synthetic(q4_model** model, const q4_config* cfg, unsigned long long seed, int rank, int gpu_count,
                              int tp_mode, q4_comm* comm);
int q4_model_free(q4_model* model);
int q4_model_config(const q4_model* model, q4_config* out);
/* Pinned mailbox of this rank (tokens[], pos) and device buffers, for tests and for the host loop. */
q4_shared_data* q4_model_shared(q4_model* model);
const uint16_t* q4_model_logits(const q4_model* model); /* device, vocab_size halfs */
const uint16_t* q4_model_x(const q4_model* model);      /* device, dim halfs */
/* Synchronous device-to-host copy of a run-state vector: what = 0 logits (vocab_size halfs), 1 x (dim halfs). */
int q4_model_read(const q4_model* model, int what, uint16_t* host_out);
/* Resets position counters (device and pinned) to `pos` and copies `n` prompt ids into the mailbox.
 * Q4_ERR_INVALID when an id lies outside [0, vocab_size): the embedding gather would read outside the table. */
int q4_model_reset(q4_model* model, const int* prompt_tokens, int n, int pos);
/* run_transformer(): one token at the current position on `stream`: embedding .. logits, then the greedy
 * hand-off (gen_token != 0 writes the sampled id to tokens[pos+1]); asynchronous. `path`: 0 = per-op kernels
 * launched one by one, 1 = the same launches replayed from a captured CUDA graph, 2 = one persistent
 * cooperative kernel per token that streams re-tiled weights through a shared-memory ring and exchanges the
 * residual stream between the ranks inside the kernel (head size 128, dim a multiple of 128, Q4_TP_NONE or
 * Q4_TP_HYBRID on 1 to 8 GPUs; returns Q4_ERR_UNSUPPORTED_SIZE otherwise).
 * Q4_ERR_LIMIT when the model's sequence length has been reached since the last q4_model_reset: the call would
 * write a K/V row outside the cache. */
int q4_model_forward(q4_model* model, void* stream, int gen_token, int path);
/* Builds whatever `path` needs ahead of the first token (path 2: re-tiled weight copy and phase table; needs
 * as much extra device memory as the quantized weights). Q4_ERR_UNSUPPORTED_SIZE when the path cannot serve
 * this model; q4_model_forward calls it on demand. */
int q4_model_prepare(q4_model* model, int path);

/* Prompt prefill: the next n_tokens positions of the model's sequence (token ids from the mailbox, starting at the
 * current position) in ONE pass through the network instead of n_tokens calls of q4_model_forward - what replaces the
 * reference's token-by-token prompt loop (llama2_q4.cu:710-735; gen_token there is false for all prompt positions but the
 * last). The projections run as W4 dequant-GEMMs on the tensor cores (q4_matmul_q4_batched), attention is causal over the
 * cache, every K/V row lands in the cache the decode paths use, and the last row goes through the batch-1 tail: final
 * norm, classifier, hand-off (tokens[pos + n_tokens] when gen_token != 0), both position words advanced by n_tokens.
 * Hybrid tensor parallelism as q4_model_forward; its [n_tokens x dim] all-reduces go through NCCL when it is attached to
 * the communicator and the backend choice allows it (Q4_COMM_BACKEND_AUTO / _NCCL), else through the peer push in pieces.
 * Head size 128, dim a multiple of 128. The first call builds a re-ordered copy of the packed weights (as much device
 * memory again as the quantized weights) and the row buffers. Asynchronous on `stream`. */
int q4_model_prefill(q4_model* model, void* stream, int n_tokens, int gen_token);

/* Batched decode: n_seq (<= 16) sequences that share the model's weights, each with its own K/V cache and position; one
 * call of q4_batch_forward advances every sequence by one position (greedy), the weights are streamed once per step
 * instead of once per sequence. The reference holds a single sequence (RunState, common.h:62-78) and has no counterpart.
 * q4_batch_reset takes [n_seq][n_prompt] prompt ids (all sequences start at position 0); ids past a sequence's prompt are
 * generated. q4_batch_logits: device pointer, [n_seq][vocab_size] halfs of the last step. */
typedef struct q4_batch q4_batch;
int q4_batch_create(q4_batch** batch, q4_model* model, int n_seq);
int q4_batch_reset(q4_batch* batch, const int* prompts, int n_prompt);
int q4_batch_forward(q4_batch* batch, void* stream);
const uint16_t* q4_batch_logits(const q4_batch* batch);
int q4_batch_read_tokens(const q4_batch* batch, int* out, int len);
int q4_batch_free(q4_batch* batch);

/* build_sampler (sampler.h:28-45). temperature 0 (the state after q4_model_load) decodes greedily; otherwise every
 * generating q4_model_forward ends with q4_sample_topp instead of the argmax. One coin is drawn from the xorshift*
 * state per forward call, greedy or not, as sample() does (sampler.h:79). All ranks of a tensor-parallel group set
 * the same values. */
int q4_model_set_sampler(q4_model* model, float temperature, float topp, unsigned long long seed);
/* Limit, in nanoseconds of the device's global timer, of every wait inside the fused kernel (path 2) for data of
 * another CTA or rank; 0 restores the default of two seconds. When a wait runs out the kernel records
 * Q4_ERR_TIMEOUT, lets all later waits fall through and returns; q4_model_status reports it and q4_model_reset
 * re-arms the path. The reference has no counterpart: a missing peer blocks its host barrier for ever
 * (cuda_comm.h:184,223). */
int q4_model_set_wait_limit_ns(q4_model* model, unsigned long long ns);
/* Synchronises the device and returns Q4_OK, or the error a bounded device-side wait recorded
 * (Q4_ERR_TIMEOUT) in the fused path or the communicator. */
int q4_model_status(q4_model* model);
/* generate_thread(): the token loop with the reference's timing window (llama2_q4.cu:708-745). Runs `steps`
 * positions starting from the n_prompt given ids, stops at EOS (id 2). out_tokens receives tokens[0..steps];
 * *timed_tokens = pos-1 and *seconds is the wall time of the loop. */
/* OR-ed into `path`: the prompt positions but the last go through q4_model_prefill in one pass (the last prompt
 * position and everything after it through `path` as usual); models the many-row kernels do not serve fall back to the
 * token loop. Same timing window, same *timed_tokens. */
#define Q4_PATH_PROMPT_ONE_PASS 0x100
int q4_generate(q4_model* model, const int* prompt_tokens, int n_prompt, int steps, int path, int* out_tokens,
                int* timed_tokens, double* seconds);
/* Algorithmic bytes one token at position `pos` reads and writes on this rank (weights, metadata,
 * classifier, norms, embedding row, KV rows). */
double q4_model_token_bytes(const q4_model* model, int pos);

/* Measurement hook: launches the fused gate/up GEMV of every layer back to back `reps` times on `stream`
 * (each layer's own weights, so the working set is far larger than L2) between two CUDA events on that stream.
 * Returns the total milliseconds and the algorithmic bytes one launch moves. */
int q4_model_time_ffn(q4_model* model, void* stream, int reps, double* total_ms, double* bytes_per_launch);

/* Measurement hook: one W4 op wrapper (kind 0 q4_matmul_q4, 1 q4_qkv_matvec with kvSize = opSize, 2 q4_ffn_matvec_silu)
 * over `nmat` distinct matrices of one shape, captured as one CUDA graph (kinds 1 / 2 take three / two matrices per
 * launch) and replayed `reps` times between two events on `stream`: weights come from HBM, not from L2, and no
 * launch gap is timed. Returns microseconds and algorithmic bytes per launch. */
int q4_time_q4_op(void* stream, int kind, uint16_t* y, uint16_t* y2, uint16_t* y3, const uint16_t* x, const q4_qweight* mats,
                  int nmat, int K, int N, int reps, const int* pPos, double* us_per_launch, double* bytes_per_launch);
/* The same for the few-rows forms with M rows of x: kind 0 q4_matmul_q4_rows, 1 q4_qkv_matmul_rows (kvSize = opSize),
 * 2 q4_ffn_silu_rows. */
int q4_time_q4_rows_op(void* stream, int kind, int M, uint16_t* y, uint16_t* y2, uint16_t* y3, const uint16_t* x, const q4_qweight* mats,
                       int nmat, int K, int N, int reps, double* us_per_launch, double* bytes_per_launch);
/* Measurement hook: `reps` in-place q4_all_reduce calls of `count` halfs back to back between two events on `stream`. */
int q4_time_all_reduce(q4_comm* comm, void* stream, uint16_t* buf, int count, int reps, double* us_per_call);

/* Profiling hook of the fused path: the first call arms per-phase device timestamps (globaltimer, ns) for the
 * following launches; later calls copy the last launch's stamps to `out` ([2 CTAs][nphases][8]: phase start,
 * inputs staged, weights consumed, phase closed, then staging detail: loads back, norm reduced, quantised)
 * and a type code per phase. The stamps are global stores and perturb what they measure by a few tenths of a
 * microsecond. Returns the phase count (always larger than any status code) or a status code. */
int q4_model_trace(q4_model* model, unsigned long long* out, int* phase_types, int max_phases);

/* ---------------------------------------------------------------------------------------------
 * Tokenizer of the command line (host code, no GPU): tokenizer.h:36-223. The vocabulary file is the reference's
 * tokenizer.bin format (uint32 max_token_length, then per token float32 score, int32 length, bytes).
 * ------------------------------------------------------------------------------------------- */
typedef struct q4_tokenizer q4_tokenizer;
/* build_tokenizer: tokenizer.h:36-61. Q4_ERR_IO when the file is missing or short (the reference exits). */
int q4_tokenizer_load(q4_tokenizer** tokenizer, const char* path, int vocab_size);
void q4_tokenizer_free(q4_tokenizer* tokenizer);
/* encode: tokenizer.h:108-223. bos/eos != 0 add ids 1 / 2. *n_tokens receives the count; Q4_ERR_LIMIT when it
 * exceeds max_tokens (strlen(text) + 3 always suffices), Q4_ERR_BAD_MODEL when the vocabulary has no " " piece or
 * no byte pieces where the text needs them. */
int q4_tokenizer_encode(const q4_tokenizer* tokenizer, const char* text, int bos, int eos, int* tokens, int max_tokens,
                        int* n_tokens);
/* decode + safe_printf: tokenizer.h:72-100. The text to print for `token` following `prev_token` ("" for an
 * unprintable single byte). The pointer stays valid until the next call on the same tokenizer. */
const char* q4_tokenizer_decode(q4_tokenizer* tokenizer, int prev_token, int token);

/* Host-side shard helpers (no GPU needed): copy rank `rank`'s shard of a quantized matrix held in host
 * memory. Column split = contiguous slice of outputs (llama2_q4.cu:254-263). Row split = slice of inputs on
 * 128-input group boundaries with zero nibbles re-packed (replaces llama2_q4.cu:264-285, which misplaces
 * zeros and scales when groups-per-rank is odd or fractional). q4_row_split_range gives the input range. */
void q4_row_split_range(int K, int gpu_count, int rank, int* k_begin, int* k_count);
int q4_shard_columns_host(const q4_qweight* src, int K, int N, int gpu_count, int rank, uint32_t* w_out,
                          uint32_t* z_out, uint16_t* s_out);
int q4_shard_rows_host(const q4_qweight* src, int K, int N, int gpu_count, int rank, uint32_t* w_out, uint32_t* z_out,
                       uint16_t* s_out);

#ifdef __cplusplus
}
#endif
#endif /* Q4B200_H */
