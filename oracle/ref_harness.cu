// Harness around the reference's own CUDA code, compiled from where the reference lies
// (-I$REF, nothing copied). TEST / BASELINE INFRASTRUCTURE ONLY: the shipped library never
// loads this. It exposes the reference's host wrappers (llama2_q4.cu:347-427), its sampler
// (sampler.h:77-84) and its generation loop (llama2_q4.cu:683-757) through plain C entry
// points so that the tests can compare kernels bit for bit and bench.py can time the
// reference program on the same GPU.
#include "llama2_q4.cu"
#include <unistd.h>
#include <fcntl.h>
#include <barrier>
#include <chrono>

extern "C" {

int ref_init() {
    if (!streams) {
        streams = new PerGPUExecutionData[1];
        if (cudaStreamCreate(&streams[0].stream) != cudaSuccess) return 1;
    }
    return 0;
}

int ref_sync() { return (int)cudaStreamSynchronize(streams[0].stream); }
void* ref_stream() { return (void*)streams[0].stream; }

void ref_matmul_q4(half* y, half* x, uint32_t* w, uint32_t* z, half* s, int K, int N, int accum, int gpu_count, int loff, int* pPos) {
    QWeight qw{w, z, s};
    matmul(0, y, x, qw, K, N, accum != 0, gpu_count, loff, pPos);
}

void ref_qkv_matvec(half* q, half* kc, half* vc, half* x, uint32_t* qw, uint32_t* qz, half* qs, uint32_t* kw, uint32_t* kz, half* ks,
                    uint32_t* vw, uint32_t* vz, half* vs, int K, int N, int loff, int* pPos) {
    QWeight a{qw, qz, qs}, b{kw, kz, ks}, c{vw, vz, vs};
    qkv_matvec(0, q, kc, vc, x, a, b, c, K, N, loff, pPos);
}

void ref_ffn_matvec_silu(half* out, half* x, uint32_t* gw, uint32_t* gz, half* gs, uint32_t* uw, uint32_t* uz, half* us, int K, int N) {
    QWeight g{gw, gz, gs}, u{uw, uz, us};
    ffn_matvec_silu(0, out, x, g, u, K, N);
}

void ref_rmsnorm(half* o, half* x, half* w, int size) { rmsnorm(0, o, x, w, size); }

void ref_rope(half* q, half* k, int num_heads, int num_kv_heads, int head_size, int* pPos, int loff, float theta) {
    RoPERotation(0, q, k, num_heads, num_kv_heads, head_size, pPos, loff, theta);
}

void ref_mha(half* out, half* q, half* kc, half* vc, half* att, int num_heads, int head_size, int kv_mul, int max_seq_len, int* pPos) {
    MultiHeadAttention(0, out, q, kc, vc, att, num_heads, head_size, kv_mul, max_seq_len, pPos);
}

void ref_matmul_f16(half* out, half* x, half* w, int n, int d) { matmul(0, out, x, w, n, d); }

void ref_argmax(half* logits, int size, int* tokens_pinned, int* pos_pinned, int* pos_dev, int write_token) {
    argmax_kernel<<<1, 1024, 0, streams[0].stream>>>(logits, size, tokens_pinned, pos_pinned, pos_dev, write_token != 0);
}

// Runs the reference program's own load + generation loop at temperature 0 with the given token ids as the
// prompt: on one GPU (-x none), or on gpu_count GPUs with its hybrid tensor parallelism (-x hybrid, one host
// thread per GPU as generate() does, llama2_q4.cu:776-779). Returns rank 0's tokens[] mailbox (steps+1
// entries), its last step's logits, and the tok/s figures the reference itself printed for GPU 0 (parsed
// from its stdout).
int ref_generate(const char* path, const int* prompt_tokens, int n_prompt, int steps, int gpu_count, int* out_tokens,
                 uint16_t* out_logits, double* out_toks, int* out_timed_tokens, double* out_seconds) {
    if (gpu_count < 1 || gpu_count > MAX_GPUS) return 1;
    const TP_MODE mode = gpu_count > 1 ? TP_HYBRID : TP_NONE;
    Transformer t;
    build_transformer(&t, gpu_count, (char*)path, false, mode);
    if (steps <= 0 || steps > t.config.seq_len) steps = t.config.seq_len;
    Tokenizer tok;
    tok.vocab_size = t.config.vocab_size;
    tok.vocab = (char**)malloc(sizeof(char*) * tok.vocab_size);
    static char empty[2] = {0, 0};
    for (int i = 0; i < tok.vocab_size; i++) tok.vocab[i] = empty;
    Sampler sampler;
    build_sampler(&sampler, t.config.vocab_size, 0.0f, 0.9f, 1, 1);
    if (streams) { delete[] streams; }
    streams = new PerGPUExecutionData[gpu_count];

    fflush(stdout);
    char tmpl[] = "/tmp/ref_q4_stdout_XXXXXX";
    int fd = mkstemp(tmpl);
    int saved = dup(1);
    dup2(fd, 1);
    if (gpu_count == 1) {
        generate_thread(&t, &tok, &sampler, (int*)prompt_tokens, n_prompt, steps, 0, 1, TP_NONE);
    } else {
        std::vector<std::thread> threads;
        for (int i = 0; i < gpu_count; i++)
            threads.push_back(std::thread(generate_thread, &t, &tok, &sampler, (int*)prompt_tokens, n_prompt, steps, i, gpu_count, mode));
        for (auto& th : threads) th.join();
        cudaSetDevice(0);
    }
    fflush(stdout);
    dup2(saved, 1);
    close(saved);

    RunState* s = &t.pInfo[0].state;
    for (int i = 0; i <= steps && i < MAX_SEQ_LEN; i++) out_tokens[i] = s->shared_data->tokens[i];
    if (out_logits) cudaMemcpy(out_logits, s->logits, sizeof(half) * t.config.vocab_size, cudaMemcpyDeviceToHost);

    *out_toks = 0; *out_timed_tokens = 0; *out_seconds = 0;
    off_t len = lseek(fd, 0, SEEK_END);
    lseek(fd, 0, SEEK_SET);
    char* buf = (char*)calloc(len + 1, 1);
    if (read(fd, buf, len) == len) {
        const char* p = strstr(buf, "[GPU: 0] achieved tok/s:");
        if (p) p = strstr(p, "achieved tok/s:");
        if (p) sscanf(p, "achieved tok/s: %lf. Tokens: %d, seconds: %lf", out_toks, out_timed_tokens, out_seconds);
    }
    free(buf);
    close(fd);
    unlink(tmpl);
    free_transformer(&t);
    free(tok.vocab);
    return 0;
}

// The reference's sample() (sampler.h:77-115) on a logits vector: builds its Sampler with the given temperature,
// top-p and seed, runs one generating call and returns the token it wrote to the mailbox, the coin it drew, and
// the probabilities it left in the logits buffer (sorted descending when 0 < topp < 1, prefix-summed in place).
int ref_sample(const uint16_t* logits_host, int n, float temperature, float topp, unsigned long long seed, int* out_token, float* out_coin) {
    Sampler sampler;
    build_sampler(&sampler, n, temperature, topp, seed, 1);
    unsigned long long st = seed;
    *out_coin = random_f32(&st);
    RunState s;
    memset(&s, 0, sizeof(s));
    cudaMalloc((void**)&s.logits, sizeof(half) * n);
    cudaMalloc((void**)&s.pos, sizeof(int));
    cudaMallocHost((void**)&s.shared_data, sizeof(SharedData));
    const int pos = 3;
    s.shared_data->pos = pos;
    cudaMemcpy(s.pos, &pos, sizeof(int), cudaMemcpyHostToDevice);
    cudaMemcpy(s.logits, logits_host, sizeof(half) * n, cudaMemcpyHostToDevice);
    sample(0, &sampler, &s, true, streams[0].stream);
    const int rc = (int)cudaStreamSynchronize(streams[0].stream);
    *out_token = s.shared_data->tokens[pos + 1];
    cudaFree(s.logits);
    cudaFree(s.pos);
    cudaFreeHost(s.shared_data);
    destroy_sampler(&sampler);
    return rc;
}

// Times the reference's W4 kernels on `nmat` distinct matrices of one shape, back to back (a captured graph of
// the reference's own wrapper calls, replayed `reps` times between two events), so that the weights come from
// HBM and not from L2. kind 0: matmul(QWeight) (mat_vec_kernel_int4), 1: qkv_matvec, 2: ffn_matvec_silu.
// w/z/s are arrays of nmat device pointers (kind 1 uses 3 consecutive entries per launch, kind 2 uses 2).
int ref_time_q4(int kind, half* y, half* y2, half* y3, half* x, uint32_t** w, uint32_t** z, half** s, int nmat, int K, int N, int reps,
                int* pPos, double* out_us_per_launch) {
    cudaStream_t st = streams[0].stream;
    const int per = kind == 1 ? 3 : kind == 2 ? 2 : 1;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return 1;
    int launches = 0;
    for (int i = 0; i + per <= nmat; i += per, launches++) {
        QWeight a{w[i], z[i], s[i]};
        if (kind == 0) matmul(0, y, x, a, K, N);
        else if (kind == 1) { QWeight b{w[i + 1], z[i + 1], s[i + 1]}, c{w[i + 2], z[i + 2], s[i + 2]}; qkv_matvec(0, y, y2, y3, x, a, b, c, K, N, 0, pPos); }
        else { QWeight b{w[i + 1], z[i + 1], s[i + 1]}; ffn_matvec_silu(0, y, x, a, b, K, N); }
    }
    if (cudaStreamEndCapture(st, &graph) != cudaSuccess) return 2;
    if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) return 3;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaGraphLaunch(exec, st);
    cudaEventRecord(e0, st);
    for (int r = 0; r < reps; r++) cudaGraphLaunch(exec, st);
    cudaEventRecord(e1, st);
    if (cudaEventSynchronize(e1) != cudaSuccess) return 4;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    *out_us_per_launch = 1e3 * ms / ((double)reps * launches);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    return 0;
}

// Times the reference's cudaAllReduce (cuda_comm.h:160-224) on gpu_count GPUs, one host thread per GPU as the
// reference runs it: `reps` in-place fp16 sum all-reduces of `count` halfs back to back, wall time of the
// slowest thread. Rank 0 initialises its communicator before the others start (the reference re-creates the
// shared host barrier in rank 0's init, cuda_comm.h:97-100, which must not overlap another rank's first wait).
int ref_time_allreduce(int gpu_count, int count, int reps, double* out_us_per_call) {
    if (gpu_count < 2 || gpu_count > MAX_GPUS) return 1;
    CudaCommId id;
    cudaCommGetUniqueId(&id);
    std::barrier<> sync(gpu_count);
    std::vector<double> us(gpu_count, 0.0);
    std::vector<std::thread> threads;
    for (int r = 0; r < gpu_count; r++) {
        threads.push_back(std::thread([&, r]() {
            cudaSetDevice(r);
            CudaComm comm;
            if (r == 0) cudaCommInitRank(&comm, gpu_count, &id, r);
            sync.arrive_and_wait();
            if (r != 0) cudaCommInitRank(&comm, gpu_count, &id, r);
            cudaStream_t st;
            cudaStreamCreate(&st);
            half* buf;
            cudaMalloc(&buf, sizeof(half) * count);
            cudaMemset(buf, 0, sizeof(half) * count);
            cudaDeviceSynchronize();
            sync.arrive_and_wait();
            for (int i = 0; i < 20; i++) cudaAllReduce(buf, buf, count, CUDA_HALF, CUDA_SUM, &comm, st);
            cudaStreamSynchronize(st);
            sync.arrive_and_wait();
            const auto t0 = std::chrono::steady_clock::now();
            for (int i = 0; i < reps; i++) cudaAllReduce(buf, buf, count, CUDA_HALF, CUDA_SUM, &comm, st);
            cudaStreamSynchronize(st);
            us[r] = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count() / reps;
            sync.arrive_and_wait();
            cudaFree(buf);
            cudaStreamDestroy(st);
            cudaCommDestroy(&comm);
        }));
    }
    for (auto& th : threads) th.join();
    cudaSetDevice(0);
    cudaCommIdDestroy(&id);
    double worst = 0;
    for (double v : us) worst = v > worst ? v : worst;
    *out_us_per_call = worst;
    return 0;
}

}  // extern "C"
