// Harness around the reference's own CUDA code, compiled from where the reference lies
// (-I$REF, nothing copied). TEST / BASELINE INFRASTRUCTURE ONLY: the shipped library never
// loads this. It exposes the reference's host wrappers (llama2_q4.cu:347-427), its sampler
// (sampler.h:77-84) and its generation loop (llama2_q4.cu:683-757) through plain C entry
// points so that the tests can compare kernels bit for bit and bench.py can time the
// reference program on the same GPU.
#include "llama2_q4.cu"
#include <unistd.h>
#include <fcntl.h>

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

// Runs the reference program's own load + generation loop on one GPU at temperature 0 with the
// given token ids as the prompt. Returns the tokens[] mailbox (steps+1 entries), the last
// step's logits, and the tok/s figures the reference itself printed (parsed from its stdout).
int ref_generate(const char* path, const int* prompt_tokens, int n_prompt, int steps, int* out_tokens,
                 uint16_t* out_logits, double* out_toks, int* out_timed_tokens, double* out_seconds) {
    Transformer t;
    build_transformer(&t, 1, (char*)path, false, TP_NONE);
    if (steps <= 0 || steps > t.config.seq_len) steps = t.config.seq_len;
    Tokenizer tok;
    tok.vocab_size = t.config.vocab_size;
    tok.vocab = (char**)malloc(sizeof(char*) * tok.vocab_size);
    static char empty[2] = {0, 0};
    for (int i = 0; i < tok.vocab_size; i++) tok.vocab[i] = empty;
    Sampler sampler;
    build_sampler(&sampler, t.config.vocab_size, 0.0f, 0.9f, 1, 1);
    if (streams) { delete[] streams; }
    streams = new PerGPUExecutionData[1];

    fflush(stdout);
    char tmpl[] = "/tmp/ref_q4_stdout_XXXXXX";
    int fd = mkstemp(tmpl);
    int saved = dup(1);
    dup2(fd, 1);
    generate_thread(&t, &tok, &sampler, (int*)prompt_tokens, n_prompt, steps, 0, 1, TP_NONE);
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
        const char* p = strstr(buf, "achieved tok/s:");
        if (p) sscanf(p, "achieved tok/s: %lf. Tokens: %d, seconds: %lf", out_toks, out_timed_tokens, out_seconds);
    }
    free(buf);
    close(fd);
    unlink(tmpl);
    free_transformer(&t);
    free(tok.vocab);
    return 0;
}

}  // extern "C"
