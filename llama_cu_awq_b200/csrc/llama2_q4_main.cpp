// llama2_q4: command-line front end with the reference program's flags and output lines
// (llama2_q4.cu:800-936 main/error_usage/get_and_print_gpu_info, :759-786 generate), driving the library
// through its C ABI only. One host thread per GPU, as in the reference (llama2_q4.cu:776-779).
//
// Extra flags (not in the reference): -k <file> reads whitespace-separated prompt token ids instead of text,
// -g <0|1|2> picks the forward path (per-op launches / CUDA-graph replay / persistent fused kernel).
#include <cuda_runtime_api.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <string>
#include <thread>
#include <vector>

#include "../../include/q4b200.h"

namespace {

constexpr int kEos = 2;  // tokenizer.h:9

// The vocabulary (tokenizer.bin) through the library's tokenizer entry points (q4_tokenizer_*).
class Vocab {
public:
    ~Vocab() { q4_tokenizer_free(t_); }
    bool load(const char* path, int vocab_size) { return q4_tokenizer_load(&t_, path, vocab_size) == Q4_OK; }
    bool loaded() const { return t_ != nullptr; }
    std::vector<int> encode(const std::string& text, bool bos) const {
        std::vector<int> out(text.size() + 3);
        int n = 0;
        if (q4_tokenizer_encode(t_, text.c_str(), bos ? 1 : 0, 0, out.data(), (int)out.size(), &n) != Q4_OK) n = 0;
        out.resize(n);
        return out;
    }
    // Printable text of `token` following `prev`; empty for unprintable single bytes.
    std::string decode(int prev, int token) const { return t_ ? q4_tokenizer_decode(t_, prev, token) : ""; }

private:
    q4_tokenizer* t_ = nullptr;
};

[[noreturn]] void error_usage(const char* argv0) {
    fprintf(stderr, "Usage:   %s <checkpoint> [options]\n", argv0);
    fprintf(stderr, "Example: %s model.bin -n 256 -i \"Write a poem on GPUs\"\n", argv0);
    fprintf(stderr, "Options:\n");
    fprintf(stderr, "  -n <int>    max number of steps to run for, default = max_seq_len\n");
    fprintf(stderr, "  -i <string> input prompt\n");
    fprintf(stderr, "  -f <string> path to file containing input prompt. Can be used with for multi-line prompts.\n");
    fprintf(stderr, "  -t <float>  temperature in [0,inf], default 0.5\n");
    fprintf(stderr, "  -p <float>  p value in top-p (nucleus) sampling in [0,1] default 0.9\n");
    fprintf(stderr, "  -s <int>    random seed, default time(NULL)\n");
    fprintf(stderr, "  -z <string> optional path to custom tokenizer\n");
    fprintf(stderr, "  -y <string> (optional) system prompt in chat mode\n");
    fprintf(stderr, "  -q <string> dataset file for computing perplexity\n");
    fprintf(stderr, "  -x <string> tensor parallel mode: none|column|hybrid, default none\n");
    fprintf(stderr, "  -k <string> path to a file of prompt token ids (replaces -i/-f)\n");
    fprintf(stderr, "  -g <int>    forward path: 0 per-op launches, 1 CUDA graph, 2 persistent fused kernel (default; falls back to 1)\n");
    fprintf(stderr, "  -b <0|1>    1: process the prompt in one pass (tensor-core prefill) instead of token by token, default 0\n");
    exit(EXIT_FAILURE);
}

int get_and_print_gpu_info() {
    int device_count = 0;
    cudaGetDeviceCount(&device_count);
    if (device_count == 0) {
        printf("No CUDA devices found!\n");
        exit(EXIT_FAILURE);
    }
    printf("Found %d CUDA devices\n", device_count);
    for (int dev = 0; dev < device_count; dev++) {
        cudaDeviceProp prop;
        cudaGetDeviceProperties(&prop, dev);
        printf("Device %d: %s\n", dev, prop.name);
        printf("  Compute capability: %d.%d\n", prop.major, prop.minor);
        printf("  Total global memory: %.2f GB\n", (float)prop.totalGlobalMem / (1024.0f * 1024.0f * 1024.0f));
        printf("  Multiprocessors: %d\n", prop.multiProcessorCount);
        printf("\n");
    }
    return device_count;
}

void die(int status, const char* what) {
    if (status == Q4_ERR_UNSUPPORTED_SIZE) printf("\nUnsupported matmul size. Exiting\n");
    else fprintf(stderr, "%s: %s\n", what, q4_status_string(status));
    exit(EXIT_FAILURE);
}

struct Shared {
    q4_comm_id* id = nullptr;
    std::vector<q4_model*> models;
    std::vector<q4_comm*> comms;
    std::atomic<int> fused_ok{1};   // cleared by any rank whose model the fused path does not serve
};

void load_thread(Shared* sh, const char* path, int rank, int gpu_count, int tp_mode, int fwd_path) {
    cudaSetDevice(rank);
    q4_comm* comm = nullptr;
    if (gpu_count > 1) {
        int e = q4_comm_init_rank(&comm, gpu_count, sh->id, rank);
        if (e) die(e, "communicator");
    }
    sh->comms[rank] = comm;
    int e = q4_model_load(&sh->models[rank], path, rank, gpu_count, tp_mode, comm);
    if (e) die(e, "build_transformer");
    // The fused path is prepared here, before the join that all ranks pass: its kernels exchange activations between
    // the ranks, so every rank must be ready before any rank launches.
    if (fwd_path == 2 && q4_model_prepare(sh->models[rank], 2) != Q4_OK) sh->fused_ok = 0;
}

// The token loop of generate_thread (llama2_q4.cu:683-757) with rank 0 streaming the text.
struct SamplerArgs { float temperature, topp; unsigned long long seed; };

void generate_thread(Shared* sh, const Vocab* vocab, const std::vector<int>* prompt, int steps, int rank, int fwd_path, SamplerArgs sa, int prompt_one_pass) {
    cudaSetDevice(rank);
    q4_model* m = sh->models[rank];
    q4_config cfg;
    q4_model_config(m, &cfg);
    cudaStream_t stream;
    cudaStreamCreate(&stream);
    q4_shared_data* mb = q4_model_shared(m);
    int e = q4_model_reset(m, prompt->data(), (int)prompt->size(), 0);
    if (e) die(e, "reset");
    e = q4_model_set_sampler(m, sa.temperature, sa.topp, sa.seed);   // build_sampler: every rank draws the same coins
    if (e) die(e, "build_sampler");
    int token = (*prompt)[0], next = 0, pos = 0;
    const auto start = std::chrono::steady_clock::now();
    const int n_prompt = (int)prompt->size();
    if (prompt_one_pass && n_prompt > 1 && steps > n_prompt - 1) {
        // -b 1: the prompt but its last position in one pass (q4_model_prefill); the text of those positions is the prompt
        // itself, so it is echoed at once. Shapes the many-row kernels do not serve keep the token loop.
        e = q4_model_prefill(m, stream, n_prompt - 1, 0);
        if (e == Q4_OK) {
            if (rank == 0)
                for (int i = 1; i < n_prompt - 1; i++) {   // what the loop would have printed at positions 1 .. n_prompt - 2
                    if (vocab->loaded()) fputs(vocab->decode((*prompt)[i - 1], (*prompt)[i]).c_str(), stdout);
                    else printf(" %d", (*prompt)[i]);
                }
            pos = n_prompt - 1;
            token = (*prompt)[pos - 1];
        } else if (e != Q4_ERR_UNSUPPORTED_SIZE) die(e, "prefill");
    }
    while (pos < steps) {
        cudaStreamSynchronize(stream);
        e = q4_model_forward(m, stream, pos >= (int)prompt->size() - 1, fwd_path);
        if (e) die(e, "run_transformer");
        if (pos > 0) {
            next = mb->tokens[pos];
            if (next >= cfg.vocab_size || next < 0) next = 0;
            if (rank == 0) {
                if (vocab->loaded()) fputs(vocab->decode(token, next).c_str(), stdout);
                else printf(" %d", next);   // no vocabulary (token-id prompt, -k): the ids themselves
                fflush(stdout);
            }
            if (next == kEos) break;
            token = next;
        }
        pos++;
    }
    cudaStreamSynchronize(stream);
    const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
    const int timed_tokens = pos - 1;
    printf("\n");
    printf("\n[GPU: %d] achieved tok/s: %f. Tokens: %d, seconds: %g\n", rank, timed_tokens / secs, timed_tokens, secs);
    cudaStreamDestroy(stream);
}

}  // namespace

int main(int argc, char* argv[]) {
    int gpu_count = get_and_print_gpu_info();

    const char* checkpoint_path = nullptr;
    const char* tokenizer_path = "tokenizer.bin";
    const char* dataset_path = nullptr;
    const char* token_file = nullptr;
    int steps = 0, fwd_path = 2, prompt_one_pass = 0;
    std::string prompt;
    bool have_prompt = false;
    float temperature = 0.5f, topp = 0.6f;  // the reference's defaults in code (llama2_q4.cu:852-853)
    unsigned long long rng_seed = 0;
    int tp_mode = Q4_TP_NONE;

    if (argc >= 2) checkpoint_path = argv[1];
    else error_usage(argv[0]);
    for (int i = 2; i < argc; i += 2) {
        if (i + 1 >= argc || argv[i][0] != '-' || strlen(argv[i]) != 2) error_usage(argv[0]);
        const char* v = argv[i + 1];
        switch (argv[i][1]) {
            case 'n': steps = atoi(v); break;
            case 'i': prompt = v; have_prompt = true; break;
            case 'z': tokenizer_path = v; break;
            case 't': temperature = (float)atof(v); break;
            case 'p': topp = (float)atof(v); break;
            case 's': rng_seed = (unsigned long long)atoi(v); break;
            case 'y': break;  // system prompt: parsed and unused, as in the reference
            case 'q': dataset_path = v; break;
            case 'k': token_file = v; break;
            case 'g': fwd_path = atoi(v); break;
            case 'b': prompt_one_pass = atoi(v); break;
            case 'x':
                if (!strcmp(v, "none")) tp_mode = Q4_TP_NONE;
                else if (!strcmp(v, "column")) tp_mode = Q4_TP_COLUMN;
                else if (!strcmp(v, "hybrid")) tp_mode = Q4_TP_HYBRID;
                else { printf("Unknown tp_mode: %s\n", v); exit(1); }
                break;
            case 'f': {
                FILE* file = fopen(v, "r");
                if (!file) { printf("Couldn't open file %s\n", v); exit(1); }
                if (have_prompt) printf("Warning: -f overrides -i\n");
                prompt.clear();
                char buf[4096];
                size_t n;
                while ((n = fread(buf, 1, sizeof(buf), file)) > 0) prompt.append(buf, n);
                fclose(file);
                have_prompt = true;
                break;
            }
            default: error_usage(argv[0]);
        }
    }
    if (tp_mode == Q4_TP_NONE) gpu_count = 1;
    if (gpu_count > Q4_MAX_GPUS) gpu_count = Q4_MAX_GPUS;
    if (rng_seed == 0) rng_seed = (unsigned int)time(nullptr);
    if (temperature < 0.0f) temperature = 0.0f;
    if (topp < 0.0f || 1.0f < topp) topp = 0.9f;
    if (dataset_path) printf("Warning: dataset path is ignored in non-perplexity mode\n");


    // header first, for the model summary the reference prints (llama2_q4.cu:633-634)
    q4_config cfg;
    {
        FILE* f = fopen(checkpoint_path, "rb");
        if (!f) { printf("Couldn't open file %s\n", checkpoint_path); exit(1); }
        if (fread(&cfg, sizeof(cfg), 1, f) != 1) { printf("Invalid header size\n"); exit(1); }
        fclose(f);
    }
    printf("\nModel params:- \ndim: %d \nhidden_dim: %d\nn_heads: %d\nn_kv_heads: %d\nn_layers: %d\nseq_len: %d\nvocab_size: %d\nrope_theta: %g\n",
           cfg.dim, cfg.hidden_dim, cfg.n_heads, cfg.n_kv_heads, cfg.n_layers, cfg.seq_len, cfg.vocab_size, cfg.rope_theta);

    Shared sh;
    sh.models.assign(gpu_count, nullptr);
    sh.comms.assign(gpu_count, nullptr);
    if (gpu_count > 1) {
        int e = q4_comm_id_create(&sh.id, gpu_count);
        if (e) die(e, "communicator id");
    }
    {
        std::vector<std::thread> th;
        for (int r = 0; r < gpu_count; r++) th.emplace_back(load_thread, &sh, checkpoint_path, r, gpu_count, tp_mode, fwd_path);
        for (auto& t : th) t.join();
    }
    if (fwd_path == 2 && !sh.fused_ok) fwd_path = 1;   // shapes the fused kernel does not serve: CUDA-graph replay
    if (steps <= 0 || steps > cfg.seq_len) steps = cfg.seq_len;

    Vocab vocab;
    std::vector<int> prompt_tokens;
    if (token_file) {
        FILE* f = fopen(token_file, "r");
        if (!f) { printf("Couldn't open file %s\n", token_file); exit(1); }
        int id;
        while (fscanf(f, "%d", &id) == 1) prompt_tokens.push_back(id);
        fclose(f);
        vocab.load(tokenizer_path, cfg.vocab_size);  // optional: ids are printed only when a vocabulary is there
    } else {
        if (!vocab.load(tokenizer_path, cfg.vocab_size)) { fprintf(stderr, "couldn't load %s\n", tokenizer_path); exit(EXIT_FAILURE); }
        printf("\nEncoding Prompt... ");
        prompt_tokens = vocab.encode(prompt, true);
        printf("Done!\n");
    }
    if (prompt_tokens.empty()) {
        fprintf(stderr, "something is wrong, expected at least 1 prompt token\n");
        exit(EXIT_FAILURE);
    }
    for (int id : prompt_tokens)
        if (id < 0 || id >= cfg.vocab_size) { fprintf(stderr, "prompt token id %d outside the vocabulary\n", id); exit(EXIT_FAILURE); }

    {
        std::vector<std::thread> th;
        for (int r = 0; r < gpu_count; r++) th.emplace_back(generate_thread, &sh, &vocab, &prompt_tokens, steps, r, fwd_path, SamplerArgs{temperature, topp, rng_seed}, prompt_one_pass);
        for (auto& t : th) t.join();
    }
    for (int r = 0; r < gpu_count; r++) {
        cudaSetDevice(r);
        q4_model_free(sh.models[r]);
        if (sh.comms[r]) q4_comm_destroy(sh.comms[r]);
    }
    if (sh.id) q4_comm_id_destroy(sh.id);
    return 0;
}
