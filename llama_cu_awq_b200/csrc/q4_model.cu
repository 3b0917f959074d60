// Host side of the decode path: packed-file loader, Megatron sharder, run state, the per-token schedule and the
// generation loop. Replaces build_transformer / init_transformer / uploadQWeight / checkpoint_init_weights
// (llama2_q4.cu:62-332,613-659), run_llama_network / run_transformer (:430-601) and generate_thread (:683-757).
#include <chrono>
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

#include "q4_model.h"

// ------------------------------------------------------------------------------------------------------------
// Shard helpers on host memory
// ------------------------------------------------------------------------------------------------------------

// Inputs [k_begin, k_begin + k_count) that rank `rank` owns when K inputs are split over gpu_count ranks on
// 128-input group boundaries; the first (G % gpu_count) ranks get one group more.
extern "C" void q4_row_split_range(int K, int gpu_count, int rank, int* k_begin, int* k_count) {
    const int G = q4_groups(K);
    const int base = G / gpu_count, rem = G % gpu_count;
    const int gb = rank * base + (rank < rem ? rank : rem);
    const int gc = base + (rank < rem ? 1 : 0);
    int kb = gb * 128, ke = (gb + gc) * 128;
    if (ke > K) ke = K;
    if (kb > K) kb = K;
    *k_begin = kb;
    *k_count = ke - kb;
}

static void shard_columns_range(const q4_qweight* src, int K, int n_begin, int n_count, uint32_t* w_out, uint32_t* z_out,
                                uint16_t* s_out) {
    const size_t PW = q4_pw(K), PZ = q4_pz(K), G = q4_groups(K);
    memcpy(w_out, src->weight + (size_t)n_begin * PW, (size_t)n_count * PW * 4);
    memcpy(z_out, src->zeros + (size_t)n_begin * PZ, (size_t)n_count * PZ * 4);
    memcpy(s_out, src->scales + (size_t)n_begin * G, (size_t)n_count * G * 2);
}

extern "C" int q4_shard_columns_host(const q4_qweight* src, int K, int N, int gpu_count, int rank, uint32_t* w_out,
                                     uint32_t* z_out, uint16_t* s_out) {
    if (!src || !w_out || !z_out || !s_out || gpu_count < 1 || rank < 0 || rank >= gpu_count) return Q4_ERR_INVALID;
    if (N % gpu_count) return Q4_ERR_UNSUPPORTED_SIZE;
    const int nc = N / gpu_count;
    shard_columns_range(src, K, rank * nc, nc, w_out, z_out, s_out);
    return Q4_OK;
}

static void shard_rows_range(const q4_qweight* src, int K, int N, int kb, int kc, uint32_t* w_out, uint32_t* z_out, uint16_t* s_out) {
    const size_t PW = q4_pw(K), PZ = q4_pz(K), G = q4_groups(K);
    const size_t pw = q4_pw(kc), pz = q4_pz(kc), gg = q4_groups(kc);
    const int gb = kb / 128;
    for (int n = 0; n < N; n++) {
        uint32_t* wd = w_out + (size_t)n * pw;
        const uint32_t* ws = src->weight + (size_t)n * PW + kb / 8;
        const size_t words = (size_t)(kc + 7) / 8;
        memcpy(wd, ws, words * 4);
        for (size_t i = words; i < pw; i++) wd[i] = 0;
        uint32_t* zd = z_out + (size_t)n * pz;
        const uint32_t* zs = src->zeros + (size_t)n * PZ;
        for (size_t i = 0; i < pz; i++) zd[i] = 0;
        for (size_t g = 0; g < gg; g++) {
            const size_t sg = gb + g;
            const uint32_t z = (zs[sg >> 3] >> (4 * (sg & 7))) & 0xFu;
            zd[g >> 3] |= z << (4 * (g & 7));
        }
        memcpy(s_out + (size_t)n * gg, src->scales + (size_t)n * G + gb, gg * 2);
    }
}

extern "C" int q4_shard_rows_host(const q4_qweight* src, int K, int N, int gpu_count, int rank, uint32_t* w_out, uint32_t* z_out,
                                  uint16_t* s_out) {
    if (!src || !w_out || !z_out || !s_out || gpu_count < 1 || rank < 0 || rank >= gpu_count) return Q4_ERR_INVALID;
    if (gpu_count > 1 && (K % 128)) return Q4_ERR_UNSUPPORTED_SIZE;
    int kb, kc;
    q4_row_split_range(K, gpu_count, rank, &kb, &kc);
    shard_rows_range(src, K, N, kb, kc, w_out, z_out, s_out);
    return Q4_OK;
}

// ------------------------------------------------------------------------------------------------------------
// Model
// ------------------------------------------------------------------------------------------------------------
namespace {

struct FileMap {
    const uint8_t* p = nullptr;
    size_t n = 0;
    int fd = -1;
    ~FileMap() {
        if (p) munmap((void*)p, n);
        if (fd >= 0) close(fd);
    }
};

struct HostQ {
    q4_qweight w;
    int K, N;
};

const uint8_t* take_q(const uint8_t* p, HostQ* q, int K, int N) {
    q->K = K;
    q->N = N;
    q->w.weight = (const uint32_t*)p; p += (size_t)N * q4_pw(K) * 4;
    q->w.zeros = (const uint32_t*)p;  p += (size_t)N * q4_pz(K) * 4;
    q->w.scales = (const uint16_t*)p; p += (size_t)N * q4_groups(K) * 2;
    return p;
}

struct Arena {
    char* base;
    size_t off, cap;
    void* take(size_t bytes) {
        off = align_up(off, 256);
        void* r = base + off;
        off += bytes;
        return off <= cap ? r : nullptr;
    }
};

enum SplitKind { SPLIT_NONE, SPLIT_COLS, SPLIT_ROWS };

// Copies (a shard of) one quantized matrix to the device. Column shards are contiguous in the file and go
// straight from the mapping; row shards are re-packed on the host first.
int upload_q(Arena& a, DevQW* dst, const HostQ& src, SplitKind kind, int begin, int count, std::vector<uint8_t>& tmp) {
    int K = src.K, N = src.N;
    if (kind == SPLIT_COLS) N = count;
    if (kind == SPLIT_ROWS) K = count;
    const size_t wb = (size_t)N * q4_pw(K) * 4, zb = (size_t)N * q4_pz(K) * 4, sb = (size_t)N * q4_groups(K) * 2;
    uint32_t* dw = (uint32_t*)a.take(wb);
    uint32_t* dz = (uint32_t*)a.take(zb);
    uint16_t* ds = (uint16_t*)a.take(sb);
    if (!dw || !dz || !ds) return Q4_ERR_BAD_MODEL;
    dst->w.weight = dw;
    dst->w.zeros = dz;
    dst->w.scales = ds;
    dst->K = K;
    dst->N = N;
    if (kind == SPLIT_ROWS) {
        tmp.resize(wb + zb + sb);
        uint32_t* hw = (uint32_t*)tmp.data();
        uint32_t* hz = (uint32_t*)(tmp.data() + wb);
        uint16_t* hs = (uint16_t*)(tmp.data() + wb + zb);
        shard_rows_range(&src.w, src.K, src.N, begin, count, hw, hz, hs);
        Q4_CUDA_TRY(cudaMemcpy(dw, hw, wb, cudaMemcpyHostToDevice));
        Q4_CUDA_TRY(cudaMemcpy(dz, hz, zb, cudaMemcpyHostToDevice));
        Q4_CUDA_TRY(cudaMemcpy(ds, hs, sb, cudaMemcpyHostToDevice));
    } else {
        const int nb = kind == SPLIT_COLS ? begin : 0;
        Q4_CUDA_TRY(cudaMemcpy(dw, src.w.weight + (size_t)nb * q4_pw(K), wb, cudaMemcpyHostToDevice));
        Q4_CUDA_TRY(cudaMemcpy(dz, src.w.zeros + (size_t)nb * q4_pz(K), zb, cudaMemcpyHostToDevice));
        Q4_CUDA_TRY(cudaMemcpy(ds, src.w.scales + (size_t)nb * q4_groups(K), sb, cudaMemcpyHostToDevice));
    }
    return Q4_OK;
}

int upload_raw(Arena& a, uint16_t** dst, const void* src, size_t bytes) {
    void* d = a.take(bytes);
    if (!d) return Q4_ERR_BAD_MODEL;
    Q4_CUDA_TRY(cudaMemcpy(d, src, bytes, cudaMemcpyHostToDevice));
    *dst = (uint16_t*)d;
    return Q4_OK;
}

}  // namespace

extern "C" int q4_model_free(q4_model* m) {
    if (!m) return Q4_OK;
    q4_fused_free(m);
    q4_rows_free(m);
    for (int i = 0; i < 3; i++)
        if (m->graph_ready[i]) cudaGraphExecDestroy(m->graph[i]);
    cudaFree(m->arena);
    cudaFree(m->x); cudaFree(m->xb); cudaFree(m->hb); cudaFree(m->q); cudaFree(m->logits);
    cudaFree(m->kc); cudaFree(m->vc); cudaFree(m->attn_scratch); cudaFree(m->pos);
    if (m->shared) cudaFreeHost(m->shared);
    delete m;
    return Q4_OK;
}

// Where a model's tensors come from: the packed file (mapped), or the counter-based synthetic generator (seed).
struct ModelSource {
    const uint8_t* file = nullptr;   // start of the mapping, or null
    unsigned long long seed = 0;
};

// One quantized matrix of the synthetic model, generated on the device straight into this rank's shard. Every value is
// a function of (seed, tensor id, logical element index), so all ranks and all tensor-parallel degrees see the same model.
static int synth_q(Arena& a, DevQW* dst, int K_full, int N_full, SplitKind kind, int begin, int count, unsigned long long seed, int tid) {
    int K = K_full, N = N_full, n0 = 0, kb = 0;
    if (kind == SPLIT_COLS) { N = count; n0 = begin; }
    if (kind == SPLIT_ROWS) { K = count; kb = begin; }
    const size_t wb = (size_t)N * q4_pw(K) * 4, zb = (size_t)N * q4_pz(K) * 4, sb = (size_t)N * q4_groups(K) * 2;
    uint32_t* dw = (uint32_t*)a.take(wb);
    uint32_t* dz = (uint32_t*)a.take(zb);
    uint16_t* ds = (uint16_t*)a.take(sb);
    if (!dw || !dz || !ds) return Q4_ERR_BAD_MODEL;
    dst->w.weight = dw; dst->w.zeros = dz; dst->w.scales = ds;
    dst->K = K; dst->N = N;
    return q4_synth_qweight(dw, dz, ds, K_full, K, kb, N, n0, seed, tid);
}

static int model_build(q4_model** out, const q4_config& c, int rank, int gpu_count, int tp_mode, q4_comm* comm, const ModelSource& src) {
    if (c.dim <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.vocab_size <= 0 ||
        c.seq_len <= 0 || c.seq_len > Q4_MAX_SEQ_LEN || c.dim % c.n_heads || c.n_heads % c.n_kv_heads || (c.dim & 7) || (c.hidden_dim & 7))
        return Q4_ERR_BAD_MODEL;
    const int g = gpu_count;
    const int hs = c.dim / c.n_heads;
    const int kv_dim = c.dim * c.n_kv_heads / c.n_heads;
    if (c.n_heads % g || c.n_kv_heads % g || c.vocab_size % (8 * g)) return Q4_ERR_UNSUPPORTED_SIZE;
    if (g > 1 && ((c.dim / g) % 128 || c.hidden_dim % 128)) return Q4_ERR_UNSUPPORTED_SIZE;

    q4_model* m = new q4_model();
    m->cfg = c;
    m->rank = rank;
    m->g = g;
    m->tp_mode = tp_mode;
    m->comm = comm;
    m->head_size = hs;
    m->kv_dim = kv_dim;
    m->kv_mul = c.n_heads / c.n_kv_heads;
    m->q_n = c.dim / g;
    m->kv_n = kv_dim / g;
    m->o_kb = rank * (c.dim / g);
    m->o_kc = c.dim / g;
    m->column = g > 1 && tp_mode == Q4_TP_COLUMN;
    if (m->column) {   // plain hidden/g slices (llama2_q4.cu:498): no row split, so no group alignment to keep
        if (c.hidden_dim % (8 * g)) { delete m; return Q4_ERR_UNSUPPORTED_SIZE; }
        m->h_kb = rank * (c.hidden_dim / g);
        m->h_kc = c.hidden_dim / g;
    } else if (g > 1) q4_row_split_range(c.hidden_dim, g, rank, &m->h_kb, &m->h_kc);
    else { m->h_kb = 0; m->h_kc = c.hidden_dim; }
    m->v_n = c.vocab_size / g;
    m->graph_ready[0] = m->graph_ready[1] = m->graph_ready[2] = false;
    m->temperature = 0.f;
    m->topp = 0.f;
    m->rng_state = 0;
    m->fused = nullptr;
    m->rows = nullptr;
    m->host_pos = 0;
    m->arena = nullptr;
    m->x = m->xb = m->hb = m->q = m->logits = m->kc = m->vc = nullptr;
    m->attn_scratch = nullptr;
    m->pos = nullptr;
    m->shared = nullptr;

    // device arena for this rank's weights
    size_t need = 0;
    auto add = [&](size_t b) { need = align_up(need, 256) + b; };
    add(2 * (size_t)c.vocab_size * c.dim);
    add(2 * (size_t)m->v_n * c.dim);
    add(2 * (size_t)c.dim);
    for (int l = 0; l < c.n_layers; l++) {
        auto addq = [&](int K, int N) { add((size_t)N * q4_pw(K) * 4); add((size_t)N * q4_pz(K) * 4); add((size_t)N * q4_groups(K) * 2); };
        addq(c.dim, m->q_n); addq(c.dim, m->kv_n); addq(c.dim, m->kv_n);
        if (m->column) addq(c.dim, c.dim / g); else addq(m->o_kc, c.dim);
        addq(c.dim, m->h_kc); addq(c.dim, m->h_kc);
        if (m->column) addq(c.hidden_dim, c.dim / g); else addq(m->h_kc, c.dim);
        add(2 * (size_t)c.dim); add(2 * (size_t)c.dim);
    }
    need += 256;
    int status = Q4_OK;
#define LOAD_TRY(expr) do { status = (expr); if (status != Q4_OK) { q4_model_free(m); return status; } } while (0)
#define LOAD_CUDA(expr) do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) { q4_note_cuda_error(e__, __FILE__, __LINE__); q4_model_free(m); return Q4_ERR_CUDA; } } while (0)
    LOAD_CUDA(cudaMalloc((void**)&m->arena, need));
    m->arena_bytes = need;
    Arena a{m->arena, 0, need};

    printf("\nLoading Weights... ");
    m->layers.resize(c.n_layers);
    const SplitKind col = g > 1 ? SPLIT_COLS : SPLIT_NONE, row = g > 1 ? SPLIT_ROWS : SPLIT_NONE;
    if (src.file) {
        const uint8_t* p = src.file + 32;
        LOAD_TRY(upload_raw(a, &m->emb, p, 2 * (size_t)c.vocab_size * c.dim));
        p += 2 * (size_t)c.vocab_size * c.dim;
        LOAD_TRY(upload_raw(a, &m->wcls, p + 2 * (size_t)rank * m->v_n * c.dim, 2 * (size_t)m->v_n * c.dim));
        p += 2 * (size_t)c.vocab_size * c.dim;
        LOAD_TRY(upload_raw(a, &m->rms_final, p, 2 * (size_t)c.dim));
        p += 2 * (size_t)c.dim;
        std::vector<uint8_t> tmp;
        for (int l = 0; l < c.n_layers; l++) {
            DevLayer& L = m->layers[l];
            HostQ hq, hk, hv, ho, hup, hgate, hdown;
            p = take_q(p, &hq, c.dim, c.dim);
            p = take_q(p, &hk, c.dim, kv_dim);
            p = take_q(p, &hv, c.dim, kv_dim);
            p = take_q(p, &ho, c.dim, c.dim);
            p = take_q(p, &hup, c.dim, c.hidden_dim);    // up precedes gate in the file (weight_packer.cpp:283-284)
            p = take_q(p, &hgate, c.dim, c.hidden_dim);
            p = take_q(p, &hdown, c.hidden_dim, c.dim);
            LOAD_TRY(upload_q(a, &L.q, hq, col, rank * m->q_n, m->q_n, tmp));
            LOAD_TRY(upload_q(a, &L.k, hk, col, rank * m->kv_n, m->kv_n, tmp));
            LOAD_TRY(upload_q(a, &L.v, hv, col, rank * m->kv_n, m->kv_n, tmp));
            if (m->column) LOAD_TRY(upload_q(a, &L.o, ho, col, rank * (c.dim / g), c.dim / g, tmp));
            else LOAD_TRY(upload_q(a, &L.o, ho, row, m->o_kb, m->o_kc, tmp));
            LOAD_TRY(upload_q(a, &L.up, hup, col, m->h_kb, m->h_kc, tmp));
            LOAD_TRY(upload_q(a, &L.gate, hgate, col, m->h_kb, m->h_kc, tmp));
            if (m->column) LOAD_TRY(upload_q(a, &L.down, hdown, col, rank * (c.dim / g), c.dim / g, tmp));
            else LOAD_TRY(upload_q(a, &L.down, hdown, row, m->h_kb, m->h_kc, tmp));
            LOAD_TRY(upload_raw(a, &L.rms_att, p, 2 * (size_t)c.dim));
            p += 2 * (size_t)c.dim;
            LOAD_TRY(upload_raw(a, &L.rms_ffn, p, 2 * (size_t)c.dim));
            p += 2 * (size_t)c.dim;
        }
    } else {
        // tensor ids of the generator: 1 embedding, 2 classifier, 16 + (layer * 8 + matrix) * 4 + part (q k v o up gate down; the
        // part is added by q4_synth_qweight: 0 weights, 1 zero points, 2 scales); the RMSNorm weights are 1.0
        auto take16 = [&](uint16_t** dst, size_t halfs) { *dst = (uint16_t*)a.take(2 * halfs); return *dst ? Q4_OK : Q4_ERR_BAD_MODEL; };
        LOAD_TRY(take16(&m->emb, (size_t)c.vocab_size * c.dim));
        LOAD_TRY(q4_synth_normal(m->emb, (long long)c.vocab_size * c.dim, 0, src.seed, 1));
        LOAD_TRY(take16(&m->wcls, (size_t)m->v_n * c.dim));
        LOAD_TRY(q4_synth_normal(m->wcls, (long long)m->v_n * c.dim, (long long)rank * m->v_n * c.dim, src.seed, 2));
        LOAD_TRY(take16(&m->rms_final, c.dim));
        LOAD_TRY(q4_synth_const(m->rms_final, c.dim, 0x3C00));
        for (int l = 0; l < c.n_layers; l++) {
            DevLayer& L = m->layers[l];
            auto tid = [&](int matrix) { return 16 + (l * 8 + matrix) * 4; };
            LOAD_TRY(synth_q(a, &L.q, c.dim, c.dim, col, rank * m->q_n, m->q_n, src.seed, tid(0)));
            LOAD_TRY(synth_q(a, &L.k, c.dim, kv_dim, col, rank * m->kv_n, m->kv_n, src.seed, tid(1)));
            LOAD_TRY(synth_q(a, &L.v, c.dim, kv_dim, col, rank * m->kv_n, m->kv_n, src.seed, tid(2)));
            if (m->column) LOAD_TRY(synth_q(a, &L.o, c.dim, c.dim, col, rank * (c.dim / g), c.dim / g, src.seed, tid(3)));
            else LOAD_TRY(synth_q(a, &L.o, c.dim, c.dim, row, m->o_kb, m->o_kc, src.seed, tid(3)));
            LOAD_TRY(synth_q(a, &L.up, c.dim, c.hidden_dim, col, m->h_kb, m->h_kc, src.seed, tid(4)));
            LOAD_TRY(synth_q(a, &L.gate, c.dim, c.hidden_dim, col, m->h_kb, m->h_kc, src.seed, tid(5)));
            if (m->column) LOAD_TRY(synth_q(a, &L.down, c.hidden_dim, c.dim, col, rank * (c.dim / g), c.dim / g, src.seed, tid(6)));
            else LOAD_TRY(synth_q(a, &L.down, c.hidden_dim, c.dim, row, m->h_kb, m->h_kc, src.seed, tid(6)));
            LOAD_TRY(take16(&L.rms_att, c.dim));
            LOAD_TRY(q4_synth_const(L.rms_att, c.dim, 0x3C00));
            LOAD_TRY(take16(&L.rms_ffn, c.dim));
            LOAD_TRY(q4_synth_const(L.rms_ffn, c.dim, 0x3C00));
        }
        LOAD_CUDA(cudaDeviceSynchronize());
    }
    printf("done!\n");

    // run state (llama2_q4.cu:62-91); the KV cache holds this rank's kv heads only
    const size_t kv_bytes = 2 * (size_t)c.n_layers * c.seq_len * m->kv_n;
    LOAD_CUDA(cudaMalloc((void**)&m->x, 2 * (size_t)c.dim));
    LOAD_CUDA(cudaMalloc((void**)&m->xb, 2 * (size_t)c.dim));
    LOAD_CUDA(cudaMalloc((void**)&m->hb, 2 * (size_t)c.hidden_dim));
    LOAD_CUDA(cudaMalloc((void**)&m->q, 2 * (size_t)c.dim));
    LOAD_CUDA(cudaMalloc((void**)&m->logits, 2 * (size_t)c.vocab_size));
    LOAD_CUDA(cudaMalloc((void**)&m->kc, kv_bytes));
    LOAD_CUDA(cudaMalloc((void**)&m->vc, kv_bytes));
    LOAD_CUDA(cudaMalloc((void**)&m->attn_scratch, q4_attention_scratch_bytes(c.n_heads / g, hs)));
    LOAD_CUDA(cudaMalloc((void**)&m->pos, sizeof(int)));
    LOAD_CUDA(cudaMallocHost((void**)&m->shared, sizeof(q4_shared_data)));
    LOAD_CUDA(cudaMemset(m->kc, 0, kv_bytes));
    LOAD_CUDA(cudaMemset(m->vc, 0, kv_bytes));
    LOAD_CUDA(cudaMemset(m->pos, 0, sizeof(int)));
    LOAD_CUDA(cudaMemset(m->x, 0, 2 * (size_t)c.dim));
    memset(m->shared, 0, sizeof(q4_shared_data));
    LOAD_CUDA(cudaDeviceSynchronize());
#undef LOAD_TRY
#undef LOAD_CUDA
    *out = m;
    return Q4_OK;
}

extern "C" int q4_model_load(q4_model** out, const char* path, int rank, int gpu_count, int tp_mode, q4_comm* comm) {
    if (!out || !path || gpu_count < 1 || gpu_count > Q4_MAX_GPUS || rank < 0 || rank >= gpu_count) return Q4_ERR_INVALID;
    if (gpu_count > 1 && tp_mode != Q4_TP_HYBRID && tp_mode != Q4_TP_COLUMN) return Q4_ERR_INVALID;
    if (gpu_count > 1 && !comm) return Q4_ERR_INVALID;

    FileMap f;
    f.fd = open(path, O_RDONLY);
    if (f.fd < 0) { fprintf(stderr, "Couldn't open file %s\n", path); return Q4_ERR_IO; }
    struct stat st;
    if (fstat(f.fd, &st) != 0) return Q4_ERR_IO;
    f.n = (size_t)st.st_size;
    if (f.n < sizeof(q4_config)) { fprintf(stderr, "Invalid header size\n"); return Q4_ERR_BAD_MODEL; }
    void* mp = mmap(nullptr, f.n, PROT_READ, MAP_PRIVATE, f.fd, 0);
    if (mp == MAP_FAILED) return Q4_ERR_IO;
    f.p = (const uint8_t*)mp;

    q4_config c;
    memcpy(&c, f.p, sizeof(c));
    if (c.dim <= 0 || c.hidden_dim <= 0 || c.n_layers <= 0 || c.n_heads <= 0 || c.n_kv_heads <= 0 || c.vocab_size <= 0 || c.dim % c.n_heads)
        return Q4_ERR_BAD_MODEL;
    const int kv_dim = (int)((long long)c.dim * c.n_kv_heads / c.n_heads);
    const size_t per_layer = 2 * qw_bytes(c.dim, c.dim) + 2 * qw_bytes(c.dim, kv_dim) + 2 * qw_bytes(c.dim, c.hidden_dim) +
                             qw_bytes(c.hidden_dim, c.dim) + 4 * (size_t)c.dim;
    const size_t expect = 32 + 4 * (size_t)c.vocab_size * c.dim + 2 * (size_t)c.dim + per_layer * c.n_layers;
    if (expect != f.n) { fprintf(stderr, "error reading weights"); return Q4_ERR_BAD_MODEL; }
    ModelSource src;
    src.file = f.p;
    return model_build(out, c, rank, gpu_count, tp_mode, comm, src);
}

extern "C" int q4_model_create_synthetic(q4_model** out, const q4_config* cfg, unsigned long long seed, int rank, int gpu_count, int tp_mode,
                                         q4_comm* comm) {
    if (!out || !cfg || gpu_count < 1 || gpu_count > Q4_MAX_GPUS || rank < 0 || rank >= gpu_count) return Q4_ERR_INVALID;
    if (gpu_count > 1 && tp_mode != Q4_TP_HYBRID && tp_mode != Q4_TP_COLUMN) return Q4_ERR_INVALID;
    if (gpu_count > 1 && !comm) return Q4_ERR_INVALID;
    ModelSource src;
    src.seed = seed;
    return model_build(out, *cfg, rank, gpu_count, tp_mode, comm, src);
}

extern "C" int q4_model_config(const q4_model* m, q4_config* out) {
    if (!m || !out) return Q4_ERR_INVALID;
    *out = m->cfg;
    return Q4_OK;
}
extern "C" q4_shared_data* q4_model_shared(q4_model* m) { return m ? m->shared : nullptr; }
extern "C" const uint16_t* q4_model_logits(const q4_model* m) { return m ? m->logits : nullptr; }
extern "C" const uint16_t* q4_model_x(const q4_model* m) { return m ? m->x : nullptr; }

extern "C" int q4_model_read(const q4_model* m, int what, uint16_t* host_out) {
    if (!m || !host_out || what < 0 || what > 1) return Q4_ERR_INVALID;
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    if (what == 0) Q4_CUDA_TRY(cudaMemcpy(host_out, m->logits, 2 * (size_t)m->cfg.vocab_size, cudaMemcpyDeviceToHost));
    else Q4_CUDA_TRY(cudaMemcpy(host_out, m->x, 2 * (size_t)m->cfg.dim, cudaMemcpyDeviceToHost));
    return Q4_OK;
}

extern "C" int q4_model_reset(q4_model* m, const int* prompt_tokens, int n, int pos) {
    if (!m || n < 0 || n > Q4_MAX_SEQ_LEN || pos < 0 || pos >= m->cfg.seq_len) return Q4_ERR_INVALID;
    // the embedding gather indexes the table with these ids on the device: refuse anything outside the vocabulary here
    if (prompt_tokens)
        for (int i = 0; i < n; i++)
            if (prompt_tokens[i] < 0 || prompt_tokens[i] >= m->cfg.vocab_size) return Q4_ERR_INVALID;
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    m->host_pos = pos;
    Q4_CUDA_TRY(cudaMemcpy(m->pos, &pos, sizeof(int), cudaMemcpyHostToDevice));
    m->shared->pos = pos;
    if (n > 0 && prompt_tokens) memcpy((void*)m->shared->tokens, prompt_tokens, sizeof(int) * (size_t)n);
    q4_fused_reset(m);
    return Q4_OK;
}

// The per-token schedule of run_llama_network (llama2_q4.cu:430-538), hybrid tensor parallelism when g > 1.
static int launch_token(q4_model* m, cudaStream_t s, int gen_token, bool handoff = true) {
    const q4_config& c = m->cfg;
    const int g = m->g, rank = m->rank;
    const int dim = c.dim, hs = m->head_size;
    int e;
#define OP(expr) do { e = (expr); if (e != Q4_OK) return e; } while (0)
    OP(q4_embed(s, m->x, m->emb, dim, (const int*)m->shared->tokens, m->pos));
    for (int l = 0; l < c.n_layers; l++) {
        const DevLayer& L = m->layers[l];
        const int loff = l * c.seq_len * m->kv_n;  // llama2_q4.cu:450
        OP(q4_rmsnorm(s, m->xb, m->x, L.rms_att, dim));
        OP(q4_qkv_matvec(s, m->q, m->kc, m->vc, m->xb, &L.q.w, &L.k.w, &L.v.w, dim, m->q_n, m->kv_n, loff, m->pos));
        OP(q4_rope(s, m->q, m->kc, c.n_heads / g, c.n_kv_heads / g, hs, m->pos, loff, c.rope_theta));
        OP(q4_attention(s, m->xb + m->o_kb, m->q, m->kc + loff, m->vc + loff, m->attn_scratch, c.n_heads / g, hs, m->kv_mul,
                        c.seq_len, m->pos));
        const int xs = rank * (dim / g), xn = dim / g;   // this rank's slice of x in column mode
        if (m->column) {   // llama2_q4.cu:479-493: gather the attention output, o projection on a column slice, gather x
            OP(q4_all_gather(m->comm, s, m->xb + m->o_kb, m->xb, m->o_kc));
            OP(q4_matmul_q4(s, m->x + xs, m->xb, &L.o.w, dim, xn, 1, 1, -1, nullptr));
            OP(q4_all_gather(m->comm, s, m->x + xs, m->x, xn));
        } else {
            OP(q4_matmul_q4(s, m->x, m->xb + m->o_kb, &L.o.w, m->o_kc, dim, 1, g, -1, nullptr));
            if (g > 1) OP(q4_all_reduce(m->comm, s, m->x, dim));
        }
        OP(q4_rmsnorm(s, m->xb, m->x, L.rms_ffn, dim));
        OP(q4_ffn_matvec_silu(s, m->hb + m->h_kb, m->xb, &L.gate.w, &L.up.w, dim, m->h_kc));
        if (m->column) {   // llama2_q4.cu:510-524
            OP(q4_all_gather(m->comm, s, m->hb + m->h_kb, m->hb, m->h_kc));
            OP(q4_matmul_q4(s, m->x + xs, m->hb, &L.down.w, c.hidden_dim, xn, 1, 1, -1, nullptr));
            OP(q4_all_gather(m->comm, s, m->x + xs, m->x, xn));
        } else {
            OP(q4_matmul_q4(s, m->x, m->hb + m->h_kb, &L.down.w, m->h_kc, dim, 1, g, -1, nullptr));
            if (g > 1) OP(q4_all_reduce(m->comm, s, m->x, dim));
        }
    }
    OP(q4_rmsnorm(s, m->x, m->x, m->rms_final, dim));
    OP(q4_matmul_f16(s, m->logits + (size_t)rank * m->v_n, m->x, m->wcls, dim, m->v_n, 1.0f));
    if (g > 1) OP(q4_all_gather(m->comm, s, m->logits + (size_t)rank * m->v_n, m->logits, m->v_n));
    if (handoff) OP(q4_argmax(s, m->logits, c.vocab_size, (int*)m->shared->tokens, &m->shared->pos, m->pos, gen_token));
#undef OP
    return Q4_OK;
}

extern "C" int q4_model_forward(q4_model* m, void* stream, int gen_token, int path) {
    if (!m) return Q4_ERR_INVALID;
    cudaStream_t s = (cudaStream_t)stream;
    gen_token = gen_token != 0;
    if (path < 0 || path > 2) return Q4_ERR_INVALID;
    // One call = one position. The kernels write K/V row `pos` and tokens[pos + 1]: a call past the model's sequence
    // length would write outside the cache, so it is refused here (the host counts the calls since the last reset; the
    // device-side position cannot be read without waiting for the stream).
    if (m->host_pos >= m->cfg.seq_len || m->host_pos >= Q4_MAX_SEQ_LEN - 1) return Q4_ERR_LIMIT;
    m->host_pos++;
    // sample() draws one coin per call, used or not (sampler.h:79); the greedy branch is taken at temperature 0 and for
    // prompt positions (sampler.h:81)
    const float coin = q4_random_f32(&m->rng_state);
    const bool sampled = m->temperature != 0.0f && gen_token;
    int e = Q4_OK;
    if (path == 0) {
        e = launch_token(m, s, gen_token, !sampled);
    } else if (path == 1) {
        const int gi = sampled ? 2 : gen_token;
        if (!m->graph_ready[gi]) {
            cudaGraph_t graph = nullptr;
            Q4_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
            e = launch_token(m, s, gen_token, !sampled);
            cudaError_t ce = cudaStreamEndCapture(s, &graph);
            if (e != Q4_OK) { if (graph) cudaGraphDestroy(graph); return e; }
            Q4_CUDA_TRY(ce);
            Q4_CUDA_TRY(cudaGraphInstantiate(&m->graph[gi], graph, 0));
            Q4_CUDA_TRY(cudaGraphDestroy(graph));
            m->graph_ready[gi] = true;
        }
        Q4_CUDA_TRY(cudaGraphLaunch(m->graph[gi], s));
    } else {
        if ((e = q4_fused_prepare(m)) != Q4_OK) return e;
        e = q4_fused_forward(m, s, gen_token, sampled);
    }
    if (e != Q4_OK || !sampled) return e;
    return q4_sample_topp(s, m->logits, m->cfg.vocab_size, m->temperature, m->topp, coin, (int*)m->shared->tokens, &m->shared->pos, m->pos);
}

/* build_sampler (sampler.h:28-45): temperature 0 decodes greedily. */
extern "C" int q4_model_set_sampler(q4_model* m, float temperature, float topp, unsigned long long seed) {
    if (!m || temperature < 0.0f) return Q4_ERR_INVALID;
    m->temperature = temperature;
    m->topp = topp;
    m->rng_state = seed;
    return Q4_OK;
}

extern "C" int q4_model_prepare(q4_model* m, int path) {
    if (!m || path < 0 || path > 2) return Q4_ERR_INVALID;
    return path == 2 ? q4_fused_prepare(m) : Q4_OK;
}

extern "C" int q4_model_set_wait_limit_ns(q4_model* m, unsigned long long ns) {
    if (!m) return Q4_ERR_INVALID;
    if (int e = q4_fused_prepare(m)) return e;
    q4_fused_set_wait_limit(m, ns);
    return Q4_OK;
}

extern "C" int q4_model_status(q4_model* m) {
    if (!m) return Q4_ERR_INVALID;
    Q4_CUDA_TRY(cudaDeviceSynchronize());
    int st = q4_fused_status(m);
    if (st == Q4_OK) st = q4_rows_status(m);
    if (st == Q4_OK && m->comm) st = q4_comm_status(m->comm);
    return st;
}

extern "C" int q4_generate(q4_model* m, const int* prompt_tokens, int n_prompt, int steps, int path, int* out_tokens, int* timed_tokens,
                           double* seconds) {
    if (!m || !prompt_tokens || n_prompt < 1) return Q4_ERR_INVALID;
    if (steps <= 0 || steps > m->cfg.seq_len) steps = m->cfg.seq_len;  // llama2_q4.cu:917
    cudaStream_t s;
    Q4_CUDA_TRY(cudaStreamCreate(&s));
    int e = q4_model_reset(m, prompt_tokens, n_prompt, 0);
    if (e != Q4_OK) { cudaStreamDestroy(s); return e; }
    int pos = 0;
    const bool one_pass = (path & Q4_PATH_PROMPT_ONE_PASS) != 0;
    path &= ~Q4_PATH_PROMPT_ONE_PASS;
    const auto start = std::chrono::steady_clock::now();
    if (one_pass && n_prompt > 1 && steps > n_prompt - 1) {
        // all prompt positions but the last in one pass; the last one goes through the token path, which also draws the
        // first generated id (greedy or sampled). A model the many-row kernels do not serve falls back to the loop.
        e = q4_model_prefill(m, s, n_prompt - 1, 0);
        if (e == Q4_OK) pos = n_prompt - 1;
        else if (e != Q4_ERR_UNSUPPORTED_SIZE) { cudaStreamDestroy(s); return e; }
    }
    while (pos < steps) {
        cudaStreamSynchronize(s);  // previous token done; its id is in the mailbox
        e = q4_model_forward(m, s, pos >= n_prompt - 1, path);
        if (e != Q4_OK) break;
        if (pos > 0) {
            int next = m->shared->tokens[pos];
            if (next >= m->cfg.vocab_size || next < 0) next = 0;
            if (next == 2) break;  // EOS, tokenizer.h:9
        }
        pos++;
    }
    cudaError_t ce = cudaStreamSynchronize(s);
    const auto end = std::chrono::steady_clock::now();
    cudaStreamDestroy(s);
    if (e != Q4_OK) return e;
    Q4_CUDA_TRY(ce);
    if (seconds) *seconds = std::chrono::duration<double>(end - start).count();
    if (timed_tokens) *timed_tokens = pos - 1;
    if (out_tokens) {
        const int upto = steps < Q4_MAX_SEQ_LEN - 1 ? steps : Q4_MAX_SEQ_LEN - 1;
        for (int i = 0; i <= upto; i++) out_tokens[i] = m->shared->tokens[i];
    }
    return Q4_OK;
}

extern "C" double q4_model_token_bytes(const q4_model* m, int pos) {
    if (!m) return 0;
    const q4_config& c = m->cfg;
    double b = 0;
    auto qb = [](int K, int N) { return (double)qw_bytes(K, N); };
    const DevLayer& L0 = m->layers[0];
    b += c.n_layers * (qb(c.dim, m->q_n) + 2 * qb(c.dim, m->kv_n) + qb(L0.o.K, L0.o.N) + 2 * qb(c.dim, m->h_kc) + qb(L0.down.K, L0.down.N));
    b += 2.0 * m->v_n * c.dim;                      // classifier
    b += 2.0 * c.dim * (2 * c.n_layers + 1);        // norm weights
    b += 2.0 * c.dim;                               // embedding row
    b += 2.0 * c.n_layers * m->kv_n * 2 * (pos + 1);  // K and V rows read
    b += 2.0 * c.n_layers * m->kv_n * 2;            // K and V row written
    return b;
}

extern "C" int q4_model_time_ffn(q4_model* m, void* stream, int reps, double* total_ms, double* bytes_per_launch) {
    if (!m || reps < 1 || !total_ms || !bytes_per_launch) return Q4_ERR_INVALID;
    cudaStream_t s = (cudaStream_t)stream;
    const int dim = m->cfg.dim;
    cudaEvent_t e0, e1;
    Q4_CUDA_TRY(cudaEventCreate(&e0));
    Q4_CUDA_TRY(cudaEventCreate(&e1));
    int e = Q4_OK;
    for (int l = 0; l < m->cfg.n_layers && e == Q4_OK; l++)  // warm-up pass
        e = q4_ffn_matvec_silu(s, m->hb + m->h_kb, m->xb, &m->layers[l].gate.w, &m->layers[l].up.w, dim, m->h_kc);
    Q4_CUDA_TRY(cudaEventRecord(e0, s));
    for (int r = 0; r < reps && e == Q4_OK; r++)
        for (int l = 0; l < m->cfg.n_layers && e == Q4_OK; l++)
            e = q4_ffn_matvec_silu(s, m->hb + m->h_kb, m->xb, &m->layers[l].gate.w, &m->layers[l].up.w, dim, m->h_kc);
    Q4_CUDA_TRY(cudaEventRecord(e1, s));
    Q4_CUDA_TRY(cudaEventSynchronize(e1));
    float ms = 0.f;
    Q4_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *total_ms = ms;
    *bytes_per_launch = 2.0 * (double)qw_bytes(dim, m->h_kc) + 2.0 * dim + 2.0 * m->h_kc;
    return e;
}

// Measurement hook: one W4 wrapper (kind 0 q4_matmul_q4, 1 q4_qkv_matvec, 2 q4_ffn_matvec_silu) over `nmat` distinct
// matrices of one shape, captured as one CUDA graph (kind 1 takes three, kind 2 two matrices per launch) and replayed
// `reps` times between two events on `stream`, so that the weights come from HBM and not from L2 and no launch gap is
// timed. Returns microseconds per launch and the algorithmic bytes of one launch.
extern "C" int q4_time_q4_op(void* stream, int kind, uint16_t* y, uint16_t* y2, uint16_t* y3, const uint16_t* x, const q4_qweight* mats, int nmat,
                             int K, int N, int reps, const int* pPos, double* us_per_launch, double* bytes_per_launch) {
    if (!y || !x || !mats || nmat < 1 || reps < 1 || !us_per_launch || !bytes_per_launch || kind < 0 || kind > 2) return Q4_ERR_INVALID;
    const int per = kind == 1 ? 3 : kind == 2 ? 2 : 1;
    if (nmat < per || (kind == 1 && (!y2 || !y3 || !pPos))) return Q4_ERR_INVALID;
    cudaStream_t s = (cudaStream_t)stream;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    Q4_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    int e = Q4_OK, launches = 0;
    for (int i = 0; i + per <= nmat && e == Q4_OK; i += per, launches++) {
        if (kind == 0) e = q4_matmul_q4(s, y, x, &mats[i], K, N, 0, 1, -1, nullptr);
        else if (kind == 1) e = q4_qkv_matvec(s, y, y2, y3, x, &mats[i], &mats[i + 1], &mats[i + 2], K, N, N, 0, pPos);
        else e = q4_ffn_matvec_silu(s, y, x, &mats[i], &mats[i + 1], K, N);
    }
    cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (e != Q4_OK) { if (graph) cudaGraphDestroy(graph); return e; }
    Q4_CUDA_TRY(ce);
    Q4_CUDA_TRY(cudaGraphInstantiate(&exec, graph, 0));
    cudaEvent_t e0, e1;
    Q4_CUDA_TRY(cudaEventCreate(&e0));
    Q4_CUDA_TRY(cudaEventCreate(&e1));
    for (int r = 0; r < 3; r++) Q4_CUDA_TRY(cudaGraphLaunch(exec, s));   // warm-up
    Q4_CUDA_TRY(cudaEventRecord(e0, s));
    for (int r = 0; r < reps; r++) Q4_CUDA_TRY(cudaGraphLaunch(exec, s));
    Q4_CUDA_TRY(cudaEventRecord(e1, s));
    Q4_CUDA_TRY(cudaEventSynchronize(e1));
    float ms = 0.f;
    Q4_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    *us_per_launch = 1e3 * ms / ((double)reps * launches);
    *bytes_per_launch = per * (double)qw_bytes(K, N) + 2.0 * K + 2.0 * N * per / (kind == 2 ? 2 : 1);
    return Q4_OK;
}

// The same for the few-rows forms (kind 0 q4_matmul_q4_rows, 1 q4_qkv_matmul_rows, 2 q4_ffn_silu_rows) with M rows of x.
extern "C" int q4_time_q4_rows_op(void* stream, int kind, int M, uint16_t* y, uint16_t* y2, uint16_t* y3, const uint16_t* x, const q4_qweight* mats,
                                  int nmat, int K, int N, int reps, double* us_per_launch, double* bytes_per_launch) {
    if (!y || !x || !mats || nmat < 1 || reps < 1 || !us_per_launch || !bytes_per_launch || kind < 0 || kind > 2) return Q4_ERR_INVALID;
    const int per = kind == 1 ? 3 : kind == 2 ? 2 : 1;
    if (nmat < per || (kind == 1 && (!y2 || !y3))) return Q4_ERR_INVALID;
    cudaStream_t s = (cudaStream_t)stream;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    Q4_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    int e = Q4_OK, launches = 0;
    for (int i = 0; i + per <= nmat && e == Q4_OK; i += per, launches++) {
        if (kind == 0) e = q4_matmul_q4_rows(s, y, x, &mats[i], M, K, N, nullptr, 0.f);
        else if (kind == 1) e = q4_qkv_matmul_rows(s, y, y2, y3, x, &mats[i], &mats[i + 1], &mats[i + 2], M, K, N, N);
        else e = q4_ffn_silu_rows(s, y, x, &mats[i], &mats[i + 1], M, K, N);
    }
    cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (e != Q4_OK) { if (graph) cudaGraphDestroy(graph); return e; }
    Q4_CUDA_TRY(ce);
    Q4_CUDA_TRY(cudaGraphInstantiate(&exec, graph, 0));
    cudaEvent_t e0, e1;
    Q4_CUDA_TRY(cudaEventCreate(&e0));
    Q4_CUDA_TRY(cudaEventCreate(&e1));
    for (int r = 0; r < 3; r++) Q4_CUDA_TRY(cudaGraphLaunch(exec, s));   // warm-up
    Q4_CUDA_TRY(cudaEventRecord(e0, s));
    for (int r = 0; r < reps; r++) Q4_CUDA_TRY(cudaGraphLaunch(exec, s));
    Q4_CUDA_TRY(cudaEventRecord(e1, s));
    Q4_CUDA_TRY(cudaEventSynchronize(e1));
    float ms = 0.f;
    Q4_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    *us_per_launch = 1e3 * ms / ((double)reps * launches);
    *bytes_per_launch = per * (double)qw_bytes(K, N) + 2.0 * M * K + 2.0 * M * N * per / (kind == 2 ? 2 : 1);
    return Q4_OK;
}

// Measurement hook: `reps` in-place all-reduces of `count` halfs back to back on `stream` between two events (the
// caller aligns the ranks with a host barrier first and takes the maximum over the ranks).
extern "C" int q4_time_all_reduce(q4_comm* comm, void* stream, uint16_t* buf, int count, int reps, double* us_per_call) {
    if (!comm || !buf || reps < 1 || !us_per_call) return Q4_ERR_INVALID;
    cudaStream_t s = (cudaStream_t)stream;
    cudaEvent_t e0, e1;
    Q4_CUDA_TRY(cudaEventCreate(&e0));
    Q4_CUDA_TRY(cudaEventCreate(&e1));
    int e = Q4_OK;
    for (int r = 0; r < 10 && e == Q4_OK; r++) e = q4_all_reduce(comm, s, buf, count);
    Q4_CUDA_TRY(cudaEventRecord(e0, s));
    for (int r = 0; r < reps && e == Q4_OK; r++) e = q4_all_reduce(comm, s, buf, count);
    Q4_CUDA_TRY(cudaEventRecord(e1, s));
    Q4_CUDA_TRY(cudaEventSynchronize(e1));
    float ms = 0.f;
    Q4_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *us_per_call = 1e3 * ms / reps;
    return e;
}
