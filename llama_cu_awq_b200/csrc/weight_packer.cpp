// weight_packer: HuggingFace config.json + raw AWQ tensors (one .bin per tensor, as convert_awq_to_bin.py dumps them)
// -> one packed model file in the layout the decode path loads (header, embedding, classifier, final norm, then per
// layer q k v o up gate down + the two norm vectors). Same command line and the same output bytes as the reference's
// tool (weight_packer.cpp:233-297), with one deliberate difference: zero-point nibbles past a row's last group are
// written as 0, where the reference's re-packer leaves whatever its scratch buffer held (weight_packer.cpp:117-121 reads
// past `height` when the group count is not a multiple of 8); no kernel ever reads those nibbles.
//
//   weight_packer <config.json> <dir with the .bin tensors> <output file> <old AWQ format: 0 or 1>
//
// Old AWQ format (1): qweight u32[K][N/8] and qzeros u32[G][N/8], eight outputs per word with nibble i holding output
// 8j + order[i], order = 0,2,4,6,1,3,5,7; scales f16[G][N]. New format (0): qweight u32[N][K/8], qzeros u32[N][ceil(G/8)],
// scales f16[N][8*ceil(G/8)] (padded). Output per matrix: weight u32[N][ceil(K/8)] (nibble i of word j = input 8j+i),
// zeros u32[N][ceil(G/8)], scales f16[N][G], G = ceil(K/128).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Header {
    int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
    float rope_theta;
};

[[noreturn]] void fail(const std::string& what) {
    printf("%s\n", what.c_str());
    exit(1);
}

// The value after "key": in the JSON text (the reference scans the text the same way: first occurrence, atoi / atof).
bool find_number(const std::string& json, const char* key, double* out) {
    const std::string pat = std::string("\"") + key + "\":";
    const size_t at = json.find(pat);
    if (at == std::string::npos) return false;
    *out = atof(json.c_str() + at + pat.size());
    return true;
}

Header read_config(const char* path) {
    FILE* f = fopen(path, "rb");
    if (!f) fail("unable to open config file");
    std::string json;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) json.append(buf, n);
    fclose(f);
    if (json.empty()) fail("unable to read config file");
    Header h;
    double v;
    auto need = [&](const char* key) {
        if (!find_number(json, key, &v)) fail(std::string("error parsing config.json ") + key + " not found");
        return (int32_t)v;
    };
    h.dim = need("hidden_size");
    h.hidden_dim = need("intermediate_size");
    h.n_layers = need("num_hidden_layers");
    h.n_heads = need("num_attention_heads");
    h.n_kv_heads = find_number(json, "num_key_value_heads", &v) ? (int32_t)v : h.n_heads;
    h.vocab_size = need("vocab_size");
    h.seq_len = need("max_position_embeddings");
    h.rope_theta = find_number(json, "rope_theta", &v) ? (float)v : 10000.0f;
    printf("\nModel params:- \ndim: %d \nhidden_dim: %d\nn_heads: %d\nn_kv_heads: %d\nn_layers: %d\nseq_len: %d\nvocab_size: %d\nrope_theta: %g\n", h.dim,
           h.hidden_dim, h.n_heads, h.n_kv_heads, h.n_layers, h.seq_len, h.vocab_size, h.rope_theta);
    return h;
}

std::vector<uint8_t> read_exact(const std::string& path, size_t bytes) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) fail("\nUnable to open " + path);
    std::vector<uint8_t> buf(bytes);
    if (fread(buf.data(), 1, bytes, f) != bytes) fail("error reading weights from " + path);
    fclose(f);
    return buf;
}

void write_all(FILE* out, const void* p, size_t bytes, const std::string& what) {
    if (fwrite(p, 1, bytes, out) != bytes) fail("error writing output file from input " + what);
}

size_t div_up(size_t a, size_t b) { return (a + b - 1) / b; }

// rows x cols nibbles held N-packed with AWQ's order map (u32[rows][cols/8]) -> transposed and packed along the former
// row index: u32[cols][ceil(rows/8)], nibble (r % 8) of word r / 8 in output row c = element (r, c).
std::vector<uint32_t> transpose_pack(const uint32_t* in, size_t rows, size_t cols) {
    static const int order[8] = {0, 2, 4, 6, 1, 3, 5, 7};
    const size_t words_in = cols / 8, words_out = div_up(rows, 8);
    std::vector<uint32_t> out(cols * words_out, 0u);
    for (size_t r = 0; r < rows; r++) {
        const unsigned shift = 4 * (unsigned)(r & 7);
        const size_t wo = r >> 3;
        for (size_t j = 0; j < words_in; j++) {
            const uint32_t w = in[r * words_in + j];
            for (int i = 0; i < 8; i++) out[(j * 8 + order[i]) * words_out + wo] |= ((w >> (4 * i)) & 0xFu) << shift;
        }
    }
    return out;
}

void pack_matrix(FILE* out, const std::string& base, const char* name, size_t K, size_t N, bool old_format) {
    const size_t G = div_up(K, 128), PW = div_up(K, 8), PZ = div_up(G, 8);
    const std::string stem = base + "." + name;
    if (old_format) {
        if (N % 8) fail("output size of " + stem + " is not a multiple of 8");
        const std::vector<uint8_t> qw = read_exact(stem + ".qweight.bin", K * (N / 8) * 4);
        const std::vector<uint8_t> qz = read_exact(stem + ".qzeros.bin", G * (N / 8) * 4);
        const std::vector<uint8_t> sc = read_exact(stem + ".scales.bin", G * N * 2);
        const std::vector<uint32_t> w = transpose_pack(reinterpret_cast<const uint32_t*>(qw.data()), K, N);
        const std::vector<uint32_t> z = transpose_pack(reinterpret_cast<const uint32_t*>(qz.data()), G, N);
        std::vector<uint16_t> s(N * G);
        const uint16_t* sin = reinterpret_cast<const uint16_t*>(sc.data());
        for (size_t g = 0; g < G; g++)
            for (size_t n = 0; n < N; n++) s[n * G + g] = sin[g * N + n];
        write_all(out, w.data(), w.size() * 4, stem);
        write_all(out, z.data(), z.size() * 4, stem);
        write_all(out, s.data(), s.size() * 2, stem);
    } else {
        const size_t padded = PZ * 8;   // the AWQ exporter pads the scales of a row to a multiple of 8
        const std::vector<uint8_t> qw = read_exact(stem + ".qweight.bin", N * PW * 4);
        const std::vector<uint8_t> qz = read_exact(stem + ".qzeros.bin", N * PZ * 4);
        const std::vector<uint8_t> sc = read_exact(stem + ".scales.bin", N * padded * 2);
        std::vector<uint16_t> s(N * G);
        const uint16_t* sin = reinterpret_cast<const uint16_t*>(sc.data());
        for (size_t n = 0; n < N; n++) memcpy(&s[n * G], sin + n * padded, G * 2);
        write_all(out, qw.data(), qw.size(), stem);
        write_all(out, qz.data(), qz.size(), stem);
        write_all(out, s.data(), s.size() * 2, stem);
    }
}

void copy_tensor(FILE* out, const std::string& path, size_t bytes) {
    const std::vector<uint8_t> buf = read_exact(path, bytes);
    write_all(out, buf.data(), bytes, path);
}

}  // namespace

int main(int argc, char* argv[]) {
    if (argc != 5) {
        printf("usage: weight_packer <config.json from huggingface> <path_to_awq_bin_weights> <output_bin_filename> [OldAwqFormat: 0 or 1]\n");
        return 0;
    }
    const Header h = read_config(argv[1]);
    const std::string dir = argv[2];
    const bool old_format = atoi(argv[4]) != 0;
    FILE* out = fopen(argv[3], "wb+");
    if (!out) { printf("unable to open output file\n"); return 0; }
    if (fwrite(&h, sizeof(h), 1, out) != 1) { printf("unable to write model metadata\n"); return 0; }
    const size_t dim = h.dim, hid = h.hidden_dim, vocab = h.vocab_size;
    copy_tensor(out, dir + "/model.embed_tokens.weight.bin", vocab * dim * 2);
    copy_tensor(out, dir + "/lm_head.weight.bin", vocab * dim * 2);
    copy_tensor(out, dir + "/model.norm.weight.bin", dim * 2);
    const size_t kv_dim = dim * h.n_kv_heads / h.n_heads;
    for (int l = 0; l < h.n_layers; l++) {
        printf("\nProcessing weights for layer: %d\n", l);
        const std::string base = dir + "/model.layers." + std::to_string(l);
        pack_matrix(out, base, "self_attn.q_proj", dim, dim, old_format);
        pack_matrix(out, base, "self_attn.k_proj", dim, kv_dim, old_format);
        pack_matrix(out, base, "self_attn.v_proj", dim, kv_dim, old_format);
        pack_matrix(out, base, "self_attn.o_proj", dim, dim, old_format);
        pack_matrix(out, base, "mlp.up_proj", dim, hid, old_format);     // up before gate: the order the loader reads
        pack_matrix(out, base, "mlp.gate_proj", dim, hid, old_format);
        pack_matrix(out, base, "mlp.down_proj", hid, dim, old_format);
        copy_tensor(out, base + ".input_layernorm.weight.bin", dim * 2);
        copy_tensor(out, base + ".post_attention_layernorm.weight.bin", dim * 2);
    }
    printf("\nDone!\n");
    fclose(out);
    return 0;
}
