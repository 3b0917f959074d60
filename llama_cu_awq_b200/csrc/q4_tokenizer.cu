// Tokenizer of the llama2_q4 command line, behind the C ABI (host code only): the llama2.c-format vocabulary file
// (tokenizer.bin: uint32 max_token_length, then per token float32 score, int32 length, bytes) and the behaviour of
// build_tokenizer / encode / decode / safe_printf (tokenizer.h:36-223): greedy best-score pair merging over UTF-8
// code points with byte fallback (+3), a dummy-prefix space, the leading space stripped after BOS, <0xXX> pieces
// mapped to raw bytes. The reference's tokenizer.bin holds its byte pieces twice (e.g. "," as id 47 and as id 29892), and
// which id a lookup returns decides the token stream: lookups therefore probe a stably sorted table exactly like the C
// library's binary search does over the reference's sorted array (first probe at (lo + hi) / 2, lower half on "less").
#include <ctype.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../include/q4b200.h"

struct q4_tokenizer {
    std::vector<std::string> pieces;
    std::vector<float> scores;
    std::vector<int> sorted;   // ids ordered by piece (byte-wise, as strcmp orders them), equal pieces in id order
    std::string scratch;       // storage behind the pointer q4_tokenizer_decode returns

    // id of `key`, or -1 (str_lookup, tokenizer.h:102-106)
    int lookup(const std::string& key) const {
        size_t lo = 0, hi = sorted.size();
        while (lo < hi) {
            const size_t mid = (lo + hi) / 2;
            const int c = strcmp(key.c_str(), pieces[sorted[mid]].c_str());
            if (c < 0) hi = mid;
            else if (c > 0) lo = mid + 1;
            else return sorted[mid];
        }
        return -1;
    }
};

namespace {
constexpr int kBos = 1, kEos = 2;  // tokenizer.h:8-9
}

extern "C" int q4_tokenizer_load(q4_tokenizer** out, const char* path, int vocab_size) {
    if (!out || !path || vocab_size <= 0) return Q4_ERR_INVALID;
    FILE* f = fopen(path, "rb");
    if (!f) return Q4_ERR_IO;
    q4_tokenizer* t = new q4_tokenizer();
    uint32_t max_len = 0;
    bool ok = fread(&max_len, 4, 1, f) == 1;
    t->pieces.resize(vocab_size);
    t->scores.resize(vocab_size);
    for (int i = 0; ok && i < vocab_size; i++) {
        int len = 0;
        ok = fread(&t->scores[i], 4, 1, f) == 1 && fread(&len, 4, 1, f) == 1 && len >= 0 && len < (1 << 20);
        if (!ok) break;
        t->pieces[i].resize(len);
        if (len) ok = fread(&t->pieces[i][0], len, 1, f) == 1;
        if (ok) t->pieces[i].resize(strlen(t->pieces[i].c_str()));   // pieces are C strings in the reference: cut at a NUL byte
    }
    fclose(f);
    if (!ok) { delete t; return Q4_ERR_IO; }
    t->sorted.resize(vocab_size);
    for (int i = 0; i < vocab_size; i++) t->sorted[i] = i;
    std::stable_sort(t->sorted.begin(), t->sorted.end(),
                     [&](int a, int b) { return strcmp(t->pieces[a].c_str(), t->pieces[b].c_str()) < 0; });
    *out = t;
    return Q4_OK;
}

extern "C" void q4_tokenizer_free(q4_tokenizer* t) { delete t; }

extern "C" int q4_tokenizer_encode(const q4_tokenizer* t, const char* text, int bos, int eos, int* tokens, int max_tokens, int* n_tokens) {
    if (!t || !text || !tokens || !n_tokens || max_tokens < 0) return Q4_ERR_INVALID;
    const size_t len = strlen(text);
    std::vector<int> out;
    out.reserve(len + 3);
    if (bos) out.push_back(kBos);
    if (len) {   // dummy prefix, only for non-empty text (tokenizer.h:136-140; -1 when the vocabulary has no " ")
        out.push_back(t->lookup(" "));
    }
    for (size_t i = 0; i < len;) {
        size_t n = 1;   // one UTF-8 code point: a byte and its continuation bytes, four bytes at most
        while (i + n < len && (static_cast<unsigned char>(text[i + n]) & 0xC0) == 0x80 && n < 4) n++;
        const int id = t->lookup(std::string(text + i, n));
        if (id >= 0) out.push_back(id);
        else
            for (size_t b = 0; b < n; b++) out.push_back(static_cast<unsigned char>(text[i + b]) + 3);
        i += n;
    }
    for (int id : out)
        if (id < 0 || id >= (int)t->pieces.size()) return Q4_ERR_BAD_MODEL;   // the vocabulary lacks " " or the byte pieces
    for (;;) {   // merge the best-scoring adjacent pair until none is left (first position wins among equal scores)
        float best = -1e10f;
        int best_id = -1;
        size_t best_at = 0;
        for (size_t i = 0; i + 1 < out.size(); i++) {
            const int id = t->lookup(t->pieces[out[i]] + t->pieces[out[i + 1]]);
            if (id >= 0 && t->scores[id] > best) { best = t->scores[id]; best_id = id; best_at = i; }
        }
        if (best_id < 0) break;
        out[best_at] = best_id;
        out.erase(out.begin() + best_at + 1);
    }
    if (eos) out.push_back(kEos);
    *n_tokens = (int)out.size();
    if ((int)out.size() > max_tokens) return Q4_ERR_LIMIT;
    memcpy(tokens, out.data(), out.size() * sizeof(int));
    return Q4_OK;
}

extern "C" const char* q4_tokenizer_decode(q4_tokenizer* t, int prev_token, int token) {
    if (!t || token < 0 || token >= (int)t->pieces.size()) return "";
    const char* piece = t->pieces[token].c_str();
    if (prev_token == kBos && piece[0] == ' ') piece++;
    unsigned byte = 0;
    if (sscanf(piece, "<0x%02X>", &byte) == 1) {   // raw-byte piece (tokenizer.h:78-82)
        t->scratch.assign(1, (char)byte);
        piece = t->scratch.c_str();
        if (byte == 0) return "";
    }
    // safe_printf (tokenizer.h:88-100): a single unprintable byte is not shown
    if (piece[0] != '\0' && piece[1] == '\0') {
        const unsigned char c = (unsigned char)piece[0];
        if (!(isprint(c) || isspace(c))) return "";
    }
    return piece;
}
