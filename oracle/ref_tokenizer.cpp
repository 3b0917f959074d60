// Harness around the reference's own tokenizer (tokenizer.h, plain host code), compiled from where the reference
// lies (-I$REF, nothing copied). TEST INFRASTRUCTURE ONLY: used to record tests/golden/tokenizer_golden.json and,
// where the reference is present, to compare live against q4_tokenizer_*.
#include <ctype.h>
#include <stdint.h>
#include <stdio.h>

#include "tokenizer.h"

extern "C" {

void* ref_tok_open(const char* path, int vocab_size) {
    Tokenizer* t = new Tokenizer();
    build_tokenizer(t, (char*)path, vocab_size);
    return t;
}

int ref_tok_encode(void* t, const char* text, int bos, int eos, int* tokens) {
    int n = 0;
    encode((Tokenizer*)t, (char*)text, (int8_t)bos, (int8_t)eos, tokens, &n);
    return n;
}

// decode() followed by the filter of safe_printf(): what the reference would print for the token
const char* ref_tok_decode(void* t, int prev, int token) {
    char* piece = decode((Tokenizer*)t, prev, token);
    if (piece == NULL || piece[0] == '\0') return "";
    if (piece[1] == '\0') {
        unsigned char b = piece[0];
        if (!(isprint(b) || isspace(b))) return "";
    }
    return piece;
}

void ref_tok_close(void* t) {
    free_tokenizer((Tokenizer*)t);
    delete (Tokenizer*)t;
}
}
