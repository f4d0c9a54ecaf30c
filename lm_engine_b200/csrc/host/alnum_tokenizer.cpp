// Character-level tokenizer over [0-9a-zA-Z] (vocabulary of the reference's AlphaNumericTokenizer,
// lm_engine/tokenizers/alpha_numeric/alpha_numeric.cpp:14-149).
#include "lme_host.h"

#include <string.h>

static const char kEosLiteral[] = "<|endoftext|>";

static inline int char_to_id(unsigned char c) {
    if (c >= '0' && c <= '9') return c - '0';
    if (c >= 'a' && c <= 'z') return 10 + (c - 'a');
    if (c >= 'A' && c <= 'Z') return 36 + (c - 'A');
    return -1;
}

extern "C" int64_t lme_alnum_encode(const char* text, int64_t len, int add_eos, int32_t* out, int64_t* bad_pos) {
    int64_t n = 0;
    const int64_t lit = static_cast<int64_t>(sizeof(kEosLiteral)) - 1;
    for (int64_t i = 0; i < len;) {
        if (text[i] == '<' && i + lit <= len && memcmp(text + i, kEosLiteral, lit) == 0) {
            out[n++] = LME_ALNUM_EOS;
            i += lit;
            continue;
        }
        const int id = char_to_id(static_cast<unsigned char>(text[i]));
        if (id < 0) {
            if (bad_pos) *bad_pos = i;
            return -1;
        }
        out[n++] = id;
        ++i;
    }
    if (add_eos) out[n++] = LME_ALNUM_EOS;
    return n;
}

extern "C" int64_t lme_alnum_encode_batch(const char* const* texts, const int64_t* lens, int64_t n, int add_eos,
                                          int pad, int32_t* out, int32_t* mask, int64_t max_len) {
    for (int64_t r = 0; r < n; ++r) {
        int32_t* row = out + r * max_len;
        int32_t* mrow = mask + r * max_len;
        // encode at the start of the row, then shift right (left padding)
        int64_t bad = 0;
        const int64_t k = lme_alnum_encode(texts[r], lens[r], add_eos, row, &bad);
        if (k < 0 || k > max_len) return -1;
        const int64_t shift = pad ? max_len - k : 0;
        if (shift > 0) memmove(row + shift, row, static_cast<size_t>(k) * sizeof(int32_t));
        for (int64_t i = 0; i < shift; ++i) {
            row[i] = LME_ALNUM_EOS;
            mrow[i] = 0;
        }
        for (int64_t i = shift; i < shift + k; ++i) mrow[i] = 1;
        for (int64_t i = shift + k; i < max_len; ++i) {
            row[i] = LME_ALNUM_EOS;
            mrow[i] = 0;
        }
    }
    return max_len;
}

extern "C" int64_t lme_alnum_decode(const int32_t* ids, int64_t n, int skip_special, char* out, int64_t cap) {
    int64_t w = 0;
    const int64_t lit = static_cast<int64_t>(sizeof(kEosLiteral)) - 1;
    for (int64_t i = 0; i < n; ++i) {
        const int32_t id = ids[i];
        if (id >= 0 && id < 10) {
            if (w + 1 > cap) return -1;
            out[w++] = static_cast<char>('0' + id);
        } else if (id < 36 && id >= 10) {
            if (w + 1 > cap) return -1;
            out[w++] = static_cast<char>('a' + id - 10);
        } else if (id < 62 && id >= 36) {
            if (w + 1 > cap) return -1;
            out[w++] = static_cast<char>('A' + id - 36);
        } else if (id == LME_ALNUM_EOS) {
            if (skip_special) continue;
            if (w + lit > cap) return -1;
            memcpy(out + w, kEosLiteral, static_cast<size_t>(lit));
            w += lit;
        } else {
            return -2;
        }
    }
    return w;
}
