// C ABI of liblme_host.so: host-side helpers that would be too slow in Python.
#pragma once
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

// ---- dataset index builders (GPT pretraining samples spanning document boundaries) ----
// Number of samples of seq_length (+1 overlapping label token) that num_epochs passes over the documents yield.
int64_t lme_num_samples(int64_t num_epochs, int64_t tokens_per_epoch, int64_t seq_length);
// out: int64[(num_samples + 1) * 2] rows of (index into doc_idx, token offset inside that document).
// doc_idx: int32[doc_idx_len] shuffled document order (epochs concatenated); sizes: int32 length per document.
int lme_build_sample_idx(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len, int64_t seq_length,
                         int64_t num_samples, int64_t* out);
// Greedy interleave of n datasets by weight: at every step the dataset that lags its quota the most is sampled.
int lme_build_blending_indices(int16_t* dataset_index, int64_t* dataset_sample_index, const double* weights,
                               int32_t num_datasets, int64_t size);

// ---- character-level alpha-numeric tokenizer: 0-9 -> 0..9, a-z -> 10..35, A-Z -> 36..61, EOS/pad = 62 ----
#define LME_ALNUM_EOS 62
#define LME_ALNUM_VOCAB 63
// returns number of ids written, -1 on an unsupported character (its byte position goes to *bad_pos)
int64_t lme_alnum_encode(const char* text, int64_t len, int add_eos, int32_t* out, int64_t* bad_pos);
// left-pads every row of a batch to the longest; out/mask are [n, max_len]; returns max_len or -1
int64_t lme_alnum_encode_batch(const char* const* texts, const int64_t* lens, int64_t n, int add_eos, int pad,
                               int32_t* out, int32_t* mask, int64_t max_len);
// writes the decoded string (no terminator) and returns its length; ids >= 62 are written as the EOS literal
// unless skip_special
int64_t lme_alnum_decode(const int32_t* ids, int64_t n, int skip_special, char* out, int64_t cap);

#ifdef __cplusplus
}
#endif
