// Index builders for the Megatron-style GPT dataset (counterparts of the reference's pybind helpers,
// lm_engine/data/megatron/utils/helpers.cpp:17-136), exposed through a plain C ABI.
#include "lme_host.h"

#include <algorithm>
#include <vector>

extern "C" int64_t lme_num_samples(int64_t num_epochs, int64_t tokens_per_epoch, int64_t seq_length) {
    return (num_epochs * tokens_per_epoch - 1) / seq_length;
}

extern "C" int lme_build_sample_idx(const int32_t* sizes, const int32_t* doc_idx, int64_t doc_idx_len,
                                    int64_t seq_length, int64_t num_samples, int64_t* out) {
    // A sample is seq_length + 1 tokens; consecutive samples overlap by one token (the label of the last input
    // position), so each sample starts on the token where the previous one ended.
    int64_t cursor = 0;   // position in doc_idx
    int64_t offset = 0;   // token offset inside doc_idx[cursor]
    out[0] = 0;
    out[1] = 0;
    for (int64_t s = 1; s <= num_samples; ++s) {
        int64_t need = seq_length + 1;
        while (need > 0) {
            if (cursor >= doc_idx_len) return -1;
            const int64_t avail = static_cast<int64_t>(sizes[doc_idx[cursor]]) - offset;
            if (avail >= need) {
                offset += need - 1;  // stay on the last consumed token: it is the next sample's first token
                need = 0;
            } else {
                need -= avail;
                ++cursor;
                offset = 0;
            }
        }
        out[2 * s] = cursor;
        out[2 * s + 1] = offset;
    }
    return 0;
}

extern "C" int lme_build_blending_indices(int16_t* dataset_index, int64_t* dataset_sample_index,
                                          const double* weights, int32_t num_datasets, int64_t size) {
    if (num_datasets <= 0) return -1;
    std::vector<int64_t> taken(num_datasets, 0);
    for (int64_t i = 0; i < size; ++i) {
        const double scale = static_cast<double>(std::max<int64_t>(i, 1));
        int32_t pick = 0;
        double worst = weights[0] * scale - static_cast<double>(taken[0]);
        for (int32_t d = 1; d < num_datasets; ++d) {
            const double lag = weights[d] * scale - static_cast<double>(taken[d]);
            if (lag > worst) {
                worst = lag;
                pick = d;
            }
        }
        dataset_index[i] = static_cast<int16_t>(pick);
        dataset_sample_index[i] = taken[pick]++;
    }
    return 0;
}
