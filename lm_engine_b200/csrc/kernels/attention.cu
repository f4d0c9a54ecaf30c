// Flash-attention forward on tcgen05 (head dim 128, bf16, causal or full, grouped K/V heads).
//
// One CTA owns 128 query rows of one (batch, head) and streams the K/V sequence in tiles of 64 rows:
//   warp 0      TMA producer   Q once; K tiles through a 2-stage ring, V through one stage
//   warp 1      MMA issuer     S_j = Q K_j^T  (128 x 64 x 128, both operands K-major, accumulator in TMEM, two S
//                              buffers so S_{j+1} is computed while the softmax warps work on S_j), then
//                              O += P_j V_j (P from shared memory, V as an MN-major operand straight from its
//                              [kv, d] tile - no transpose anywhere)
//   warps 2..5  softmax        thread = query row (tcgen05.ld 32x32b hands every thread its own row, so max and sum
//                              need no shuffles): one pass over S from TMEM (max, exp2, sum, bf16 P written
//                              into the 128-byte-swizzled K-major layout the MMA expects).  O accumulates in TMEM
//                              across tiles; the exponents are taken against a maximum that trails the true one by
//                              at most 2^8, so the rescale of O - a TMEM read-modify-write - runs only on the few
//                              tiles where the maximum jumps.
// TMEM: S0 | S1 (64 columns each) | O (128) = 256 columns.  Shared memory: Q 32 KB, K 2 x 16 KB, V 16 KB,
// P 2 x 16 KB = 112 KB, so TWO CTAs share an SM (and its 512 TMEM columns): while one CTA's softmax warps keep the
// MUFU / FMA pipes busy the other's MMAs and loads proceed.  Every wait is bounded (common.cuh); a CTA that starts
// after an error was recorded returns at once.
//
// Role of flash-attn's forward kernels used by the reference (lm_engine/modeling_utils/sequence_mixer_blocks/
// softmax_attention/utils.py flash_attention; FA2 / FA3 / FA4 selection in lm_engine/kernels.py).
namespace lme {
namespace attn {

constexpr int BM = 128, BN = 64, HD = 128;
constexpr int Q_HALF = BM * 128;               // 128 rows x 64 bf16 (one 128-byte swizzled half of the head dim)
constexpr int KV_HALF = BN * 128;              // 64 rows x 64 bf16
constexpr int Q_BYTES = 2 * Q_HALF, KV_BYTES = 2 * KV_HALF, P_BYTES = BM * BN * 2;
// K has a 2-stage ring (the next S product is issued a tile ahead), V one stage (it is needed a whole softmax after
// the previous P V product released it), P two buffers (the softmax warps never wait for the MMA that reads P)
constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + 2 * KV_BYTES, OFF_P = OFF_V + KV_BYTES;
constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
// 112 KB of tiles + barriers: two CTAs share an SM, so the softmax of one overlaps the other's MMAs and waits
constexpr int SMEM_BYTES = OFF_BAR + 128;
constexpr uint32_t TMEM_COLS = 256;            // S0 | S1 (64 columns each) | O (128)
constexpr uint32_t TM_S = 0, TM_O = 128;

struct Args {
    __nv_bfloat16* o;
    float* lse;
    long long o_ld;            // row pitch of o in elements
    int B, S_q, S_kv, Hq, Hkv, causal;
    int window;                // > 0 (with causal): query i sees keys in (i + shift - window, i + shift]
    const int* cu_seqlens;     // packed sequences: tokens of sequence b are rows cu[b] .. cu[b+1]-1 (self-attention)
    int S_pad;                 // row pitch of lse: S_q, or the padded maximum length for packed sequences
    float scale;               // softmax scale (natural units)
    // K / V rows that arrive while the kernel runs (context parallelism: the peers' key / value chunks are copied
    // into this GPU's K / V buffers by copy engines, and the stream writes kv_seq into one word per chunk once a
    // chunk is complete).  The producer waits (bounded) for the word of a tile's chunk before loading the tile;
    // chunk = key row / kv_chunk_rows (a multiple of 64), one set of words per batch entry.  null: no waiting.
    const int* kv_ready;
    int kv_chunk_rows, kv_chunks, kv_seq;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(192, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const Args p) {
    extern __shared__ __align__(1024) uint8_t smem[];      // the swizzled tiles need 1024-byte alignment (checked)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    // Barriers that can be one completion ahead of their waiter come in pairs indexed by tile parity: a single
    // barrier whose phase ran two completions ahead would show the waiter the parity it is still waiting for.
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;     // [2]
    uint64_t* k_empty = bars + 3;    // [2]
    uint64_t* v_full = bars + 5;
    uint64_t* v_empty = bars + 6;
    uint64_t* s_full = bars + 7;     // [2]
    uint64_t* p_full = bars + 9;     // [2]
    uint64_t* pv_full = bars + 11;   // [2]
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 13);
    uint32_t* poisoned = tmem_base_smem + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // With key / value chunks that are still arriving from other GPUs the producer may wait as long as a peer wait
    // lasts; every barrier behind it gets that time on top of its own.
    const uint64_t wait_limit = p.kv_ready ? lme_peer_wait_ns + LME_WAIT_LIMIT_NS : LME_WAIT_LIMIT_NS;
    // blocks are handed out x first: x runs over (head, batch) and y over the query blocks, late (long) ones first,
    // so the longest blocks of ALL heads start first and the short ones fill the tail; neighbours in x share K / V
    const int qb = gridDim.y - 1 - blockIdx.y;
    const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
    const int hk = h / (p.Hq / p.Hkv);
    const int q0 = qb * BM;
    // rows of this sequence in the token-major operands, and its lengths
    int tok_q = b * p.S_q, tok_k = b * p.S_kv, len_q = p.S_q, len_k = p.S_kv;
    if (p.cu_seqlens != nullptr) {
        tok_q = tok_k = p.cu_seqlens[b];
        len_q = len_k = p.cu_seqlens[b + 1] - tok_q;
    }
    const int shift = len_k - len_q;                   // query row i may see keys <= i + shift
    int n_tiles = (len_k + BN - 1) / BN;
    if (p.causal) n_tiles = min(n_tiles, (q0 + BM + shift + BN - 1) / BN);
    if (q0 >= len_q) n_tiles = 0;                      // a query block past the end of a packed sequence
    // a sliding window also skips the tiles before the first key the first row sees; j below counts from there
    const int j_begin = (p.causal && p.window > 0) ? max(0, (q0 + shift - p.window + 1) / BN) : 0;
    n_tiles -= j_begin;

    if (threadIdx.x == 0) {
        *poisoned = lme_status[0];
        if (smem_u32(smem) & 1023u) {
            report_error(STATUS_BOUNDS, 680);
            *poisoned = 1u;
        }
    }
    __syncthreads();
    if (*poisoned != 0u || n_tiles <= 0) return;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1);
            mbar_init(&k_empty[s], 1);
            mbar_init(&s_full[s], 1);
            mbar_init(&p_full[s], 4);    // one arrival per softmax warp
            mbar_init(&pv_full[s], 1);
        }
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_smem, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    if (warp == 0) {
        if (lane == 0) {
            const int row_q = tok_q + q0;
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(smem + OFF_Q, &tmQ, q_full, h * HD, row_q);
            tma_load_2d(smem + OFF_Q + Q_HALF, &tmQ, q_full, h * HD + 64, row_q);
            int chunk_seen = -1;    // K / V chunks up to this one have been waited for (tiles run in key order)
            auto wait_chunk = [&](int j) -> bool {
                if (p.kv_ready == nullptr) return true;
                const int c = ((j_begin + j) * BN) / p.kv_chunk_rows;
                if (c <= chunk_seen) return true;
                for (int cc = max(chunk_seen + 1, (j_begin * BN) / p.kv_chunk_rows); cc <= c; ++cc)
                    // the word follows a peer's progress: the limit of the cross-GPU waits applies
                    if (!wait_flag_sys(&p.kv_ready[b * p.kv_chunks + cc], p.kv_seq, 650)) return false;
                fence_proxy_async_all();   // the TMA (async proxy) loads below are ordered after the acquire
                chunk_seen = c;
                return true;
            };
            auto load_k = [&](int j) -> bool {
                const int s = j & 1;
                if (!wait_chunk(j)) return false;
                if (!mbar_wait_limit(&k_empty[s], ((j >> 1) & 1) ^ 1, 600 + s, wait_limit)) return false;
                uint8_t* ks = smem + OFF_K + s * KV_BYTES;
                mbar_expect_tx(&k_full[s], KV_BYTES);
                tma_load_2d(ks, &tmK, &k_full[s], hk * HD, tok_k + (j_begin + j) * BN);
                tma_load_2d(ks + KV_HALF, &tmK, &k_full[s], hk * HD + 64, tok_k + (j_begin + j) * BN);
                return true;
            };
            bool ok = load_k(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                // K runs one tile ahead of V so that the wait for V's single stage never delays the next S product
                if (j + 1 < n_tiles && !load_k(j + 1)) break;
                if (!mbar_wait_limit(v_empty, (j & 1) ^ 1, 605, wait_limit)) break;
                uint8_t* vs = smem + OFF_V;
                mbar_expect_tx(v_full, KV_BYTES);
                tma_load_2d(vs, &tmV, v_full, hk * HD, tok_k + (j_begin + j) * BN);
                tma_load_2d(vs + KV_HALF, &tmV, v_full, hk * HD + 64, tok_k + (j_begin + j) * BN);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_qk = make_idesc(1, 1, false, false, BM, BN);
            const uint32_t idesc_pv = make_idesc(1, 1, false, true, BM, HD);
            const uint32_t sq = smem_u32(smem + OFF_Q);
            bool ok = mbar_wait_limit(q_full, 0, 610, wait_limit);
            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait_limit(&k_full[s], (j >> 1) & 1, 620 + s, wait_limit)) return false;
                tc_fence_after();
                const uint32_t sk = smem_u32(smem + OFF_K + s * KV_BYTES);
                const uint32_t d = tmem_base + TM_S + s * BN;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t qoff = (kk >> 2) * Q_HALF + (kk & 3) * 32;
                    const uint32_t koff = (kk >> 2) * KV_HALF + (kk & 3) * 32;
                    umma_bf16(d, make_smem_desc_sw128(sq + qoff, 16, 1024), make_smem_desc_sw128(sk + koff, 16, 1024),
                              idesc_qk, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[s]);
                umma_commit(&k_empty[s]);
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                if (j + 1 < n_tiles && !issue_qk(j + 1)) { ok = false; break; }
                if (!mbar_wait_limit(&p_full[s], (j >> 1) & 1, 630 + s, wait_limit)) { ok = false; break; }
                if (!mbar_wait_limit(v_full, j & 1, 640, wait_limit)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sv = smem_u32(smem + OFF_V);
                const uint32_t sp = smem_u32(smem + OFF_P + s * P_BYTES);
                const uint32_t d = tmem_base + TM_O;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {
                    // P: one 64-column half, 32 bytes per k-step.  V: 16 key rows per k-step, the two 64-wide
                    // halves of the head dim KV_HALF bytes apart
                    umma_bf16(d, make_smem_desc_sw128(sp + kk * 32, 16, 1024),
                              make_smem_desc_sw128(sv + kk * (16 * 128), KV_HALF, 1024), idesc_pv,
                              (j > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&pv_full[s]);
                umma_commit(v_empty);
            }
        }
        __syncwarp();
    } else {
        const int qd = warp & 3;                      // TMEM lane quadrant this warp may access
        const int row = qd * 32 + lane;               // query row inside the tile
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
        const uint32_t to = lane_base + TM_O;         // the O accumulator
        const float sl2 = p.scale * 1.4426950408889634f;
        // last visible key of this row: the causal diagonal and / or the end of the (packed) sequence
        const int limit = p.causal ? min(q0 + row + shift, len_k - 1) : len_k - 1;
        const int low = p.window > 0 ? q0 + row + shift - p.window : -1;   // last key below this row's window
        // m is the maximum the exponents are taken against.  It follows the true row maximum lazily: O (in TMEM) and
        // l are rescaled only when the maximum grew by more than 2^8, so P stays below 256 and most tiles skip the
        // read-modify-write of O altogether.
        float m = -INFINITY, l = 0.f;
        uint8_t* prow0 = smem + OFF_P + row * 128;    // this row of the 128 x 64 P tile (buffer 0)
        bool ok = true;
        // every wait is voted on: the tcgen05.ld / st below are warp-collective, so the warp leaves together
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            ok = __all_sync(0xffffffffu, mbar_wait_limit(&s_full[s], (j >> 1) & 1, 650 + s, wait_limit));
            if (!ok) break;
            tc_fence_after();
            const uint32_t ts = lane_base + TM_S + s * BN;
            const int k0 = (j_begin + j) * BN;
            // the tile crosses the causal diagonal of some row, or the lower edge of some row's window
            const bool masked = k0 + BN > len_k ||
                                (p.causal && (k0 + BN - 1 > q0 + shift ||
                                              (p.window > 0 && k0 <= q0 + BM - 1 + shift - p.window)));
            uint32_t r[BN / 32][32];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) tmem_ld_32x32(ts + c * 32, r[c]);
            tmem_ld_wait();
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < BN / 32; ++c)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (masked && (k0 + c * 32 + i > limit || k0 + c * 32 + i <= low)) r[c][i] = 0xff800000u;   // -inf: exp2 gives 0
                    mx = fmaxf(mx, __uint_as_float(r[c][i]));
                }
            const float m_new = fmaxf(m, mx);
            if (j >= 2) {   // this P buffer was last read by the P V product of tile j - 2
                ok = __all_sync(0xffffffffu, mbar_wait_limit(&pv_full[s], ((j >> 1) - 1) & 1, 655 + s, wait_limit));
                if (!ok) break;
            }
            if (j == 0) {
                m = m_new;
            } else {
                const bool need = (m_new - m) * sl2 > 8.f;
                if (__any_sync(0xffffffffu, need)) {
                    // O may only be touched when every earlier P V product has completed
                    ok = __all_sync(0xffffffffu, mbar_wait_limit(&pv_full[(j - 1) & 1], ((j - 1) >> 1) & 1, 660, wait_limit));
                    if (!ok) break;
                    tc_fence_after();
                    const float alpha = need ? ex2((m - m_new) * sl2) : 1.f;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t t[32];
                        tmem_ld_32x32(to + c * 32, t);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
                        tmem_st_32x32(to + c * 32, t);
                    }
                    tmem_st_wait();
                    l *= alpha;
                    if (need) m = m_new;
                }
            }
            const float m_off = (m == -INFINITY) ? 0.f : m * sl2;
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = ex2(fmaf(__uint_as_float(r[c][i]), sl2, -m_off));
                    const float p1 = ex2(fmaf(__uint_as_float(r[c][i + 1]), sl2, -m_off));
                    sum += p0 + p1;
                    packed[i >> 1] = pack_bf16x2(p0, p1);
                }
                // columns c*32 .. +31 = 16-byte chunks c * 4 .. +3 of the row, XOR-swizzled by row
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = (c * 4 + q4) ^ (row & 7);
                    *reinterpret_cast<uint4*>(prow0 + s * P_BYTES + chunk * 16) =
                        make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                }
            }
            l += sum;
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[s]);
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait_limit(&pv_full[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, 670, wait_limit));
        if (ok) {
            const bool valid = q0 + row < len_q;    // tcgen05.ld is warp-collective: only the stores are predicated
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const long long grow = static_cast<long long>(tok_q) + q0 + row;
            __nv_bfloat16* dst = p.o + grow * p.o_ld + h * HD;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t t[32];
                tmem_ld_32x32(to + c * 32, t);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    v.x = pack_bf16x2(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
                    v.y = pack_bf16x2(__uint_as_float(t[i + 2]) * inv, __uint_as_float(t[i + 3]) * inv);
                    v.z = pack_bf16x2(__uint_as_float(t[i + 4]) * inv, __uint_as_float(t[i + 5]) * inv);
                    v.w = pack_bf16x2(__uint_as_float(t[i + 6]) * inv, __uint_as_float(t[i + 7]) * inv);
                    if (valid) *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
                }
            }
            if (p.lse && valid)
                p.lse[(static_cast<long long>(b) * p.Hq + h) * p.S_pad + q0 + row] =
                    l > 0.f ? m * p.scale + __logf(l) : -INFINITY;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace attn
}  // namespace lme

// q [B, S_q, Hq, 128], k / v [B, S_kv, Hkv, 128] bf16 with the 128 values of a head contiguous, heads contiguous
// inside a token, token pitch ld* elements and batches back to back (pitch S * ld); o [B, S_q, Hq, 128] bf16 with
// token pitch ldo; lse fp32 [B, Hq, S_q] or null.  S_q and S_kv are multiples of 128; causal aligns the last query
// with the last key; window > 0 (causal only) keeps the last `window` visible keys of every query.
// Packed sequences: cu_seqlens (int32 [B + 1], device) with q / k / v / o as [total_tokens, H, 128], S_q = S_kv = the
// longest sequence and lse [B, Hq, S_pad], S_pad = S_q rounded up to 128.
// kv_ready != null: K / V chunks of kv_chunk_rows rows (a multiple of 64) become valid while the kernel runs; word
// [b * chunks + c] of kv_ready holds kv_seq once chunk c of batch entry b is complete (see Args).
extern "C" int lme_attention_fwd(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                 long long ldv, void* o, long long ldo, float* lse, int B, int S_q, int S_kv, int Hq,
                                 int Hkv, int causal, int window, float scale, const int* cu_seqlens,
                                 long long total_tokens, const int* kv_ready, int kv_chunk_rows, int kv_seq,
                                 void* stream) {
    using lme::attn::Args;
    using lme::attn::HD;
    using lme::attn::SMEM_BYTES;
    using lme::attn::attn_fwd_kernel;
    constexpr int BM = lme::attn::BM, BN = lme::attn::BN;
    if (B <= 0 || S_q <= 0 || S_kv <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return LME_ERR_SHAPE;
    // packed sequences (cu_seqlens): B sequences, S_q = S_kv = the longest one, any lengths; else multiples of 128
    if (cu_seqlens ? (S_q != S_kv || total_tokens <= 0) : (S_q % BM || S_kv % BM)) return LME_ERR_SHAPE;
    if (causal && S_kv < S_q) return LME_ERR_SHAPE;
    if (window < 0 || (window > 0 && !causal)) return LME_ERR_SHAPE;
    if (kv_ready != nullptr && (cu_seqlens != nullptr || kv_chunk_rows <= 0 || kv_chunk_rows % BN)) return LME_ERR_SHAPE;
    if (B > 65535 || Hq > 65535 || (S_q + BM - 1) / BM > 65535) return LME_ERR_TOO_LARGE;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(o)) & 15)
        return LME_ERR_ALIGN;
    if ((ldq | ldk | ldv | ldo) % 8) return LME_ERR_ALIGN;
    CUtensorMap tq, tk, tv;
    const uint64_t rows_q = cu_seqlens ? static_cast<uint64_t>(total_tokens) : static_cast<uint64_t>(B) * S_q;
    const uint64_t rows_k = cu_seqlens ? static_cast<uint64_t>(total_tokens) : static_cast<uint64_t>(B) * S_kv;
    int rc = lme::make_tmap_bf16_2d(&tq, q, static_cast<uint64_t>(Hq) * HD, rows_q, ldq, 64, BM);
    if (rc) return rc;
    rc = lme::make_tmap_bf16_2d(&tk, k, static_cast<uint64_t>(Hkv) * HD, rows_k, ldk, 64, BN);
    if (rc) return rc;
    rc = lme::make_tmap_bf16_2d(&tv, v, static_cast<uint64_t>(Hkv) * HD, rows_k, ldv, 64, BN);
    if (rc) return rc;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
            return LME_ERR_LAUNCH;
        cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        configured = true;
    }
    Args p;
    p.o = static_cast<__nv_bfloat16*>(o);
    p.lse = lse;
    p.o_ld = ldo;
    p.B = B; p.S_q = S_q; p.S_kv = S_kv; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.window = window;
    p.cu_seqlens = cu_seqlens;
    p.S_pad = (S_q + BM - 1) / BM * BM;
    p.scale = scale;
    p.kv_ready = kv_ready;
    p.kv_chunk_rows = kv_ready ? kv_chunk_rows : 1;
    p.kv_chunks = kv_ready ? (S_kv + kv_chunk_rows - 1) / kv_chunk_rows : 0;
    p.kv_seq = kv_seq;
    dim3 grid(static_cast<unsigned>(Hq) * B, (S_q + BM - 1) / BM, 1);
    attn_fwd_kernel<<<grid, 192, SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
