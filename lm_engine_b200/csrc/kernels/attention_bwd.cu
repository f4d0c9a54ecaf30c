// Flash-attention backward on tcgen05, as two kernels without atomics (head dim 128, bf16, causal or full, GQA):
//
//   attn_dq_kernel   one CTA per 128 query rows of one (batch, head); streams K/V in tiles of 64 rows like the
//                    forward kernel:  S = Q K^T, dP = dO V^T (TMEM), dS = P (dP - delta) scale with
//                    P = exp2(S scale log2e - lse log2e) recomputed from the saved log-sum-exp (no running maximum),
//                    dQ += dS K (K's tile read a second time as an MN-major operand).
//   attn_dkv_kernel  one CTA per 128 key rows of one (batch, kv head); streams the query rows of every query head
//                    of its group in tiles of 64, in the TRANSPOSED orientation so that a thread owns a key row:
//                    S^T = K Q^T, dP^T = V dO^T, P^T and dS^T written as K-major operands,
//                    dV += P^T dO, dK += dS^T Q (Q and dO tiles read a second time as MN-major operands).
// Recomputing S and dP in both kernels costs 7 tile products per (query, key) tile pair instead of 5, and buys
// ownership: every output row has exactly one writer, so there is no atomic accumulation of dQ and the result is
// deterministic.  delta = rowsum(dO * O) comes from the caller.
//
// Warp roles, barriers and bounded waits follow attention.cu (warp 0 TMA, warp 1 MMA issuer, warps 2..9 one row
// and half of the streamed columns per thread); barriers that can run one completion ahead of their waiter are paired by tile parity.
//
// Role of flash-attn's backward kernels used by the reference (lm_engine/modeling_utils/sequence_mixer_blocks/
// softmax_attention/utils.py flash_attention).
namespace lme {
namespace attn_bwd {

using attn::ex2;

constexpr int HD = 128;
constexpr int ROWS = 128;                      // rows owned by a CTA (queries in dq, keys in dkv)
constexpr int TN = 64;                         // streamed tile rows
constexpr int BIG_HALF = ROWS * 128;           // 128 rows x 64 bf16, one swizzled half of the head dim: 16 KB
constexpr int SMALL_HALF = TN * 128;           // 64 rows x 64 bf16: 8 KB
constexpr int BIG = 2 * BIG_HALF, SMALL = 2 * SMALL_HALF;
constexpr int PT = ROWS * TN * 2;              // a 128 x 64 bf16 operand written by the row threads: 16 KB
constexpr float LOG2E = 1.4426950408889634f;

struct DqArgs {
    __nv_bfloat16* dq;
    long long dq_ld;
    const float* lse;        // [B, Hq, S_q] natural log
    const float* delta;      // [B, Hq, S_q]
    int B, S_q, S_kv, Hq, Hkv, causal, window;
    float scale;
    const int* cu_seqlens;   // packed sequences (self-attention): rows cu[b] .. cu[b+1]-1; null = [B, S] batches
    int S_pad;               // row pitch of lse / delta
};

// row r of a 128 x 64 K-major operand tile: 16-byte chunk c (8 columns) lands at chunk c ^ (r & 7)
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int row, int chunk, uint4 v) {
    *reinterpret_cast<uint4*>(tile + row * 128 + ((chunk ^ (row & 7)) << 4)) = v;
}

namespace dq {
// The K/V ring is deeper than the double buffering of S / dP / dS: a stage is held from its load until the dQ
// product of its tile has read K, so two stages would leave the next load no time to arrive.
constexpr int NS = 4;
constexpr int OFF_Q = 0, OFF_DO = BIG, OFF_K = 2 * BIG, OFF_V = OFF_K + NS * SMALL, OFF_DS = OFF_V + NS * SMALL;
constexpr int OFF_BAR = OFF_DS + 2 * PT;
constexpr int SMEM_BYTES = OFF_BAR + 256;
constexpr uint32_t TMEM_COLS = 512;            // S0 S1 | dP0 dP1 (64 each) | dQ (128)
constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DQ = 256;
}  // namespace dq

__global__ void __launch_bounds__(320, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
               const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const DqArgs p) {
    using namespace dq;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* q_full = bars + 0;
    uint64_t* kv_full = bars + 1;    // [NS]
    uint64_t* kv_empty = bars + 5;   // [NS]
    uint64_t* sdp_full = bars + 9;   // [2]
    uint64_t* ds_full = bars + 11;   // [2]
    uint64_t* dq_done = bars + 13;   // [2]
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 16);
    uint32_t* poisoned = tmem_base_smem + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = gridDim.y - 1 - blockIdx.y;        // x = (head, batch), y = query blocks, long ones first
    const int h = blockIdx.x % p.Hq, b = blockIdx.x / p.Hq;
    const int hk = h / (p.Hq / p.Hkv);
    const int q0 = qb * ROWS;
    int tok_q = b * p.S_q, tok_k = b * p.S_kv, len_q = p.S_q, len_k = p.S_kv;
    if (p.cu_seqlens != nullptr) {
        tok_q = tok_k = p.cu_seqlens[b];
        len_q = len_k = p.cu_seqlens[b + 1] - tok_q;
    }
    const int shift = len_k - len_q;
    int n_tiles = (len_k + TN - 1) / TN;
    if (p.causal) n_tiles = min(n_tiles, (q0 + ROWS + shift + TN - 1) / TN);
    if (q0 >= len_q) n_tiles = 0;
    // sliding window: skip the tiles before the first key the first row sees; j below counts from there
    const int j_begin = (p.causal && p.window > 0) ? max(0, (q0 + shift - p.window + 1) / TN) : 0;
    n_tiles -= j_begin;

    if (threadIdx.x == 0) {
        *poisoned = lme_status[0];
        if (smem_u32(smem) & 1023u) {
            report_error(STATUS_BOUNDS, 780);
            *poisoned = 1u;
        }
    }
    __syncthreads();
    if (*poisoned != 0u || n_tiles <= 0) return;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmDO);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_init(q_full, 1);
        for (int s = 0; s < NS; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sdp_full[s], 1);
            mbar_init(&ds_full[s], 8);     // one arrival per row warp
            mbar_init(&dq_done[s], 1);
        }
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
            mbar_expect_tx(q_full, 2 * BIG);
            tma_load_2d(smem + OFF_Q, &tmQ, q_full, h * HD, row_q);
            tma_load_2d(smem + OFF_Q + BIG_HALF, &tmQ, q_full, h * HD + 64, row_q);
            tma_load_2d(smem + OFF_DO, &tmDO, q_full, h * HD, row_q);
            tma_load_2d(smem + OFF_DO + BIG_HALF, &tmDO, q_full, h * HD + 64, row_q);
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % NS;
                if (!mbar_wait(&kv_empty[s], ((j / NS) & 1) ^ 1, 700 + s)) break;
                const int row_k = tok_k + (j_begin + j) * TN;
                uint8_t* ks = smem + OFF_K + s * SMALL;
                uint8_t* vs = smem + OFF_V + s * SMALL;
                mbar_expect_tx(&kv_full[s], 2 * SMALL);
                tma_load_2d(ks, &tmK, &kv_full[s], hk * HD, row_k);
                tma_load_2d(ks + SMALL_HALF, &tmK, &kv_full[s], hk * HD + 64, row_k);
                tma_load_2d(vs, &tmV, &kv_full[s], hk * HD, row_k);
                tma_load_2d(vs + SMALL_HALF, &tmV, &kv_full[s], hk * HD + 64, row_k);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(1, 1, false, false, ROWS, TN);      // 128 x 64, both K-major
            const uint32_t idesc_dq = make_idesc(1, 1, false, true, ROWS, HD);      // 128 x 128, B MN-major
            const uint32_t sq = smem_u32(smem + OFF_Q), sdo = smem_u32(smem + OFF_DO);
            bool ok = mbar_wait(q_full, 0, 710);
            auto issue_sdp = [&](int j) -> bool {
                const int s = j & 1, st = j % NS;
                if (!mbar_wait(&kv_full[st], (j / NS) & 1, 720 + st)) return false;
                tc_fence_after();
                const uint32_t sk = smem_u32(smem + OFF_K + st * SMALL), sv = smem_u32(smem + OFF_V + st * SMALL);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t big = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
                    const uint32_t small = (kk >> 2) * SMALL_HALF + (kk & 3) * 32;
                    umma_bf16(tmem_base + TM_S + s * TN, make_smem_desc_sw128(sq + big, 16, 1024),
                              make_smem_desc_sw128(sk + small, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
                }
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t big = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
                    const uint32_t small = (kk >> 2) * SMALL_HALF + (kk & 3) * 32;
                    umma_bf16(tmem_base + TM_DP + s * TN, make_smem_desc_sw128(sdo + big, 16, 1024),
                              make_smem_desc_sw128(sv + small, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(&sdp_full[s]);
                return true;
            };
            if (ok) ok = issue_sdp(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j & 1;
                if (j + 1 < n_tiles && !issue_sdp(j + 1)) { ok = false; break; }
                if (!mbar_wait(&ds_full[s], (j >> 1) & 1, 730 + s)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sds = smem_u32(smem + OFF_DS + s * PT);
                const uint32_t sk = smem_u32(smem + OFF_K + (j % NS) * SMALL);
#pragma unroll
                for (int kk = 0; kk < TN / 16; ++kk)
                    umma_bf16(tmem_base + TM_DQ, make_smem_desc_sw128(sds + kk * 32, 16, 1024),
                              make_smem_desc_sw128(sk + kk * (16 * 128), SMALL_HALF, 1024), idesc_dq,
                              (j > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&dq_done[s]);
                umma_commit(&kv_empty[j % NS]);
            }
        }
        __syncwarp();
    } else {
        // eight row warps: warps w and w + 4 share TMEM quadrant w & 3 and each take 32 of the 64 streamed columns
        // (no row statistics are formed here, so the two halves of a row never talk to each other)
        const int qd = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row = qd * 32 + lane;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
        const float sl2 = p.scale * LOG2E;
        const int limit = p.causal ? min(q0 + row + shift, len_k - 1) : len_k - 1;
        const int low = p.window > 0 ? q0 + row + shift - p.window : -1;
        const long long stat = (static_cast<long long>(b) * p.Hq + h) * p.S_pad + q0 + row;
        const float lse2 = p.lse[stat] * LOG2E;
        const float delta = p.delta[stat];
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            ok = __all_sync(0xffffffffu, mbar_wait(&sdp_full[s], (j >> 1) & 1, 750 + s));
            if (!ok) break;
            tc_fence_after();
            const int k0 = (j_begin + j) * TN;
            const bool masked = k0 + TN > len_k ||
                                (p.causal && (k0 + TN - 1 > q0 + shift ||
                                              (p.window > 0 && k0 <= q0 + ROWS - 1 + shift - p.window)));
            uint32_t sv[32], dp[32];
            tmem_ld_32x32(lane_base + TM_S + s * TN + half * 32, sv);
            tmem_ld_32x32(lane_base + TM_DP + s * TN + half * 32, dp);
            tmem_ld_wait();
            if (j >= 2) {   // this dS buffer was last read by the dQ product of tile j - 2
                ok = __all_sync(0xffffffffu, mbar_wait(&dq_done[s], ((j >> 1) - 1) & 1, 755 + s));
                if (!ok) break;
            }
            uint8_t* tile = smem + OFF_DS + s * PT;
            {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float d0 = ex2(fmaf(__uint_as_float(sv[i]), sl2, -lse2)) * (__uint_as_float(dp[i]) - delta) * p.scale;
                    float d1 = ex2(fmaf(__uint_as_float(sv[i + 1]), sl2, -lse2)) * (__uint_as_float(dp[i + 1]) - delta) * p.scale;
                    if (masked) {
                        if (k0 + half * 32 + i > limit || k0 + half * 32 + i <= low) d0 = 0.f;
                        if (k0 + half * 32 + i + 1 > limit || k0 + half * 32 + i + 1 <= low) d1 = 0.f;
                    }
                    packed[i >> 1] = pack_bf16x2(d0, d1);
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    store_row_chunk(tile, row, half * 4 + q4,
                                    make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]));
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ds_full[s]);
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&dq_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, 770));
        if (ok) {
            tc_fence_after();
            const bool valid = q0 + row < len_q;    // the loads below are warp-collective: only stores are predicated
            __nv_bfloat16* dst = p.dq + (static_cast<long long>(tok_q) + q0 + row) * p.dq_ld + h * HD;
#pragma unroll 1
            for (int c = 2 * half; c < 2 * half + 2; ++c) {
                uint32_t t[32];
                tmem_ld_32x32(lane_base + TM_DQ + c * 32, t);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    v.x = pack_bf16x2(__uint_as_float(t[i]), __uint_as_float(t[i + 1]));
                    v.y = pack_bf16x2(__uint_as_float(t[i + 2]), __uint_as_float(t[i + 3]));
                    v.z = pack_bf16x2(__uint_as_float(t[i + 4]), __uint_as_float(t[i + 5]));
                    v.w = pack_bf16x2(__uint_as_float(t[i + 6]), __uint_as_float(t[i + 7]));
                    if (valid) *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, dq::TMEM_COLS);
    }
}


// delta[b, h, s] = sum_d dout[tok, h, d] * out[tok, h, d] with tok = b S + s (or cu[b] + s for packed sequences, 0
// past the end of a sequence): one warp per (b, s, h)
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, long long lddo, const __nv_bfloat16* __restrict__ out,
                  long long ldo, float* __restrict__ delta, int B, int S, int S_pad, int H,
                  const int* __restrict__ cu) {
    const long long rowi = blockIdx.x * 8ll + (threadIdx.x >> 5);     // (b * S_pad + s) * H + h
    if (rowi >= static_cast<long long>(B) * S_pad * H) return;
    const int lane = threadIdx.x & 31;
    const int h = static_cast<int>(rowi % H);
    const int sidx = static_cast<int>((rowi / H) % S_pad), b = static_cast<int>(rowi / H / S_pad);
    long long tok = static_cast<long long>(b) * S + sidx;
    int len = S;
    if (cu != nullptr) {
        tok = cu[b] + sidx;
        len = cu[b + 1] - cu[b];
    }
    float v = 0.f;
    if (sidx < len) {
        const uint2 a = *reinterpret_cast<const uint2*>(dout + tok * lddo + h * HD + lane * 4);
        const uint2 c = *reinterpret_cast<const uint2*>(out + tok * ldo + h * HD + lane * 4);
        const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), c0 = unpack_bf16x2(c.x), c1 = unpack_bf16x2(c.y);
        v = warp_sum(a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y);
    }
    if (lane == 0) delta[(static_cast<long long>(b) * H + h) * S_pad + sidx] = v;
}

struct DkvArgs {
    __nv_bfloat16 *dk, *dv;
    long long dk_ld, dv_ld;
    const float* lse;        // [B, Hq, S_q] natural log
    const float* delta;      // [B, Hq, S_q]
    int B, S_q, S_kv, Hq, Hkv, causal, window;
    float scale;
    const int* cu_seqlens;   // packed sequences (self-attention): rows cu[b] .. cu[b+1]-1; null = [B, S] batches
    int S_pad;               // row pitch of lse / delta
};

namespace dkv {
constexpr int NS = 3;       // Q / dO / statistics ring (a stage is held until dV and dK of its tile are done)
constexpr int OFF_K = 0, OFF_V = BIG, OFF_Q = 2 * BIG, OFF_DO = OFF_Q + NS * SMALL, OFF_PT = OFF_DO + NS * SMALL;
constexpr int OFF_DST = OFF_PT + 2 * PT, OFF_STAT = OFF_DST + 2 * PT;     // stats: NS stages x (64 lse + 64 delta)
constexpr int STAT_BYTES = 2 * TN * 4;
constexpr int OFF_BAR = OFF_STAT + NS * STAT_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256;
constexpr uint32_t TMEM_COLS = 512;            // S^T0 S^T1 | dP^T0 dP^T1 (64 each) | dV (128) | dK (128)
constexpr uint32_t TM_S = 0, TM_DP = 128, TM_DV = 256, TM_DK = 384;
}  // namespace dkv

__global__ void __launch_bounds__(320, 1)
attn_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const DkvArgs p) {
    using namespace dkv;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* kv_full = bars + 0;
    uint64_t* qdo_full = bars + 1;   // [NS]
    uint64_t* qdo_empty = bars + 4;  // [NS]
    uint64_t* sdp_full = bars + 7;   // [2]
    uint64_t* pds_full = bars + 9;   // [2]
    uint64_t* acc_done = bars + 11;  // [2]
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(bars + 14);
    uint32_t* poisoned = tmem_base_smem + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb = blockIdx.y;                         // x = (K/V head, batch), y = key blocks, long (early) ones first
    const int hk = blockIdx.x % p.Hkv, b = blockIdx.x / p.Hkv;
    const int G = p.Hq / p.Hkv;
    const int k0 = kb * ROWS;
    int tok_q = b * p.S_q, tok_k = b * p.S_kv, len_q = p.S_q, len_k = p.S_kv;
    if (p.cu_seqlens != nullptr) {
        tok_q = tok_k = p.cu_seqlens[b];
        len_q = len_k = p.cu_seqlens[b + 1] - tok_q;
    }
    const int shift = len_k - len_q;
    const int nq = (len_q + TN - 1) / TN;
    // first query tile with a row that sees key k0: 64 i + 63 + shift >= k0
    const int i_start = p.causal ? max(0, (k0 - shift) / TN) : 0;
    // sliding window: the last query that sees key k0 + 127 is k0 + 127 - shift + window - 1
    const int i_end = (p.causal && p.window > 0) ? min(nq, (k0 + ROWS - 1 - shift + p.window - 1) / TN + 1) : nq;
    const int per_g = i_end - i_start;
    const int n_it = (per_g > 0 && k0 < len_k) ? G * per_g : 0;

    if (threadIdx.x == 0) {
        *poisoned = lme_status[0];
        if (smem_u32(smem) & 1023u) {
            report_error(STATUS_BOUNDS, 880);
            *poisoned = 1u;
        }
    }
    __syncthreads();
    if (*poisoned != 0u) return;
    if (n_it <= 0) {        // no query sees these keys: their gradients are zero
        if (warp >= 2 && warp < 6) {
            const int row = (warp & 3) * 32 + lane;
            const long long grow = static_cast<long long>(tok_k) + k0 + row;
            for (int i = 0; i < HD && k0 + row < len_k; i += 8) {
                *reinterpret_cast<uint4*>(p.dk + grow * p.dk_ld + hk * HD + i) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(p.dv + grow * p.dv_ld + hk * HD + i) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        return;
    }

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmDO);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        mbar_init(kv_full, 1);
        for (int s = 0; s < NS; ++s) {
            mbar_init(&qdo_full[s], 1);
            mbar_init(&qdo_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sdp_full[s], 1);
            mbar_init(&pds_full[s], 8);    // one arrival per row warp
            mbar_init(&acc_done[s], 1);
        }
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
            const int row_k = tok_k + k0;
            mbar_expect_tx(kv_full, 2 * BIG);
            tma_load_2d(smem + OFF_K, &tmK, kv_full, hk * HD, row_k);
            tma_load_2d(smem + OFF_K + BIG_HALF, &tmK, kv_full, hk * HD + 64, row_k);
            tma_load_2d(smem + OFF_V, &tmV, kv_full, hk * HD, row_k);
            tma_load_2d(smem + OFF_V + BIG_HALF, &tmV, kv_full, hk * HD + 64, row_k);
            for (int it = 0; it < n_it; ++it) {
                const int s = it % NS;
                if (!mbar_wait(&qdo_empty[s], ((it / NS) & 1) ^ 1, 800 + s)) break;
                const int h = hk * G + it / per_g, i = i_start + it % per_g;
                const int row_q = tok_q + i * TN;
                uint8_t* qs = smem + OFF_Q + s * SMALL;
                uint8_t* dos = smem + OFF_DO + s * SMALL;
                float* st = reinterpret_cast<float*>(smem + OFF_STAT + s * STAT_BYTES);
                const long long stat = (static_cast<long long>(b) * p.Hq + h) * p.S_pad + i * TN;
                mbar_expect_tx(&qdo_full[s], 2 * SMALL + STAT_BYTES);
                tma_load_2d(qs, &tmQ, &qdo_full[s], h * HD, row_q);
                tma_load_2d(qs + SMALL_HALF, &tmQ, &qdo_full[s], h * HD + 64, row_q);
                tma_load_2d(dos, &tmDO, &qdo_full[s], h * HD, row_q);
                tma_load_2d(dos + SMALL_HALF, &tmDO, &qdo_full[s], h * HD + 64, row_q);
                bulk_g2s(st, p.lse + stat, TN * 4, &qdo_full[s]);
                bulk_g2s(st + TN, p.delta + stat, TN * 4, &qdo_full[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(1, 1, false, false, ROWS, TN);
            const uint32_t idesc_acc = make_idesc(1, 1, false, true, ROWS, HD);
            const uint32_t sk = smem_u32(smem + OFF_K), sv = smem_u32(smem + OFF_V);
            bool ok = mbar_wait(kv_full, 0, 810);
            auto issue_sdp = [&](int it) -> bool {
                const int s = it & 1, st = it % NS;
                if (!mbar_wait(&qdo_full[st], (it / NS) & 1, 820 + st)) return false;
                tc_fence_after();
                const uint32_t sq = smem_u32(smem + OFF_Q + st * SMALL), sdo = smem_u32(smem + OFF_DO + st * SMALL);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t big = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
                    const uint32_t small = (kk >> 2) * SMALL_HALF + (kk & 3) * 32;
                    umma_bf16(tmem_base + TM_S + s * TN, make_smem_desc_sw128(sk + big, 16, 1024),
                              make_smem_desc_sw128(sq + small, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
                }
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint32_t big = (kk >> 2) * BIG_HALF + (kk & 3) * 32;
                    const uint32_t small = (kk >> 2) * SMALL_HALF + (kk & 3) * 32;
                    umma_bf16(tmem_base + TM_DP + s * TN, make_smem_desc_sw128(sv + big, 16, 1024),
                              make_smem_desc_sw128(sdo + small, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(&sdp_full[s]);
                return true;
            };
            if (ok) ok = issue_sdp(0);
            for (int it = 0; it < n_it && ok; ++it) {
                const int s = it & 1;
                if (it + 1 < n_it && !issue_sdp(it + 1)) { ok = false; break; }
                if (!mbar_wait(&pds_full[s], (it >> 1) & 1, 830 + s)) { ok = false; break; }
                tc_fence_after();
                const uint32_t spt = smem_u32(smem + OFF_PT + s * PT), sdst = smem_u32(smem + OFF_DST + s * PT);
                const uint32_t sq = smem_u32(smem + OFF_Q + (it % NS) * SMALL), sdo = smem_u32(smem + OFF_DO + (it % NS) * SMALL);
#pragma unroll
                for (int kk = 0; kk < TN / 16; ++kk)
                    umma_bf16(tmem_base + TM_DV, make_smem_desc_sw128(spt + kk * 32, 16, 1024),
                              make_smem_desc_sw128(sdo + kk * (16 * 128), SMALL_HALF, 1024), idesc_acc,
                              (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < TN / 16; ++kk)
                    umma_bf16(tmem_base + TM_DK, make_smem_desc_sw128(sdst + kk * 32, 16, 1024),
                              make_smem_desc_sw128(sq + kk * (16 * 128), SMALL_HALF, 1024), idesc_acc,
                              (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(&acc_done[s]);
                umma_commit(&qdo_empty[it % NS]);
            }
        }
        __syncwarp();
    } else {
        const int qd = warp & 3;
        const int half = (warp - 2) >> 2;             // which 32 of the 64 streamed query columns this warp takes
        const int row = qd * 32 + lane;               // key row inside the tile
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
        const float sl2 = p.scale * LOG2E;
        const int kr = k0 + row;
        bool ok = true;
        for (int it = 0; it < n_it; ++it) {
            const int s = it & 1;
            const int i = i_start + it % per_g;
            // the statistics of this tile were written by the bulk copies that complete qdo_full
            ok = __all_sync(0xffffffffu, mbar_wait(&qdo_full[it % NS], (it / NS) & 1, 845));
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&sdp_full[s], (it >> 1) & 1, 850 + s));
            if (!ok) break;
            tc_fence_after();
            const bool masked = i * TN + TN > len_q ||
                                (p.causal && (i * TN + shift < k0 + ROWS - 1 ||
                                              (p.window > 0 && i * TN + TN - 1 + shift >= k0 + p.window)));
            uint32_t sv[32], dp[32];
            tmem_ld_32x32(lane_base + TM_S + s * TN + half * 32, sv);
            tmem_ld_32x32(lane_base + TM_DP + s * TN + half * 32, dp);
            tmem_ld_wait();
            if (it >= 2) {   // these operand buffers were last read by the products of iteration it - 2
                ok = __all_sync(0xffffffffu, mbar_wait(&acc_done[s], ((it >> 1) - 1) & 1, 855 + s));
                if (!ok) break;
            }
            const float* st = reinterpret_cast<const float*>(smem + OFF_STAT + (it % NS) * STAT_BYTES);
            uint8_t* pt = smem + OFF_PT + s * PT;
            uint8_t* dst = smem + OFF_DST + s * PT;
            {
                uint32_t pp[16], dd[16];
                // the statistics are the same for every lane: read them as 16-byte broadcasts, four columns at a time
                const float4* lse4 = reinterpret_cast<const float4*>(st + half * 32);
                const float4* del4 = reinterpret_cast<const float4*>(st + TN + half * 32);
#pragma unroll
                for (int e4 = 0; e4 < 8; ++e4) {
                    const float4 l4 = lse4[e4], d4 = del4[e4];
                    const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, ds[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const int e = e4 * 4 + h2 * 2;
                        const int col = half * 32 + e;
                        float p0 = ex2(fmaf(__uint_as_float(sv[e]), sl2, -ls[h2 * 2] * LOG2E));
                        float p1 = ex2(fmaf(__uint_as_float(sv[e + 1]), sl2, -ls[h2 * 2 + 1] * LOG2E));
                        if (masked) {
                            const int qc = i * TN + col;              // query of this column; it sees keys <= qc + shift
                            const int qv = qc + shift;
                            if (qc >= len_q || (p.causal && (kr > qv || (p.window > 0 && kr <= qv - p.window)))) p0 = 0.f;
                            if (qc + 1 >= len_q || (p.causal && (kr > qv + 1 || (p.window > 0 && kr <= qv + 1 - p.window)))) p1 = 0.f;
                        }
                        const float d0 = p0 * (__uint_as_float(dp[e]) - ds[h2 * 2]) * p.scale;
                        const float d1 = p1 * (__uint_as_float(dp[e + 1]) - ds[h2 * 2 + 1]) * p.scale;
                        pp[e >> 1] = pack_bf16x2(p0, p1);
                        dd[e >> 1] = pack_bf16x2(d0, d1);
                    }
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    store_row_chunk(pt, row, half * 4 + q4, make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]));
                    store_row_chunk(dst, row, half * 4 + q4, make_uint4(dd[4 * q4], dd[4 * q4 + 1], dd[4 * q4 + 2], dd[4 * q4 + 3]));
                }
            }
            fence_proxy_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&pds_full[s]);
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&acc_done[(n_it - 1) & 1], ((n_it - 1) >> 1) & 1, 870));
        if (ok) {
            tc_fence_after();
            const bool valid = kr < len_k;
            const long long grow = static_cast<long long>(tok_k) + kr;
            __nv_bfloat16* dvp = p.dv + grow * p.dv_ld + hk * HD;
            __nv_bfloat16* dkp = p.dk + grow * p.dk_ld + hk * HD;
#pragma unroll 1
            for (int c = 4 * half; c < 4 * half + 4; ++c) {      // warps of half 0 store dV, of half 1 dK
                uint32_t t[32];
                tmem_ld_32x32(lane_base + TM_DV + c * 32, t);     // columns 256 .. 511: dV then dK
                tmem_ld_wait();
                __nv_bfloat16* o = (c < 4 ? dvp : dkp) + (c & 3) * 32;
#pragma unroll
                for (int e = 0; e < 32; e += 8) {
                    uint4 v;
                    v.x = pack_bf16x2(__uint_as_float(t[e]), __uint_as_float(t[e + 1]));
                    v.y = pack_bf16x2(__uint_as_float(t[e + 2]), __uint_as_float(t[e + 3]));
                    v.z = pack_bf16x2(__uint_as_float(t[e + 4]), __uint_as_float(t[e + 5]));
                    v.w = pack_bf16x2(__uint_as_float(t[e + 6]), __uint_as_float(t[e + 7]));
                    if (valid) *reinterpret_cast<uint4*>(o + e) = v;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, dkv::TMEM_COLS);
    }
}

}  // namespace attn_bwd
}  // namespace lme

// Gradients of lme_attention_fwd.  q / k / v / dout / out layouts as there (token pitches ld*), lse fp32
// [B, Hq, S_q]; delta is fp32 scratch of the same shape (filled here with rowsum(dout * out));
// dq [B, S_q, Hq, 128], dk / dv [B, S_kv, Hkv, 128] bf16, written whole.
extern "C" int lme_attention_bwd(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                 long long ldv, const void* dout, long long lddo, const void* out, long long ldo,
                                 const float* lse, float* delta, void* dq, long long lddq, void* dk, long long lddk, void* dv,
                                 long long lddv, int B, int S_q, int S_kv, int Hq, int Hkv, int causal, int window,
                                 float scale, const int* cu_seqlens, long long total_tokens, void* stream) {
    using namespace lme::attn_bwd;
    if (B <= 0 || S_q <= 0 || S_kv <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv) return LME_ERR_SHAPE;
    if (cu_seqlens ? (S_q != S_kv || total_tokens <= 0) : (S_q % ROWS || S_kv % ROWS)) return LME_ERR_SHAPE;
    if (causal && S_kv < S_q) return LME_ERR_SHAPE;
    if (window < 0 || (window > 0 && !causal)) return LME_ERR_SHAPE;
    if (B > 65535 || Hq > 65535 || (S_kv + ROWS - 1) / ROWS > 65535) return LME_ERR_TOO_LARGE;
    const uintptr_t ptrs = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                           reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
                           reinterpret_cast<uintptr_t>(dv) | reinterpret_cast<uintptr_t>(lse) | reinterpret_cast<uintptr_t>(delta);
    if (ptrs & 15) return LME_ERR_ALIGN;
    if ((ldq | ldk | ldv | lddo | lddq | lddk | lddv) % 8) return LME_ERR_ALIGN;
    const uint64_t wq = static_cast<uint64_t>(Hq) * HD, wk = static_cast<uint64_t>(Hkv) * HD;
    const uint64_t rq = cu_seqlens ? static_cast<uint64_t>(total_tokens) : static_cast<uint64_t>(B) * S_q;
    const uint64_t rk = cu_seqlens ? static_cast<uint64_t>(total_tokens) : static_cast<uint64_t>(B) * S_kv;
    const int S_pad = (S_q + ROWS - 1) / ROWS * ROWS;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dq::SMEM_BYTES) != cudaSuccess ||
            cudaFuncSetAttribute(attn_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::SMEM_BYTES) != cudaSuccess)
            return LME_ERR_LAUNCH;
        configured = true;
    }
    if ((reinterpret_cast<uintptr_t>(out) & 15) || ldo % 8) return LME_ERR_ALIGN;
    {
        const long long rows = static_cast<long long>(B) * S_pad * Hq;
        attn_delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(dout), lddo, static_cast<const __nv_bfloat16*>(out), ldo, delta, B, S_q,
            S_pad, Hq, cu_seqlens);
        if (cudaGetLastError() != cudaSuccess) return LME_ERR_LAUNCH;
    }
    int rc;
    {   // dQ: Q and dO in 128-row boxes, K and V in 64-row boxes
        CUtensorMap tq, tdo, tk, tv;
        if ((rc = lme::make_tmap_bf16_2d(&tq, q, wq, rq, ldq, 64, ROWS))) return rc;
        if ((rc = lme::make_tmap_bf16_2d(&tdo, dout, wq, rq, lddo, 64, ROWS))) return rc;
        if ((rc = lme::make_tmap_bf16_2d(&tk, k, wk, rk, ldk, 64, TN))) return rc;
        if ((rc = lme::make_tmap_bf16_2d(&tv, v, wk, rk, ldv, 64, TN))) return rc;
        DqArgs a;
        a.dq = static_cast<__nv_bfloat16*>(dq); a.dq_ld = lddq; a.lse = lse; a.delta = delta;
        a.B = B; a.S_q = S_q; a.S_kv = S_kv; a.Hq = Hq; a.Hkv = Hkv; a.causal = causal; a.window = window; a.scale = scale;
        a.cu_seqlens = cu_seqlens; a.S_pad = S_pad;
        attn_dq_kernel<<<dim3(static_cast<unsigned>(Hq) * B, (S_q + ROWS - 1) / ROWS, 1), 320, dq::SMEM_BYTES, st>>>(tq, tdo, tk, tv, a);
        if (cudaGetLastError() != cudaSuccess) return LME_ERR_LAUNCH;
    }
    {   // dK, dV: K and V in 128-row boxes, Q and dO in 64-row boxes
        CUtensorMap tq, tdo, tk, tv;
        if ((rc = lme::make_tmap_bf16_2d(&tq, q, wq, rq, ldq, 64, TN))) return rc;
        if ((rc = lme::make_tmap_bf16_2d(&tdo, dout, wq, rq, lddo, 64, TN))) return rc;
        if ((rc = lme::make_tmap_bf16_2d(&tk, k, wk, rk, ldk, 64, ROWS))) return rc;
        if ((rc = lme::make_tmap_bf16_2d(&tv, v, wk, rk, ldv, 64, ROWS))) return rc;
        DkvArgs a;
        a.dk = static_cast<__nv_bfloat16*>(dk); a.dv = static_cast<__nv_bfloat16*>(dv); a.dk_ld = lddk; a.dv_ld = lddv;
        a.lse = lse; a.delta = delta;
        a.B = B; a.S_q = S_q; a.S_kv = S_kv; a.Hq = Hq; a.Hkv = Hkv; a.causal = causal; a.window = window; a.scale = scale;
        a.cu_seqlens = cu_seqlens; a.S_pad = S_pad;
        attn_dkv_kernel<<<dim3(static_cast<unsigned>(Hkv) * B, (S_kv + ROWS - 1) / ROWS, 1), 320, dkv::SMEM_BYTES, st>>>(tq, tdo, tk, tv, a);
        if (cudaGetLastError() != cudaSuccess) return LME_ERR_LAUNCH;
    }
    return LME_OK;
}
