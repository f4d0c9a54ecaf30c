// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = sum_k A(m,k) * B(n,k)   (fp32 accumulate)
//
// One persistent CTA per SM, warp-specialised:
//   warp 0        TMA producer   (cp.async.bulk.tensor, per-CTA loads, 128-byte swizzle, STAGES-deep ring)
//   warp 1        MMA issuer     (one elected thread issues tcgen05.mma 128 x BN x 16; accumulators live in TMEM,
//                                 two accumulator buffers so the epilogue of tile i overlaps the main loop of i+1)
//   warps 2..5    epilogue       (tcgen05.ld -> registers -> fused epilogue -> global)
//
// Either operand may be K-major (row-major [rows, K]) or MN-major (stored [K, rows], i.e. the "transposed"
// operand of dgrad / wgrad) - the tensor core reads both straight from shared memory, so no transposes are ever
// materialised:   forward  y = x W^T : A = x (K-major), B = W (K-major)
//                 dgrad    dx = dy W : A = dy (K-major), B = W (MN-major)
//                 wgrad    dW = dy^T x: A = dy (MN-major), B = x (MN-major)
//
// Fused epilogues (runtime flags): + bias[n], + residual[m,n], C += acc (gradient accumulation, bf16 or fp32 C),
// and SwiGLU on interleaved columns: out[m, j] = acc[m, 2j+1] * silu(acc[m, 2j]) with optional store of the
// pre-activation (the layout the MLP's fused gate/up projection uses).
#include "common.cuh"
#include "../lme_api.h"

#include "gather.cuh"

#include <mutex>
#include <stdlib.h>
#include <stdio.h>

namespace lme {

static constexpr int BM = 128;
static constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
static constexpr int UMMA_K = 16;

struct GemmArgs {
    int M, N, K;
    void* C;
    long long ldc;
    const __nv_bfloat16* bias;
    const __nv_bfloat16* residual;
    long long ldr;
    __nv_bfloat16* preact;
    long long ldp;
    int flags;
    int tiles_m, tiles_n, group_m;
    // 8-bit operands (kind::f8f6f4): element formats (0 = e4m3, 1 = e5m2) and the de-quantisation scales, read on the
    // device so that no host synchronisation sits between the quantiser and the GEMM
    int a_fmt, b_fmt;
    const float* scale_a;
    const float* scale_b;
    // Grouped (mixture-of-experts) forms.  Rows are laid out so that every 128-row tile belongs to one group:
    //   tile_group != null : tile_group[m-tile] = group of that tile (< 0: tile unused, skipped); the B operand of
    //                        group e starts group_b_stride rows (K-major B) / contraction rows (MN-major B) further
    //   num_groups_w > 0   : one product per group with its own contraction range (weight gradients):
    //                        k in [group_k0[e], group_k0[e] + 64 * group_kb[e]), output e at C + e * group_c_stride
    const int* tile_group;
    int group_b_stride;
    int num_groups_w;
    const int* group_k0;
    const int* group_kb;
    long long group_c_stride;
    // Batched form (BATCHED kernels): `batch` independent products; the operands are addressed through 3-D tensor
    // maps whose outermost coordinate is the batch index, output b starts batch_c_stride elements further.
    int batch;
    long long batch_c_stride;
};

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILES_BYTES = STAGES * STAGE_BYTES;
    // barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then the TMEM base address
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
    static constexpr int TOTAL = TILES_BYTES + BAR_BYTES + 1024;  // + slack for 1024-byte alignment
};

__device__ __forceinline__ void tile_coords(int tile, const GemmArgs& p, int& mb, int& nb) {
    int per_group = p.group_m * p.tiles_n;
    int g = tile / per_group;
    int first_m = g * p.group_m;
    int gsz = min(p.tiles_m - first_m, p.group_m);
    int in = tile - g * per_group;
    mb = first_m + in % gsz;
    nb = in / gsz;
}

// Fused epilogue for 32 consecutive accumulator columns of one output row (held by one thread).
__device__ __forceinline__ void epilogue_store(const uint32_t (&r)[32], int row, int col0, const GemmArgs& p,
                                               bool out_f32, bool accumulate, bool swiglu, long long c_off = 0) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        const int ncols = min(32, p.N - col0);  // N % 8 == 0 is enforced on the host
        if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                if (i < ncols) {
                    uint4 b = *reinterpret_cast<const uint4*>(p.bias + col0 + i);
                    float2 f;
                    f = unpack_bf16x2(b.x); v[i] += f.x; v[i + 1] += f.y;
                    f = unpack_bf16x2(b.y); v[i + 2] += f.x; v[i + 3] += f.y;
                    f = unpack_bf16x2(b.z); v[i + 4] += f.x; v[i + 5] += f.y;
                    f = unpack_bf16x2(b.w); v[i + 6] += f.x; v[i + 7] += f.y;
                }
            }
        }
        if (swiglu) {
            if (p.preact != nullptr) {
                __nv_bfloat16* pp = p.preact + static_cast<long long>(row) * p.ldp + col0;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    if (i < ncols) {
                        uint4 o;
                        o.x = pack_bf16x2(v[i], v[i + 1]); o.y = pack_bf16x2(v[i + 2], v[i + 3]);
                        o.z = pack_bf16x2(v[i + 4], v[i + 5]); o.w = pack_bf16x2(v[i + 6], v[i + 7]);
                        *reinterpret_cast<uint4*>(pp + i) = o;
                    }
                }
            }
            // interleaved (gate, up) pairs -> 16 outputs per 32 accumulator columns
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) +
                                 static_cast<long long>(row) * p.ldc + (col0 >> 1);
#pragma unroll
            for (int i = 0; i < 32; i += 16) {
                if (i < ncols) {
                    float o8[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // silu(g) = g * sigmoid(g) with the approximate exp and reciprocal units: far fewer
                        // instructions (and less power) than an IEEE division per element, error well below
                        // bf16 resolution
                        const float g = v[i + 2 * j], u = v[i + 2 * j + 1];
                        o8[j] = __fdividef(u * g, 1.0f + __expf(-g));
                    }
                    uint4 o;
                    o.x = pack_bf16x2(o8[0], o8[1]); o.y = pack_bf16x2(o8[2], o8[3]);
                    o.z = pack_bf16x2(o8[4], o8[5]); o.w = pack_bf16x2(o8[6], o8[7]);
                    *reinterpret_cast<uint4*>(out + (i >> 1)) = o;
                }
            }
            return;
        }
        if (p.residual != nullptr) {
            const __nv_bfloat16* rp = p.residual + static_cast<long long>(row) * p.ldr + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                if (i < ncols) {
                    uint4 b = *reinterpret_cast<const uint4*>(rp + i);
                    float2 f;
                    f = unpack_bf16x2(b.x); v[i] += f.x; v[i + 1] += f.y;
                    f = unpack_bf16x2(b.y); v[i + 2] += f.x; v[i + 3] += f.y;
                    f = unpack_bf16x2(b.z); v[i + 4] += f.x; v[i + 5] += f.y;
                    f = unpack_bf16x2(b.w); v[i + 6] += f.x; v[i + 7] += f.y;
                }
            }
        }
        if (out_f32) {
            float* out = reinterpret_cast<float*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                if (i < ncols) {
                    float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    if (accumulate) {
                        float4 old = *reinterpret_cast<const float4*>(out + i);
                        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                    }
                    *reinterpret_cast<float4*>(out + i) = o;
                }
            }
        } else {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off +
                                 static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                if (i < ncols) {
                    if (accumulate) {
                        uint4 b = *reinterpret_cast<const uint4*>(out + i);
                        float2 f;
                        f = unpack_bf16x2(b.x); v[i] += f.x; v[i + 1] += f.y;
                        f = unpack_bf16x2(b.y); v[i + 2] += f.x; v[i + 3] += f.y;
                        f = unpack_bf16x2(b.z); v[i + 4] += f.x; v[i + 5] += f.y;
                        f = unpack_bf16x2(b.w); v[i + 6] += f.x; v[i + 7] += f.y;
                    }
                    uint4 o;
                    o.x = pack_bf16x2(v[i], v[i + 1]); o.y = pack_bf16x2(v[i + 2], v[i + 3]);
                    o.z = pack_bf16x2(v[i + 4], v[i + 5]); o.w = pack_bf16x2(v[i + 6], v[i + 7]);
                    *reinterpret_cast<uint4*>(out + i) = o;
                }
            }
        }
}

// F8: operands are 1-byte e4m3 / e5m2, K-major; a 128-byte swizzle row then holds 128 elements of K and one MMA
// consumes 32 of them, so the byte geometry of the pipeline is identical to the bf16 one.
// GATHER: the first g.n_copy CTAs of the grid pull an operand's rows from the peers (gather.cuh) while the others
// multiply; the TMA producer waits for the segments under each operand tile.
// RS: the epilogue reduce-scatters the product over the ranks (RsArgs in gather.cuh).
template <int BN, int STAGES, bool A_MN, bool B_MN, bool F8 = false, bool GATHER = false, bool RS = false,
          bool BATCHED = false>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmArgs p, const __grid_constant__ GatherArgs g,
                 const __grid_constant__ CUtensorMap tmLocal, const __grid_constant__ RsArgs rs) {
    static_assert(!(GATHER && RS), "one fused collective per kernel");
    static_assert(!F8 || (!A_MN && !B_MN), "8-bit operands are K-major");
    static_assert(!GATHER || !A_MN, "the gathered operand is K-major");
    static_assert(!BATCHED || (!F8 && !GATHER && !RS), "the batched form is the plain bf16 product");
    constexpr int BKE = F8 ? 2 * BK : BK;  // K elements per pipeline stage
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::TILES_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tempty_bar + 2);

    const int n_copy = GATHER ? g.n_copy : 0;
    if (GATHER && static_cast<int>(blockIdx.x) < n_copy) {
        gather_copy_cta(g, smem, blockIdx.x);
        return;
    }
    const int cta = blockIdx.x - n_copy, n_cta = gridDim.x - n_copy;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_per_group = p.tiles_m * p.tiles_n;
    const int num_tiles = tiles_per_group * (BATCHED ? p.batch : (p.num_groups_w > 0 ? p.num_groups_w : 1));
    const int num_kb = (p.K + BKE - 1) / BKE;
    constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                   : (2 * BN <= 256) ? 256 : 512;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tfull_bar[a], 1);
            mbar_init(&tempty_bar[a], 4);  // one arrival per epilogue warp
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
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cta; tile < num_tiles && ok; tile += n_cta) {
                int mb, nb;
                const int grp = (BATCHED || p.num_groups_w > 0) ? tile / tiles_per_group : 0;
                tile_coords(tile - grp * tiles_per_group, p, mb, nb);
                if (GATHER) mb = (mb + g.rotate_tiles) % p.tiles_m;
                if (RS) mb = (mb + rs.rotate) % p.tiles_m;
                int b_off = 0;
                if (p.tile_group != nullptr) {
                    const int e = __ldg(&p.tile_group[mb]);
                    if (e < 0) continue;   // unused tile of the padded row layout (all three roles skip it)
                    b_off = e * p.group_b_stride;
                }
                const int tile_kb = p.num_groups_w > 0 ? __ldg(&p.group_kb[grp]) : num_kb;
                const int k_base = p.num_groups_w > 0 ? __ldg(&p.group_k0[grp]) : 0;
                const int m0 = mb * BM, n0 = nb * BN;
                // rows that are entirely this rank's own contribution are read where they already are
                bool own_rows = false;
                if (GATHER) {
                    own_rows = g.which == 0 && m0 >= g.local_row0 && m0 + BM <= g.local_row0 + g.local_rows;
                    if (!own_rows) {
                        const bool arrived = g.which == 0 ? gather_wait_rows(g, m0, BM, p.M)
                                                          : gather_wait_rows(g, n0, BN, p.N);
                        if (!arrived) { ok = false; break; }
                    }
                }
                for (int kb = 0; kb < tile_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1, 100 + s)) { ok = false; break; }
                    uint8_t* sa = smem + s * L::STAGE_BYTES;
                    uint8_t* sb = sa + L::A_BYTES;
                    if (p.flags & LME_GEMM_PROBE_NO_LOAD) {   // timing probe: the stage is declared full as it is
                        mbar_arrive(&full_bar[s]);
                        continue;
                    }
                    mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
                    const int k0 = k_base + kb * BKE;
                    if (BATCHED) {
                        // 3-D maps: (inner, rows, batch); rows beyond a batch's extent read zeros
                        if (A_MN) {
#pragma unroll
                            for (int c = 0; c < BM / 64; ++c)
                                tma_load_3d(sa + c * (BK * 128), &tmA, &full_bar[s], m0 + c * 64, k0, grp);
                        } else {
                            tma_load_3d(sa, &tmA, &full_bar[s], k0, m0, grp);
                        }
                        if (B_MN) {
#pragma unroll
                            for (int c = 0; c < BN / 64; ++c)
                                tma_load_3d(sb + c * (BK * 128), &tmB, &full_bar[s], n0 + c * 64, k0, grp);
                        } else {
                            tma_load_3d(sb, &tmB, &full_bar[s], k0, n0, grp);
                        }
                        continue;
                    }
                    if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c)
                            tma_load_2d(sa + c * (BK * 128), &tmA, &full_bar[s], m0 + c * 64, k0);
                    } else if (GATHER && own_rows) {
                        tma_load_2d(sa, &tmLocal, &full_bar[s], k0, m0 - g.local_row0);
                    } else {
                        tma_load_2d(sa, &tmA, &full_bar[s], k0, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tma_load_2d(sb + c * (BK * 128), &tmB, &full_bar[s], n0 + c * 64,
                                        (p.num_groups_w > 0 ? k0 : kb * BKE) + b_off);
                    } else {
                        tma_load_2d(sb, &tmB, &full_bar[s], k0, n0 + b_off);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = F8 ? make_idesc(p.a_fmt, p.b_fmt, false, false, BM, BN)
                                      : make_idesc(1, 1, A_MN, B_MN, BM, BN);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = cta; tile < num_tiles && ok; tile += n_cta) {
                const int grp = p.num_groups_w > 0 ? tile / tiles_per_group : 0;
                if (p.tile_group != nullptr) {
                    int mb, nb;
                    tile_coords(tile - grp * tiles_per_group, p, mb, nb);
                    if (__ldg(&p.tile_group[mb]) < 0) continue;
                }
                const int tile_kb = p.num_groups_w > 0 ? __ldg(&p.group_kb[grp]) : num_kb;
                const int acc = tcount & 1;
                const uint32_t aph = (tcount >> 1) & 1;
                ++tcount;
                if (!mbar_wait(&tempty_bar[acc], aph ^ 1, 200 + acc)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                if (tile_kb == 0) {   // a group without rows: nothing to multiply, the epilogue writes zeros
                    mbar_arrive(&tfull_bar[acc]);
                    continue;
                }
                for (int kb = 0; kb < tile_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&full_bar[s], ph, 300 + s)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                    const uint32_t sb = sa + L::A_BYTES;
                    if (p.flags & LME_GEMM_PROBE_NO_MMA) {    // timing probe: the stage is released unread
                        mbar_arrive(&empty_bar[s]);
                        continue;
                    }
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // K-major: step 16 elements (32 bytes) inside the swizzled 128-byte row.
                        // MN-major: step 16 rows of 128 bytes.
                        const uint64_t da = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
                        if (F8) umma_f8(tmem_d, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                        else umma_bf16(tmem_d, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty_bar[s]);  // frees the smem slot once these MMAs have read it
                }
                if (ok) umma_commit(&tfull_bar[acc]);  // accumulator complete
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;  // TMEM lane quadrant this warp may access
        uint32_t tcount = 0;
        bool ok = true;
        const bool out_f32 = p.flags & LME_GEMM_OUT_F32;
        const bool accumulate = p.flags & LME_GEMM_ACCUMULATE;
        const bool swiglu = p.flags & LME_GEMM_SWIGLU;
        float dequant = 1.0f;
        if (F8) dequant = __ldg(p.scale_a) * __ldg(p.scale_b);
        for (int tile = cta; tile < num_tiles && ok; tile += n_cta) {
            int mb, nb;
            const int grp = (BATCHED || p.num_groups_w > 0) ? tile / tiles_per_group : 0;
            tile_coords(tile - grp * tiles_per_group, p, mb, nb);
            if (GATHER) mb = (mb + g.rotate_tiles) % p.tiles_m;
            if (RS) mb = (mb + rs.rotate) % p.tiles_m;
            if (p.tile_group != nullptr && __ldg(&p.tile_group[mb]) < 0) continue;
            const bool empty_group = p.num_groups_w > 0 && __ldg(&p.group_kb[grp]) == 0;
            const long long c_off = BATCHED ? grp * p.batch_c_stride
                                            : (p.num_groups_w > 0 ? grp * p.group_c_stride : 0);
            const int acc = tcount & 1;
            const uint32_t aph = (tcount >> 1) & 1;
            ++tcount;
            if (!mbar_wait(&tfull_bar[acc], aph, 400 + acc)) { ok = false; break; }
            tc_fence_after();
            const int row = mb * BM + q * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
            if (RS) {
                const int owner = mb / rs.tiles_per_rank;
                const int lmt = mb - owner * rs.tiles_per_rank;
                const int lrow = lmt * BM + q * 32 + lane;   // row inside the owner's block
                if (owner != rs.rank) {
                    // A peer's rows: bf16 partial product into the owner's slab, then the arrival flag.  The
                    // accumulator arrives one row per lane; it is turned through shared memory (16-byte chunks
                    // XOR-swizzled by row) so that a store instruction covers two full 256-byte row pieces: NVLink
                    // then carries full-size write packets instead of 32 scattered 16-byte ones.
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(rs.slab[owner]) +
                                         (static_cast<long long>(rs.rank) * rs.rows_per_rank + lmt * BM + q * 32) *
                                             rs.slab_ld;
                    uint8_t* wst = smem + L::TILES_BYTES + 1024 + q * 8192;
#pragma unroll 1
                    for (int half = 0; half < BN / 128; ++half) {
#pragma unroll 1
                        for (int c4 = 0; c4 < 4; ++c4) {
                            uint32_t r[32];
                            tmem_ld_32x32(taddr + (half * 4 + c4) * 32, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 o;
                                o.x = pack_bf16x2(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]));
                                o.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                                o.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                                o.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                                const int phys = (c4 * 4 + i) ^ (lane & 15);
                                *reinterpret_cast<uint4*>(wst + lane * 256 + phys * 16) = o;
                            }
                        }
                        __syncwarp();
                        const int k = lane & 15;
                        const int col = nb * BN + half * 128 + k * 8;
#pragma unroll 4
                        for (int rr = 0; rr < 16; ++rr) {
                            const int rw = rr * 2 + (lane >> 4);
                            const uint4 v = *reinterpret_cast<const uint4*>(wst + rw * 256 + ((k ^ (rw & 15)) * 16));
                            if (col < p.N) *reinterpret_cast<uint4*>(dst + rw * rs.slab_ld + col) = v;
                        }
                        __syncwarp();
                    }
                    tc_fence_before();
                    __threadfence_system();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&tempty_bar[acc]);
                        st_release_sys(&rs.flags[owner][((rs.rank * rs.tiles_per_rank + lmt) * p.tiles_n + nb) * 4 + q],
                                       rs.seq);
                    }
                    continue;
                }
                // own rows: the peers' partial products must have arrived
                int arrived = 1;
                if (lane == 0) {
                    for (int src = 0; src < rs.world && arrived; ++src)
                        if (src != rs.rank)
                            arrived = wait_flag_sys(
                                &rs.flags[rs.rank][((src * rs.tiles_per_rank + lmt) * p.tiles_n + nb) * 4 + q], rs.seq,
                                840 + src);
                }
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (!arrived) { ok = false; break; }
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + c * 32, r);
                    tmem_ld_wait();
                    const int col0 = nb * BN + c * 32;
                    if (col0 < p.N) {
                        for (int src = 0; src < rs.world; ++src) {
                            if (src == rs.rank) continue;
                            const __nv_bfloat16* part = reinterpret_cast<const __nv_bfloat16*>(rs.slab[rs.rank]) +
                                (static_cast<long long>(src) * rs.rows_per_rank + lrow) * rs.slab_ld + col0;
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                if (col0 + i < p.N) {
                                    uint4 b = *reinterpret_cast<const uint4*>(part + i);
                                    float2 f;
                                    f = unpack_bf16x2(b.x);
                                    r[i] = __float_as_uint(__uint_as_float(r[i]) + f.x);
                                    r[i + 1] = __float_as_uint(__uint_as_float(r[i + 1]) + f.y);
                                    f = unpack_bf16x2(b.y);
                                    r[i + 2] = __float_as_uint(__uint_as_float(r[i + 2]) + f.x);
                                    r[i + 3] = __float_as_uint(__uint_as_float(r[i + 3]) + f.y);
                                    f = unpack_bf16x2(b.z);
                                    r[i + 4] = __float_as_uint(__uint_as_float(r[i + 4]) + f.x);
                                    r[i + 5] = __float_as_uint(__uint_as_float(r[i + 5]) + f.y);
                                    f = unpack_bf16x2(b.w);
                                    r[i + 6] = __float_as_uint(__uint_as_float(r[i + 6]) + f.x);
                                    r[i + 7] = __float_as_uint(__uint_as_float(r[i + 7]) + f.y);
                                }
                            }
                        }
                        epilogue_store(r, lrow, col0, p, out_f32, accumulate, swiglu);
                    }
                    __syncwarp();
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty_bar[acc]);
                continue;
            }
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_ld_wait();
                if (F8) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * dequant);
                }
                if (empty_group) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                }
                const int col0 = nb * BN + c * 32;
                if (row_ok && col0 < p.N) epilogue_store(r, row, col0, p, out_f32, accumulate, swiglu, c_off);
                __syncwarp();
            }
            // accumulator buffer may be overwritten by the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        }
    }

    // ---------------------------------------------------------------- tear-down
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ----------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows, row pitch `ld` elements,
// box = [box_inner x box_outer], 128-byte swizzle (box_inner must be 64).
int make_tmap_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                 uint32_t box_outer, int elem_bytes);

int make_tmap_bf16_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
                      uint32_t box_inner, uint32_t box_outer) {
    return make_tmap_2d(m, ptr, inner, outer, ld, box_inner, box_outer, 2);
}

// elem_bytes 2 = bf16, 1 = 8-bit; the box's inner extent must span 128 bytes (the swizzle row)
int make_tmap_2d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner,
                 uint32_t box_outer, int elem_bytes) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return LME_ERR_DRIVER;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    // The encode call is a driver entry point and needs a current context.  A thread that has made no runtime
    // call yet (an autograd worker whose first op is this GEMM) has none bound: bind the primary context once.
    thread_local bool context_bound = false;
    if (!context_bound) {
        cudaFree(nullptr);
        context_bound = true;
    }
    CUresult r = enc(m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                     const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "lme: cuTensorMapEncodeTiled failed (CUresult %d): ptr=%p inner=%llu outer=%llu ld=%llu box=%ux%u\n",
                static_cast<int>(r), ptr, static_cast<unsigned long long>(inner),
                static_cast<unsigned long long>(outer), static_cast<unsigned long long>(ld), box_inner, box_outer);
        return LME_ERR_TMAP;
    }
    return LME_OK;
}

// 3-D bf16 tensor map (inner, rows, batch): row pitch `ld` and batch pitch `batch_ld` in elements, box
// [box_inner x box_rows x 1], 128-byte swizzle.
int make_tmap_bf16_3d(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t rows, uint64_t batch, uint64_t ld,
                      uint64_t batch_ld, uint32_t box_inner, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return LME_ERR_DRIVER;
    cuuint64_t dims[3] = {inner, rows, batch};
    cuuint64_t strides[2] = {ld * 2, batch_ld * 2};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    thread_local bool context_bound = false;
    if (!context_bound) {
        cudaFree(nullptr);
        context_bound = true;
    }
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "lme: cuTensorMapEncodeTiled (3-D) failed (CUresult %d): ptr=%p inner=%llu rows=%llu batch=%llu "
                "ld=%llu batch_ld=%llu\n", static_cast<int>(r), ptr, static_cast<unsigned long long>(inner),
                static_cast<unsigned long long>(rows), static_cast<unsigned long long>(batch),
                static_cast<unsigned long long>(ld), static_cast<unsigned long long>(batch_ld));
        return LME_ERR_TMAP;
    }
    return LME_OK;
}

static int g_num_sms = 0;
static int num_sms() {
    if (g_num_sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return g_num_sms;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool F8 = false, bool GATHER = false, bool RS = false,
          bool BATCHED = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs& p, int max_ctas,
                       cudaStream_t stream, const GatherArgs* gather = nullptr,
                       const CUtensorMap* tlocal = nullptr, const RsArgs* scatter = nullptr) {
    using L = SmemLayout<BN, STAGES>;
    static_assert(!GATHER || L::TILES_BYTES >= GATHER_SLOTS * GATHER_SEG_BYTES, "copy CTAs reuse the tile ring");
    auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, F8, GATHER, RS, BATCHED>;
    // RS: + 4 x 8 KB behind the barriers, where the epilogue warps turn their tiles for coalesced peer stores
    constexpr int SMEM = L::TOTAL + (RS ? 1024 + 4 * 8192 : 0);
    static_assert(SMEM <= 232448, "dynamic shared memory of one CTA");
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
            return LME_ERR_LAUNCH;
        configured = true;
    }
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.N + BN - 1) / BN;
    p.group_m = 8;
    int tiles = p.tiles_m * p.tiles_n * (BATCHED ? p.batch : 1);
    GatherArgs g;
    RsArgs rs;
    rs.enabled = 0;
    if (RS) rs = *scatter;
    if (GATHER) {
        g = *gather;
        // every CTA of this grid must be resident at once (the multiplying CTAs wait for the copy CTAs)
        int gemm_ctas = max_ctas - g.n_copy;
        if (gemm_ctas < 1) return LME_ERR_SHAPE;
        if (tiles < gemm_ctas) gemm_ctas = tiles;
        kern<<<gemm_ctas + g.n_copy, 192, SMEM, stream>>>(ta, tb, p, g, *tlocal, rs);
        return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
    }
    g.enabled = 0;
    g.n_copy = 0;
    int grid = tiles < max_ctas ? tiles : max_ctas;
    kern<<<grid, 192, SMEM, stream>>>(ta, tb, p, g, ta, rs);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

}  // namespace lme

using namespace lme;

extern "C" int lme_gemm_bf16(const void* A, int a_mn_major, long long lda, const void* B, int b_mn_major,
                             long long ldb, void* C, long long ldc, int M, int N, int K, int flags,
                             const void* bias, const void* residual, long long ldr, void* preact, long long ldp,
                             int max_ctas, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return LME_OK;
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldc % 4)) return LME_ERR_SHAPE;
    if ((flags & LME_GEMM_SWIGLU) && (N % 16)) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return LME_ERR_ALIGN;
    const int BN = (N <= 128) ? 128 : 256;
    CUtensorMap ta, tb;
    int rc;
    // K-major operand [rows, K]: inner = K, box 64 x rows_per_tile.  MN-major operand [K, rows]: inner = rows,
    // box 64 x BK (one 64-wide chunk per copy).
    rc = a_mn_major ? make_tmap_bf16_2d(&ta, A, M, K, lda, 64, BK) : make_tmap_bf16_2d(&ta, A, K, M, lda, 64, BM);
    if (rc) return rc;
    rc = b_mn_major ? make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, BK) : make_tmap_bf16_2d(&tb, B, K, N, ldb, 64, BN);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldp = ldp;
    p.flags = flags;
    p.a_fmt = p.b_fmt = 0;
    p.scale_a = p.scale_b = nullptr;
    if (max_ctas <= 0) max_ctas = num_sms();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LME_DISPATCH(BN_, ST_)                                                          \
    do {                                                                                \
        if (a_mn_major && b_mn_major) return launch_gemm<BN_, ST_, true, true>(ta, tb, p, max_ctas, st);   \
        if (a_mn_major) return launch_gemm<BN_, ST_, true, false>(ta, tb, p, max_ctas, st);                \
        if (b_mn_major) return launch_gemm<BN_, ST_, false, true>(ta, tb, p, max_ctas, st);                \
        return launch_gemm<BN_, ST_, false, false>(ta, tb, p, max_ctas, st);                               \
    } while (0)
    if (BN == 128) LME_DISPATCH(128, 6);
    LME_DISPATCH(256, 4);
#undef LME_DISPATCH
}

// Batched GEMM: C[b] (+)= A[b] x B[b]^T for b < batch.  Operand b of A / B starts a_batch_ld / b_batch_ld elements
// after operand b - 1 (row pitches lda / ldb), either layout per operand as in lme_gemm_bf16; C[b] at
// C + b * c_batch_ld.  Flags: LME_GEMM_OUT_F32, LME_GEMM_ACCUMULATE.
extern "C" int lme_gemm_bf16_batched(const void* A, int a_mn_major, long long lda, long long a_batch_ld,
                                     const void* B, int b_mn_major, long long ldb, long long b_batch_ld, void* C,
                                     long long ldc, long long c_batch_ld, int batch, int M, int N, int K, int flags,
                                     int max_ctas, void* stream) {
    if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return LME_OK;
    if ((N % 8) || (lda % 8) || (ldb % 8) || (a_batch_ld % 8) || (b_batch_ld % 8) || (ldc % 4) || (c_batch_ld % 4))
        return LME_ERR_SHAPE;
    if (flags & ~(LME_GEMM_OUT_F32 | LME_GEMM_ACCUMULATE)) return LME_ERR_SHAPE;
    // the innermost extent of a tensor map is a multiple of 16 bytes
    if ((a_mn_major ? M : K) % 8 || (b_mn_major ? N : K) % 8) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return LME_ERR_ALIGN;
    const int BN = (N <= 128) ? 128 : 256;
    CUtensorMap ta, tb;
    int rc;
    rc = a_mn_major ? make_tmap_bf16_3d(&ta, A, M, K, batch, lda, a_batch_ld, 64, BK)
                    : make_tmap_bf16_3d(&ta, A, K, M, batch, lda, a_batch_ld, 64, BM);
    if (rc) return rc;
    rc = b_mn_major ? make_tmap_bf16_3d(&tb, B, N, K, batch, ldb, b_batch_ld, 64, BK)
                    : make_tmap_bf16_3d(&tb, B, K, N, batch, ldb, b_batch_ld, 64, BN);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.flags = flags;
    p.batch = batch;
    p.batch_c_stride = c_batch_ld;
    if (max_ctas <= 0) max_ctas = num_sms();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LME_DISPATCH(BN_, ST_)                                                                              \
    do {                                                                                                    \
        if (a_mn_major && b_mn_major)                                                                       \
            return launch_gemm<BN_, ST_, true, true, false, false, false, true>(ta, tb, p, max_ctas, st);   \
        if (a_mn_major)                                                                                     \
            return launch_gemm<BN_, ST_, true, false, false, false, false, true>(ta, tb, p, max_ctas, st);  \
        if (b_mn_major)                                                                                     \
            return launch_gemm<BN_, ST_, false, true, false, false, false, true>(ta, tb, p, max_ctas, st);  \
        return launch_gemm<BN_, ST_, false, false, false, false, false, true>(ta, tb, p, max_ctas, st);     \
    } while (0)
    if (BN == 128) LME_DISPATCH(128, 6);
    LME_DISPATCH(256, 4);
#undef LME_DISPATCH
}

// Grouped GEMM for mixture-of-experts layers.  Rows of A / C are in the padded per-group layout: every 128-row tile
// belongs to one group, tile_group[m-tile] names it (< 0: unused tile, skipped).  Group e multiplies with
//   B[e] = rows [e * N, (e + 1) * N) of a K-major [G * N, K] matrix (forward:  y = x W_e^T), or
//   B[e] = rows [e * K, (e + 1) * K) of an MN-major [G * K, N] matrix (input gradient: dx = dy W_e).
extern "C" int lme_gemm_bf16_grouped(const void* A, long long lda, const void* B, int b_mn_major, long long ldb,
                                     void* C, long long ldc, int M, int N, int K, int num_groups, int flags,
                                     void* preact, long long ldp, const int* tile_group, int max_ctas,
                                     void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return LME_OK;
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldc % 4) || (M % BM) || tile_group == nullptr) return LME_ERR_SHAPE;
    if (b_mn_major && (K % BK)) return LME_ERR_SHAPE;   // a partial K block would read the next group's rows
    if ((flags & LME_GEMM_SWIGLU) && (N % 16)) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return LME_ERR_ALIGN;
    const int BN = (N <= 128) ? 128 : 256;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16_2d(&ta, A, K, M, lda, 64, BM);
    if (rc) return rc;
    rc = b_mn_major ? make_tmap_bf16_2d(&tb, B, N, static_cast<uint64_t>(num_groups) * K, ldb, 64, BK)
                    : make_tmap_bf16_2d(&tb, B, K, static_cast<uint64_t>(num_groups) * N, ldb, 64, BN);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldp = ldp;
    p.flags = flags;
    p.tile_group = tile_group;
    p.group_b_stride = b_mn_major ? K : N;
    if (max_ctas <= 0) max_ctas = num_sms();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (b_mn_major) {
        if (BN == 128) return launch_gemm<128, 6, false, true>(ta, tb, p, max_ctas, st);
        return launch_gemm<256, 4, false, true>(ta, tb, p, max_ctas, st);
    }
    if (BN == 128) return launch_gemm<128, 6, false, false>(ta, tb, p, max_ctas, st);
    return launch_gemm<256, 4, false, false>(ta, tb, p, max_ctas, st);
}

// Weight gradients of a grouped layer: dW[e] [M, N] (+)= dY[rows of e]^T * X[rows of e] for every group e, rows in
// the padded layout (group e owns rows [group_k0[e], group_k0[e] + 64 * group_kb[e]), padding rows of X are zero).
// dY is [rows, M], X is [rows, N]; dW is [G, M, N] with row pitch ldw.  A group without rows yields zeros.
extern "C" int lme_gemm_bf16_grouped_wgrad(const void* dY, long long lddy, const void* X, long long ldx, void* dW,
                                           long long ldw, int M, int N, int rows, int num_groups,
                                           const int* group_k0, const int* group_kb, int flags, int max_ctas,
                                           void* stream) {
    if (M <= 0 || N <= 0 || rows <= 0 || num_groups <= 0) return LME_OK;
    if ((N % 8) || (M % 8) || (lddy % 8) || (ldx % 8) || (ldw % 4)) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(dY) | reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(dW)) & 15)
        return LME_ERR_ALIGN;
    const int BN = (N <= 128) ? 128 : 256;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16_2d(&ta, dY, M, rows, lddy, 64, BK);
    if (rc) return rc;
    rc = make_tmap_bf16_2d(&tb, X, N, rows, ldx, 64, BK);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = rows;
    p.C = dW; p.ldc = ldw;
    p.flags = flags & (LME_GEMM_OUT_F32 | LME_GEMM_ACCUMULATE);
    p.num_groups_w = num_groups;
    p.group_k0 = group_k0;
    p.group_kb = group_kb;
    p.group_c_stride = static_cast<long long>(M) * ldw;
    if (max_ctas <= 0) max_ctas = num_sms();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (BN == 128) return launch_gemm<128, 6, true, true>(ta, tb, p, max_ctas, st);
    return launch_gemm<256, 4, true, true>(ta, tb, p, max_ctas, st);
}

// C[M,N] = (A[M,K] * B[N,K]^T) * scale_a * scale_b with 1-byte e4m3 / e5m2 operands, both K-major.
extern "C" int lme_gemm_fp8(const void* A, int a_fmt, long long lda, const void* B, int b_fmt, long long ldb,
                            const float* scale_a, const float* scale_b, void* C, long long ldc, int M, int N, int K,
                            int flags, const void* bias, const void* residual, long long ldr, void* preact,
                            long long ldp, int max_ctas, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return LME_OK;
    if ((N % 8) || (lda % 16) || (ldb % 16) || (ldc % 4) || (K % 16)) return LME_ERR_SHAPE;
    if ((flags & LME_GEMM_SWIGLU) && (N % 16)) return LME_ERR_SHAPE;
    if ((a_fmt | b_fmt) & ~1) return LME_ERR_SHAPE;
    if (scale_a == nullptr || scale_b == nullptr) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return LME_ERR_ALIGN;
    const int BN = (N <= 128) ? 128 : 256;
    CUtensorMap ta, tb;
    int rc = make_tmap_2d(&ta, A, K, M, lda, 128, BM, 1);
    if (rc) return rc;
    rc = make_tmap_2d(&tb, B, K, N, ldb, 128, BN, 1);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldp = ldp;
    p.flags = flags;
    p.a_fmt = a_fmt; p.b_fmt = b_fmt;
    p.scale_a = scale_a; p.scale_b = scale_b;
    if (max_ctas <= 0) max_ctas = num_sms();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (BN == 128) return launch_gemm<128, 6, false, false, true>(ta, tb, p, max_ctas, st);
    return launch_gemm<256, 4, false, false, true>(ta, tb, p, max_ctas, st);
}

// C[M, N] = A_gathered[M, K] * B[N, K]^T where the rows of A are the concatenation, in rank order, of `world`
// contributions of shard_bytes each.  This rank's contribution is `local_src`; the peers' arrive through the
// symmetric staging buffers `stage[r]` (already offset to the slot of this call) and are written to `A_gathered`
// (local) by copy CTAs of the same grid while the other CTAs multiply the rows that are there.
//   pads[r]   : int32 signal pad (16 words) of rank r in symmetric memory
//   ready     : local int32, world * ceil(shard_bytes / 32 KB) words, never reset (compared against seq)
//   counters  : local uint32[2], zero before the first call
//   seq       : 1, 2, 3, ... per call on this set of buffers (the same on every rank)
extern "C" int lme_gemm_bf16_allgather_a(void* A_gathered, long long lda, const void* B, int b_mn_major,
                                         long long ldb, void* C,
                                         long long ldc, int M, int N, int K, int flags, const void* bias,
                                         const void* residual, long long ldr, void* preact, long long ldp,
                                         const void* local_src, void* const* stage, int* const* pads, int* ready,
                                         unsigned int* counters, long long shard_bytes, int rank, int world,
                                         int seq, int n_copy, int seg_shift, int max_ctas, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return LME_OK;
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldc % 4)) return LME_ERR_SHAPE;
    if (world < 2 || world > GATHER_MAX_RANKS || rank < 0 || rank >= world || seq < 1 || n_copy < 0)
        return LME_ERR_SHAPE;
    if (lda != K || shard_bytes * world != static_cast<long long>(M) * K * 2 || (shard_bytes % 16))
        return LME_ERR_SHAPE;   // the gathered operand is dense and splits evenly
    if ((reinterpret_cast<uintptr_t>(A_gathered) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
         reinterpret_cast<uintptr_t>(local_src)) & 15)
        return LME_ERR_ALIGN;
    const int BN = (N <= 128) ? 128 : 256;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16_2d(&ta, A_gathered, K, M, lda, 64, BM);
    if (rc) return rc;
    rc = b_mn_major ? make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, BK) : make_tmap_bf16_2d(&tb, B, K, N, ldb, 64, BN);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldp = ldp;
    p.flags = flags;
    p.a_fmt = p.b_fmt = 0;
    p.scale_a = p.scale_b = nullptr;
    GatherArgs g;
    g.enabled = 1;
    g.rank = rank; g.world = world; g.n_copy = n_copy; g.seq = seq;
    g.shard_bytes = shard_bytes;
    g.operand_off = 0;
    g.row_bytes = lda * 2;
    g.rows_per_tile = BM;
    g.which = 0;
    const int tiles_m = (M + BM - 1) / BM;
    g.rotate_tiles = static_cast<int>((static_cast<long long>(rank) * tiles_m) / world);
    g.local_src = static_cast<const uint8_t*>(local_src);
    for (int r = 0; r < GATHER_MAX_RANKS; ++r) {
        g.stage[r] = r < world ? static_cast<uint8_t*>(stage[r]) : nullptr;
        g.pad[r] = r < world ? pads[r] : nullptr;
    }
    g.dst = static_cast<uint8_t*>(A_gathered);
    g.ready = ready;
    g.counters = counters;
    g.local_rows = M / world;
    g.local_row0 = rank * g.local_rows;
    g.seg_shift = n_copy > 0 ? GATHER_SEG_SHIFT : seg_shift;
    if (g.seg_shift < 12 || g.seg_shift > 30) return LME_ERR_SHAPE;
    g.flag_every = 4;
    if (const char* e = getenv("LME_GATHER_FLAG_EVERY")) g.flag_every = atoi(e) > 0 ? atoi(e) : 4;
    CUtensorMap tl;
    rc = make_tmap_bf16_2d(&tl, local_src, K, g.local_rows, lda, 64, BM);
    if (rc) return rc;
    if (max_ctas <= 0) max_ctas = num_sms();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (b_mn_major) {
        if (BN == 128) return launch_gemm<128, 6, false, true, false, true>(ta, tb, p, max_ctas, st, &g, &tl);
        return launch_gemm<256, 4, false, true, false, true>(ta, tb, p, max_ctas, st, &g, &tl);
    }
    if (BN == 128) return launch_gemm<128, 6, false, false, false, true>(ta, tb, p, max_ctas, st, &g, &tl);
    return launch_gemm<256, 4, false, false, false, true>(ta, tb, p, max_ctas, st, &g, &tl);
}

// out[M / world, N] = sum over ranks of (A[M, K] * B[N, K]^T)[rows of this rank] (+ bias) (+ residual): the
// reduce-scatter runs inside the GEMM epilogue (RsArgs in kernels/gather.cuh).  slabs[r] / flags[r]: receive slab
// (already offset to the slot of this call) and arrival flags of rank r in symmetric memory.  M / world must be a
// multiple of 128.  seq = 1, 2, ... per call on one set of buffers.
extern "C" int lme_gemm_bf16_reduce_scatter(const void* A, long long lda, const void* B, int b_mn_major,
                                            long long ldb, void* out,
                                            long long ldo, int M, int N, int K, const void* bias,
                                            const void* residual, long long ldr, void* const* slabs,
                                            int* const* flags, int rank, int world, int seq, int max_ctas,
                                            void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return LME_OK;
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldo % 4)) return LME_ERR_SHAPE;
    if (world < 2 || world > GATHER_MAX_RANKS || rank < 0 || rank >= world || seq < 1) return LME_ERR_SHAPE;
    if (M % (world * BM)) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
        return LME_ERR_ALIGN;
    const int BN = (N <= 128) ? 128 : 256;
    CUtensorMap ta, tb;
    int rc = make_tmap_bf16_2d(&ta, A, K, M, lda, 64, BM);
    if (rc) return rc;
    rc = b_mn_major ? make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, BK) : make_tmap_bf16_2d(&tb, B, K, N, ldb, 64, BN);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = K;
    p.C = out; p.ldc = ldo;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
    p.preact = nullptr; p.ldp = 0;
    p.flags = 0;
    p.a_fmt = p.b_fmt = 0;
    p.scale_a = p.scale_b = nullptr;
    RsArgs rs;
    rs.enabled = 1;
    rs.rank = rank; rs.world = world; rs.seq = seq;
    rs.rows_per_rank = M / world;
    rs.tiles_per_rank = rs.rows_per_rank / BM;
    rs.rotate = ((rank + 1) % world) * rs.tiles_per_rank;
    rs.slab_ld = N;
    for (int r = 0; r < GATHER_MAX_RANKS; ++r) {
        rs.slab[r] = r < world ? static_cast<uint8_t*>(slabs[r]) : nullptr;
        rs.flags[r] = r < world ? flags[r] : nullptr;
    }
    if (max_ctas <= 0) max_ctas = num_sms();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (b_mn_major) {
        if (BN == 128)
            return launch_gemm<128, 6, false, true, false, false, true>(ta, tb, p, max_ctas, st, nullptr, nullptr,
                                                                         &rs);
        return launch_gemm<256, 4, false, true, false, false, true>(ta, tb, p, max_ctas, st, nullptr, nullptr, &rs);
    }
    if (BN == 128)
        return launch_gemm<128, 6, false, false, false, false, true>(ta, tb, p, max_ctas, st, nullptr, nullptr, &rs);
    return launch_gemm<256, 4, false, false, false, false, true>(ta, tb, p, max_ctas, st, nullptr, nullptr, &rs);
}

// Stream-side pieces of the copy-engine-fed all-gather (n_copy == 0 above): announce the staging slot to the peers;
// hold a stream until a peer has announced; write a readiness word from the stream itself (a stream memory
// operation, no kernel, so it progresses while persistent GEMM CTAs occupy every SM).
extern "C" int lme_gather_signal(int* const* pads, int rank, int world, int seq, void* stream) {
    GatherArgs g;
    g.rank = rank; g.world = world; g.seq = seq;
    for (int r = 0; r < GATHER_MAX_RANKS; ++r) g.pad[r] = r < world ? pads[r] : nullptr;
    gather_signal_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(g);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
extern "C" int lme_gather_wait_peer(const int* pad, int src, int seq, void* stream) {
    gather_wait_peer_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(pad + PAD_SIG + src, seq, 860 + src);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
typedef CUresult (*WriteValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
extern "C" int lme_stream_write_words(int* words, int count, int value, void* stream) {
    static WriteValue32Fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<WriteValue32Fn>(f);
    });
    if (!fn) return LME_ERR_DRIVER;
    for (int i = 0; i < count; ++i)
        if (fn(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(words + i), static_cast<cuuint32_t>(value),
               0) != CUDA_SUCCESS)
            return LME_ERR_LAUNCH;
    return LME_OK;
}

// Holds `stream` until *word >= value (a stream memory operation: no kernel, so it needs no SM while other kernels
// of this GPU wait for what the stream delivers afterwards).  Not bounded by itself: the kernels that consume the
// delivery have bounded waits and report a missing peer through the status block.
typedef CUresult (*WaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
extern "C" int lme_stream_wait_word(const int* word, int value, void* stream) {
    static WaitValue32Fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<WaitValue32Fn>(f);
    });
    if (!fn) return LME_ERR_DRIVER;
    return fn(static_cast<CUstream>(stream), reinterpret_cast<CUdeviceptr>(word), static_cast<cuuint32_t>(value),
              CU_STREAM_WAIT_VALUE_GEQ) == CUDA_SUCCESS
               ? LME_OK
               : LME_ERR_LAUNCH;
}

extern "C" int lme_read_status(unsigned int* out8, int clear) {
    unsigned int h[8];
    if (cudaMemcpyFromSymbol(h, lme_status, sizeof(h)) != cudaSuccess) return LME_ERR_LAUNCH;
    for (int i = 0; i < 8; ++i) out8[i] = h[i];
    if (clear) {
        unsigned int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (cudaMemcpyToSymbol(lme_status, z, sizeof(z)) != cudaSuccess) return LME_ERR_LAUNCH;
    }
    return LME_OK;
}
