// bf16 GEMM, two-SM variant: a thread-block cluster of two CTAs computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128 of the 256 B rows per k-block
// (per-CTA TMA loads, no multicast), so every operand byte is fetched from L2 and read from shared memory once per
// CTA pair instead of once per CTA - less data movement per FLOP than the one-SM kernel in gemm.cu, which is what
// matters once the part is running against its power limit.
//
// Roles per CTA are those of gemm.cu (warp 0 TMA, warp 1 MMA, warps 2..5 epilogue); only the leader CTA (cluster rank
// 0) issues MMAs.  Cross-CTA signalling:
//   full[s]    (leader)   both producers' TMA transactions land on the leader's barrier
//   empty[s]   (each CTA) the leader's tcgen05.commit arrives on its own and on the peer's barrier
//   tfull[a]   (each CTA) same, when an accumulator is complete
//   tempty[a]  (leader)   8 arrivals: the 4 epilogue warps of both CTAs
#include "common.cuh"
#include "../lme_api.h"

namespace lme {

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (an address in this CTA's shared memory) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2cta() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_2cta(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// one arrival on the barrier at shared::cluster address `cluster_addr` once all MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_2cta(uint32_t cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
                 : "memory");
}
// the same arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, from one instruction (a
// signal multicast, no data moves): the two separate commits it replaces each held up the issuing thread
__device__ __forceinline__ void umma_commit_2cta_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(mask)
        : "memory");
}
// per-CTA tile load whose completion is counted on a barrier that may live in the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

static constexpr int BN2 = 256;        // N of the pair's tile
static constexpr int HALF_N = 128;     // B rows staged by each CTA

template <int STAGES>
struct SmemLayout2 {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = HALF_N * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TILES_BYTES = STAGES * STAGE_BYTES;
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
    static constexpr int TOTAL = TILES_BYTES + BAR_BYTES + 1024;
};

template <int STAGES, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const GemmArgs p) {
    using L = SmemLayout2<STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::TILES_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tfull_bar = empty_bar + STAGES;
    uint64_t* tempty_bar = tfull_bar + 2;
    uint32_t* tmem_base_smem = reinterpret_cast<uint32_t*>(tempty_bar + 2);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int num_tiles = p.tiles_m * p.tiles_n;  // tiles_m counts 256-row super tiles
    const int num_kb = (p.K + BK - 1) / BK;
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;
    constexpr uint32_t TMEM_COLS = 512;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tfull_bar[a], 1);
            mbar_init(&tempty_bar[a], 8);  // 4 epilogue warps of each CTA of the pair
        }
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_2cta(tmem_base_smem, TMEM_COLS);
        tmem_relinquish_2cta();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_base_smem;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
                if (p.flags & 768) break;   // timing probes without stage hand-over: nothing to produce
                int mb2, nb;
                tile_coords(tile, p, mb2, nb);
                const int m0 = (mb2 * 2 + static_cast<int>(rank)) * BM;
                const int n0 = nb * BN2 + static_cast<int>(rank) * HALF_N;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&empty_bar[s], ph ^ 1, 1100 + s)) { ok = false; break; }
                    uint8_t* sa = smem + s * L::STAGE_BYTES;
                    uint8_t* sb = sa + L::A_BYTES;
                    if (p.flags & LME_GEMM_PROBE_NO_LOAD) {   // timing probe: the stage is declared full as it is
                        if (leader) mbar_arrive(&full_bar[s]);
                        continue;
                    }
                    if (leader) mbar_expect_tx(&full_bar[s], 2 * L::STAGE_BYTES);
                    const uint32_t bar = map_to_cta(&full_bar[s], 0);
                    const int k0 = kb * BK;
                    if (A_MN) {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c)
                            tma_load_2d_pair(sa + c * (BK * 128), &tmA, bar, m0 + c * 64, k0);
                    } else {
                        tma_load_2d_pair(sa, &tmA, bar, k0, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int c = 0; c < HALF_N / 64; ++c)
                            tma_load_2d_pair(sb + c * (BK * 128), &tmB, bar, n0 + c * 64, k0);
                    } else {
                        tma_load_2d_pair(sb, &tmB, bar, k0, n0);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader && lane == 0) {
            constexpr uint32_t idesc = make_idesc(1, 1, A_MN, B_MN, 2 * BM, BN2);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++tcount) {
                const int acc = tcount & 1;
                const uint32_t aph = (tcount >> 1) & 1;
                if (!mbar_wait(&tempty_bar[acc], aph ^ 1, 1200 + acc)) { ok = false; break; }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN2;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    // probes 256 / 512: MMAs on whatever the stage holds, no full-barrier wait (512: but with the
                    // per-stage commit, which then signals barriers nobody waits for)
                    if (!(p.flags & 768) && !mbar_wait(&full_bar[s], ph, 1300 + s)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
                    const uint32_t sb = sa + L::A_BYTES;
                    if (p.flags & LME_GEMM_PROBE_NO_MMA) {    // timing probe: the stage is released unread
                        mbar_arrive(&empty_bar[s]);
                        mbar_arrive_remote(map_to_cta(&empty_bar[s], 1));
                        continue;
                    }
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t da = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
                        const uint64_t db = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), BK * 128, 1024)
                                                 : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
                        umma_bf16_2cta(tmem_d, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    // the stage is free in both CTAs once these MMAs have read it
                    if (!(p.flags & 256)) umma_commit_2cta_pair(&empty_bar[s]);
                }
                if (ok) umma_commit_2cta_pair(&tfull_bar[acc]);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const int q = warp & 3;
        uint32_t tcount = 0;
        bool ok = true;
        const bool out_f32 = p.flags & LME_GEMM_OUT_F32;
        const bool accumulate = p.flags & LME_GEMM_ACCUMULATE;
        const bool swiglu = p.flags & LME_GEMM_SWIGLU;
        for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, ++tcount) {
            int mb2, nb;
            tile_coords(tile, p, mb2, nb);
            const int acc = tcount & 1;
            const uint32_t aph = (tcount >> 1) & 1;
            if (!mbar_wait(&tfull_bar[acc], aph, 1400 + acc)) { ok = false; break; }
            tc_fence_after();
            const int row = (mb2 * 2 + static_cast<int>(rank)) * BM + q * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN2;
#pragma unroll 1
            for (int c = 0; c < BN2 / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_ld_wait();
                const int col0 = nb * BN2 + c * 32;
                if (row_ok && col0 < p.N) epilogue_store(r, row, col0, p, out_f32, accumulate, swiglu);
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(&tempty_bar[acc]);
                else mbar_arrive_remote(map_to_cta(&tempty_bar[acc], 0));
            }
        }
    }

    // ---------------------------------------------------------------- tear-down
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves while the other may still touch its shared memory or barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_2cta(tmem_base, TMEM_COLS);
    }
}

static int g_last_max_clusters = -1;   // what the occupancy query said for the last 2-CTA launch (diagnostics)

template <int STAGES, bool A_MN, bool B_MN>
static int launch_gemm_2cta(const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs& p, int max_ctas,
                            cudaStream_t stream) {
    using L = SmemLayout2<STAGES>;
    auto kern = gemm_bf16_2cta_kernel<STAGES, A_MN, B_MN>;
    static int max_clusters = -1;
    if (max_clusters < 0) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
            return LME_ERR_LAUNCH;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 74, 1, 1);
        cfg.blockDim = dim3(192, 1, 1);
        cfg.dynamicSmemBytes = L::TOTAL;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = num_sms() / 2;
        }
        max_clusters = n;
    }
    g_last_max_clusters = max_clusters;
    p.tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
    p.tiles_n = (p.N + BN2 - 1) / BN2;
    static const int group_m_env = [] { const char* e = getenv("LME_GEMM2_GROUP_M"); return e ? atoi(e) : 0; }();
    p.group_m = group_m_env > 0 ? group_m_env : 4;
    int tiles = p.tiles_m * p.tiles_n;
    int clusters = tiles < max_clusters ? tiles : max_clusters;
    if (max_ctas > 0 && clusters > max_ctas / 2) clusters = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
    kern<<<2 * clusters, 192, L::TOTAL, stream>>>(ta, tb, p);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

}  // namespace lme

using namespace lme;

// Number of CTA pairs that can be resident at once according to cudaOccupancyMaxActiveClusters (-1 before the first
// 2-CTA launch): the persistent grid of lme_gemm_bf16_2cta is that many pairs.
extern "C" int lme_gemm_2cta_resident_pairs() { return lme::g_last_max_clusters; }

// Same contract as lme_gemm_bf16; N <= 128 is forwarded to the one-SM kernel.
extern "C" int lme_gemm_bf16_2cta(const void* A, int a_mn_major, long long lda, const void* B, int b_mn_major,
                                  long long ldb, void* C, long long ldc, int M, int N, int K, int flags,
                                  const void* bias, const void* residual, long long ldr, void* preact,
                                  long long ldp, int max_ctas, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0) return LME_OK;
    if (N <= 128)
        return lme_gemm_bf16(A, a_mn_major, lda, B, b_mn_major, ldb, C, ldc, M, N, K, flags, bias, residual, ldr,
                             preact, ldp, max_ctas, stream);
    if ((N % 8) || (lda % 8) || (ldb % 8) || (ldc % 4)) return LME_ERR_SHAPE;
    if ((flags & LME_GEMM_SWIGLU) && (N % 16)) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
        return LME_ERR_ALIGN;
    CUtensorMap ta, tb;
    int rc;
    rc = a_mn_major ? make_tmap_bf16_2d(&ta, A, M, K, lda, 64, BK) : make_tmap_bf16_2d(&ta, A, K, M, lda, 64, BM);
    if (rc) return rc;
    rc = b_mn_major ? make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, BK)
                    : make_tmap_bf16_2d(&tb, B, K, N, ldb, 64, HALF_N);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.K = K;
    p.C = C; p.ldc = ldc;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
    p.preact = static_cast<__nv_bfloat16*>(preact); p.ldp = ldp;
    p.flags = flags;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    static const int stages_env = [] { const char* e = getenv("LME_GEMM2_STAGES"); return e ? atoi(e) : 6; }();
    if (a_mn_major && b_mn_major) return launch_gemm_2cta<6, true, true>(ta, tb, p, max_ctas, st);
    if (a_mn_major) return launch_gemm_2cta<6, true, false>(ta, tb, p, max_ctas, st);
    if (b_mn_major) return launch_gemm_2cta<6, false, true>(ta, tb, p, max_ctas, st);
    if (stages_env == 7) return launch_gemm_2cta<7, false, false>(ta, tb, p, max_ctas, st);
    if (stages_env == 4) return launch_gemm_2cta<4, false, false>(ta, tb, p, max_ctas, st);
    return launch_gemm_2cta<6, false, false>(ta, tb, p, max_ctas, st);
}
