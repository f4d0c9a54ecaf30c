// All-gather fused into a GEMM: a few "copy CTAs" of the GEMM's own grid pull the peers' contributions over NVLink
// into the local operand buffer while the remaining CTAs already multiply the tiles that have arrived.
//
// Data path of a copy CTA (one elected thread): bulk asynchronous copies global -> shared (peer or local memory,
// no multicast) tracked by mbarriers, then shared -> global into the local gathered buffer, 32 KB segments in a
// 6-slot ring, so ~160 KB per copy CTA are in flight with no register traffic at all.  Every segment that is
// complete in local memory publishes `ready[segment] = seq`; the GEMM's TMA producer warp waits for the segments
// under an operand tile before loading it.
//
// Cross-rank protocol (all words live in symmetric memory, zero at start, `seq` grows by one per call):
//   own contribution  -> stage[rank][seq & 1] (symmetric), once the peers' done[] words show they finished reading
//                        the previous use of that slot (call seq - 2)
//   sig[rank] := seq     written into every peer's pad after the stage is complete: "rank's data for seq is there"
//   pull from peer p     after our pad shows sig[p] >= seq
//   done[rank] := seq    written into every peer's pad after all pulls of this call are complete
// Every wait is bounded (LME_WAIT_LIMIT_NS); on expiry the status word is set and the CTA returns, which makes the
// GEMM CTAs run into their own bounded waits and return as well.
#pragma once

namespace lme {

static constexpr int GATHER_MAX_RANKS = 8;
static constexpr int GATHER_SEG_SHIFT = 15;                 // 32 KB segments
static constexpr int GATHER_SEG_BYTES = 1 << GATHER_SEG_SHIFT;
static constexpr int GATHER_SLOTS = 6;
static constexpr int GATHER_LAG = 4;                        // loads in flight ahead of the store stage

// layout of the int32 signal pad of one rank (symmetric memory)
static constexpr int PAD_SIG = 0;                           // [8]  sig[src]: src published its stage for call n
static constexpr int PAD_DONE = 8;                          // [8]  done[src]: src finished pulling our call n
static constexpr int PAD_WORDS = 16;

struct GatherArgs {
    int enabled;
    int rank, world, n_copy, seq;
    long long shard_bytes;      // contribution of one rank (multiple of 16; the last segment may be partial)
    long long operand_off;      // byte offset of the gathered GEMM operand inside the gathered buffer
    long long row_bytes;        // pitch of that operand
    int rows_per_tile;          // BM (A gathered) or BN (B gathered)
    int which;                  // 0: rows of A arrive, 1: rows of B arrive
    int rotate_tiles;           // m-tile rotation so that locally available rows are multiplied first
    const uint8_t* local_src;   // this rank's contribution, any local memory
    uint8_t* stage[GATHER_MAX_RANKS];   // slot-selected staging buffer of every rank ([rank] = ours)
    uint8_t* dst;               // local gathered buffer, world * shard_bytes
    int* ready;                 // local, one word per segment of dst
    int* pad[GATHER_MAX_RANKS];         // signal pad of every rank ([rank] = ours)
    unsigned int* counters;     // local, 2 words: copy-CTA arrival counters (monotonic)
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// bounded wait for *p >= want (system scope: the word is written by another GPU)
__device__ __forceinline__ bool wait_flag_sys(const int* p, int want, unsigned int id) {
    if (ld_acquire_sys(p) >= want) return true;
    uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (ld_acquire_sys(p) < want) {
        __nanosleep(64);
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > LME_WAIT_LIMIT_NS) {
            report_error(STATUS_FLAG_TIMEOUT, id);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ bool wait_flag_gpu(const int* p, int want, unsigned int id) {
    if (ld_acquire_gpu(p) >= want) return true;
    uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (ld_acquire_gpu(p) < want) {
        __nanosleep(32);
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > LME_WAIT_LIMIT_NS) {
            report_error(STATUS_FLAG_TIMEOUT, id);
            return false;
        }
    }
    return true;
}

// bulk async copies (TMA engine, untiled, no multicast); addresses and sizes are multiples of 16 bytes
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// One contiguous range [0, bytes) of `src` copied to dst_a (and dst_b when not null), split into segments; this CTA
// takes the segments cta, cta + n_cta, ...  `ready` (may be null) gets `seq` per finished segment of dst_a.
// Runs on ONE thread.  Returns false on a timed-out wait.
__device__ bool gather_copy_range(uint8_t* smem, uint64_t* bars, uint32_t& ring_it, const uint8_t* src,
                                  uint8_t* dst_a, uint8_t* dst_b, long long bytes, int* ready, int seq, int cta,
                                  int n_cta) {
    const int nseg = static_cast<int>((bytes + GATHER_SEG_BYTES - 1) >> GATHER_SEG_SHIFT);
    const int mine = (nseg - cta + n_cta - 1) / n_cta;      // segments cta, cta + n_cta, ...
    if (mine <= 0) return true;
    auto seg_of = [&](int j) { return cta + j * n_cta; };
    auto seg_bytes = [&](int s) {
        long long left = bytes - (static_cast<long long>(s) << GATHER_SEG_SHIFT);
        return static_cast<uint32_t>(left < GATHER_SEG_BYTES ? left : GATHER_SEG_BYTES);
    };
    const uint32_t base_it = ring_it;
    int flagged = 0;   // number of own segments whose ready flag has been published
    for (int k = 0; k < mine + GATHER_LAG; ++k) {
        if (k < mine) {
            const uint32_t it = base_it + k;
            const int slot = it % GATHER_SLOTS;
            // the store that last used this slot must have finished reading it
            bulk_wait_read<GATHER_SLOTS - GATHER_LAG - 1>();
            const int s = seg_of(k);
            mbar_expect_tx(&bars[slot], seg_bytes(s));
            bulk_g2s(smem + slot * GATHER_SEG_BYTES, src + (static_cast<long long>(s) << GATHER_SEG_SHIFT),
                     seg_bytes(s), &bars[slot]);
        }
        const int j = k - GATHER_LAG;
        if (j >= 0) {
            const uint32_t it = base_it + j;
            const int slot = it % GATHER_SLOTS;
            if (!mbar_wait(&bars[slot], (it / GATHER_SLOTS) & 1, 700 + slot)) return false;
            const int s = seg_of(j);
            const long long off = static_cast<long long>(s) << GATHER_SEG_SHIFT;
            bulk_s2g(dst_a + off, smem + slot * GATHER_SEG_BYTES, seg_bytes(s));
            if (dst_b != nullptr) bulk_s2g(dst_b + off, smem + slot * GATHER_SEG_BYTES, seg_bytes(s));
            bulk_commit();
            if (ready != nullptr && j >= 1) {
                bulk_wait_all<1>();   // everything but the group just committed is complete
                fence_proxy_async_all();
                __threadfence();
                st_release_gpu(&ready[seg_of(j - 1)], seq);
                flagged = j;
            }
        }
    }
    bulk_wait_all<0>();
    fence_proxy_async_all();
    __threadfence_system();
    if (ready != nullptr)
        for (int j = flagged; j < mine; ++j) st_release_gpu(&ready[seg_of(j)], seq);
    ring_it = base_it + mine;
    return true;
}

// Body of a copy CTA.  `smem` is 1024-byte aligned dynamic shared memory of at least GATHER_SLOTS segments + barriers.
__device__ void gather_copy_cta(const GatherArgs& g, uint8_t* smem, int cta) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GATHER_SLOTS * GATHER_SEG_BYTES);
    if (threadIdx.x != 0) return;
    for (int s = 0; s < GATHER_SLOTS; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    fence_proxy_async_smem();
    uint32_t ring_it = 0;
    int* my_pad = g.pad[g.rank];
    const int nseg_shard = static_cast<int>((g.shard_bytes + GATHER_SEG_BYTES - 1) >> GATHER_SEG_SHIFT);
    // 0. the staging slot was last used by call seq - 2: every peer must have finished reading it
    for (int p = 0; p < g.world; ++p)
        if (p != g.rank && !wait_flag_sys(&my_pad[PAD_DONE + p], g.seq - 2, 800 + p)) return;
    // 1. own contribution -> staging (for the peers) and -> its place in the gathered buffer
    if (!gather_copy_range(smem, bars, ring_it, g.local_src, g.dst + g.rank * g.shard_bytes, g.stage[g.rank],
                           g.shard_bytes, g.ready + g.rank * nseg_shard, g.seq, cta, g.n_copy))
        return;
    // all copy CTAs have written their part of the stage -> publish
    const unsigned int target = static_cast<unsigned int>(g.seq) * g.n_copy;
    if (atomicAdd(&g.counters[0], 1u) + 1u == target) {
        __threadfence_system();
        for (int p = 0; p < g.world; ++p)
            if (p != g.rank) st_release_sys(&g.pad[p][PAD_SIG + g.rank], g.seq);
    }
    // 2. pull the peers, nearest-rank-first rotation so that the peers are read evenly
    for (int i = 1; i < g.world; ++i) {
        const int p = (g.rank + i) % g.world;
        if (!wait_flag_sys(&my_pad[PAD_SIG + p], g.seq, 820 + p)) return;
        if (!gather_copy_range(smem, bars, ring_it, g.stage[p], g.dst + p * g.shard_bytes, nullptr, g.shard_bytes,
                               g.ready + p * nseg_shard, g.seq, cta, g.n_copy))
            return;
    }
    // 3. tell the peers that their staging slot is free again
    if (atomicAdd(&g.counters[1], 1u) + 1u == target) {
        __threadfence_system();
        for (int p = 0; p < g.world; ++p)
            if (p != g.rank) st_release_sys(&g.pad[p][PAD_DONE + g.rank], g.seq);
    }
}

// Called by the GEMM's TMA producer thread before it loads rows [r0, r0 + rows) of the gathered operand.
__device__ __forceinline__ bool gather_wait_rows(const GatherArgs& g, int r0, int rows, int total_rows) {
    const int r1 = min(r0 + rows, total_rows);
    if (r1 <= r0) return true;
    const long long lo = g.operand_off + static_cast<long long>(r0) * g.row_bytes;
    const long long hi = g.operand_off + static_cast<long long>(r1) * g.row_bytes - 1;
    // segment numbering is per shard (a shard's last segment may be partial)
    const int nseg_shard = static_cast<int>((g.shard_bytes + GATHER_SEG_BYTES - 1) >> GATHER_SEG_SHIFT);
    for (long long b = lo; b <= hi;) {
        const int shard = static_cast<int>(b / g.shard_bytes);
        const long long in = b - shard * g.shard_bytes;
        const int seg = static_cast<int>(in >> GATHER_SEG_SHIFT);
        if (!wait_flag_gpu(&g.ready[shard * nseg_shard + seg], g.seq, 900)) return false;
        long long next = shard * g.shard_bytes + (static_cast<long long>(seg + 1) << GATHER_SEG_SHIFT);
        const long long shard_end = (shard + 1) * g.shard_bytes;
        b = next < shard_end ? next : shard_end;
    }
    fence_proxy_async_all();
    return true;
}

}  // namespace lme
