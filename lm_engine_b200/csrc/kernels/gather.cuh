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
//   own contribution  -> stage[rank][seq & 1] (symmetric) by a device-to-device copy ahead of the kernel
//   sig[rank] := seq     written into every peer's pad when the kernel starts: "rank's data for seq is there"
//   pull from peer p     after our pad shows sig[p] >= seq
// Every wait is bounded (LME_WAIT_LIMIT_NS); on expiry the status word is set and the CTA returns, which makes the
// GEMM CTAs run into their own bounded waits and return as well.
#pragma once

namespace lme {

static constexpr int GATHER_MAX_RANKS = 8;
static constexpr int GATHER_SEG_SHIFT = 15;                 // 32 KB segments
static constexpr int GATHER_SEG_BYTES = 1 << GATHER_SEG_SHIFT;
static constexpr int GATHER_SLOTS = 6;
static constexpr int GATHER_LAG = 4;                        // loads in flight ahead of the store stage
static constexpr int GATHER_FLAG_LAG = 3;                   // stores allowed in flight behind a published flag

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
    const uint8_t* local_src;   // this rank's contribution (the GEMM reads its own rows from here)
    uint8_t* stage[GATHER_MAX_RANKS];   // slot-selected staging buffer of every rank ([rank] = ours)
    uint8_t* dst;               // local gathered buffer, world * shard_bytes
    int* ready;                 // local, one word per segment of dst
    int* pad[GATHER_MAX_RANKS];         // signal pad of every rank ([rank] = ours)
    unsigned int* counters;     // local, 2 words: copy-CTA arrival counters (monotonic)
    int local_row0, local_rows; // rows of the gathered operand that are this rank's own (read from local_src)
    int flag_every;             // publish readiness every this many segments of a copy CTA
    int seg_shift;              // log2 of the bytes covered by one ready word (15 with copy CTAs; the chunk size
                                // when copy engines deliver the data and the stream writes the words)
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
    const uint64_t limit = lme_peer_wait_ns;
    uint32_t spins = 0;
    while (ld_acquire_sys(p) < want) {
        __nanosleep(64);
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > limit) {
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
                                  int n_cta, int flag_every) {
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
            if (ready != nullptr && j >= GATHER_FLAG_LAG && ((j - GATHER_FLAG_LAG + 1) % flag_every) == 0) {
                // all but the newest groups are complete (wait_group makes their writes visible to this thread, the
                // release below publishes them): flags trail the stores so that the ring never drains
                bulk_wait_all<GATHER_FLAG_LAG>();
                for (int f = flagged; f <= j - GATHER_FLAG_LAG; ++f) st_release_gpu(&ready[seg_of(f)], seq);
                flagged = j - GATHER_FLAG_LAG + 1;
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
    // 1. This rank's contribution was copied into its staging slot before this kernel (stream order), so it can be
    //    announced right away.  Two slots need no "done" handshake before that copy overwrites one: the slot was
    //    last read by the peers in call seq - 2, and in call seq - 1 this rank waited for every peer's sig, which a
    //    peer only sends from the kernel that follows its call seq - 2 in stream order.
    if (cta == 0) {
        __threadfence_system();
        for (int p = 0; p < g.world; ++p)
            if (p != g.rank) st_release_sys(&g.pad[p][PAD_SIG + g.rank], g.seq);
    }
    // 2. pull the peers, nearest rank first, so that every peer is read by one rank at a time
    for (int i = 1; i < g.world; ++i) {
        const int p = (g.rank + i) % g.world;
        if (!wait_flag_sys(&my_pad[PAD_SIG + p], g.seq, 820 + p)) return;
        fence_proxy_async_all();   // the bulk (async proxy) reads below are ordered after the acquire above
        if (!gather_copy_range(smem, bars, ring_it, g.stage[p], g.dst + p * g.shard_bytes, nullptr, g.shard_bytes,
                               g.ready + p * nseg_shard, g.seq, cta, g.n_copy, g.flag_every))
            return;
    }
}

// Called by the GEMM's TMA producer thread before it loads rows [r0, r0 + rows) of the gathered operand.
__device__ __forceinline__ bool gather_wait_rows(const GatherArgs& g, int r0, int rows, int total_rows) {
    const int r1 = min(r0 + rows, total_rows);
    if (r1 <= r0) return true;
    const long long lo = g.operand_off + static_cast<long long>(r0) * g.row_bytes;
    const long long hi = g.operand_off + static_cast<long long>(r1) * g.row_bytes - 1;
    // segment numbering is per shard (a shard's last segment may be partial)
    const long long seg_bytes = 1ll << g.seg_shift;
    const int nseg_shard = static_cast<int>((g.shard_bytes + seg_bytes - 1) >> g.seg_shift);
    for (long long b = lo; b <= hi;) {
        const int shard = static_cast<int>(b / g.shard_bytes);
        const long long in = b - shard * g.shard_bytes;
        const int seg = static_cast<int>(in >> g.seg_shift);
        if (!wait_flag_gpu(&g.ready[shard * nseg_shard + seg], g.seq, 900)) return false;
        long long next = shard * g.shard_bytes + (static_cast<long long>(seg + 1) << g.seg_shift);
        const long long shard_end = (shard + 1) * g.shard_bytes;
        b = next < shard_end ? next : shard_end;
    }
    fence_proxy_async_all();
    return true;
}

// Announces this rank's staging slot to the peers (one thread).
__global__ void gather_signal_kernel(GatherArgs g) {
    __threadfence_system();
    for (int p = 0; p < g.world; ++p)
        if (p != g.rank) st_release_sys(&g.pad[p][PAD_SIG + g.rank], g.seq);
}
// Holds a stream until peer `src` has announced call `seq` (one thread, bounded: on expiry the status word is set
// and the stream continues, so the copies behind it read a stale slot but nothing hangs).
__global__ void gather_wait_peer_kernel(const int* word, int seq, unsigned int id) { wait_flag_sys(word, seq, id); }

// ----------------------------------------------------------------------------------------------------------------
// GEMM -> reduce-scatter fused into the epilogue.  Every rank multiplies its K-slice for all M rows; the rows are
// owned by the ranks in equal blocks.  Tiles of rows owned by a peer are stored (bf16) straight into the owner's
// receive slab over NVLink, followed by a per-(tile, warp) arrival flag; tiles of own rows are multiplied last, and
// their epilogue adds the partial results that the peers have delivered meanwhile, then bias / residual, and writes
// the final output.  No separate reduction pass, no extra CTAs.
// Two slab slots (seq & 1) need no "done" handshake: a rank overwrites a peer's slot of call seq - 2 only after its
// own call seq - 1 consumed that peer's flags of call seq - 1, which the peer wrote after finishing call seq - 2.
struct RsArgs {
    int enabled, rank, world, seq;
    int rows_per_rank, tiles_per_rank;   // rows_per_rank is a multiple of the tile height
    int rotate;                          // m-tile rotation: rows of rank + 1 first, own rows last
    long long slab_ld;                   // N
    uint8_t* slab[GATHER_MAX_RANKS];     // slot-selected receive slab of every rank: [src][rows_per_rank][N] bf16
    int* flags[GATHER_MAX_RANKS];        // arrival flags of every rank: [src][tiles_per_rank][tiles_n][4]
};

}  // namespace lme
