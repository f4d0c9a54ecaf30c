// Expert-parallel token exchange over NVLink peer memory, without a library collective and without a host round
// trip: the role of the two all-to-alls (and the count exchange before them) around the experts of a
// mixture-of-experts layer (lm_engine/modeling_utils/mlp_blocks/moe/module.py:276-291 in the reference keeps every
// expert on every rank; its expert-parallel relatives use an all-to-all of rows with host-side split sizes).
//
// Every rank owns E / world consecutive experts.  All row traffic is PULLED with 16-byte peer loads (measured here:
// peer loads reach 0.8 of the peer-copy rate from such kernels, scattered peer stores of rows 0.47); only 8-byte table
// entries and flags are stored into peer memory.  One round:
//   1. counts   every rank stores its per-expert counts into every peer's count table, then a flag (CNT).
//   2. bases    every rank waits for all CNT flags and derives, from the same table, the SAME padded per-expert
//               layout of every owner: expert e of owner r starts at k0_r[e] (multiple of 128 rows); the rows of
//               source s inside it start after those of sources < s.  The rank keeps the tables of its own experts
//               (tile -> expert, k0, kb) and, for its role as a source, the first row of each expert at its owner.
//   3. offer    the source copies its rows into its staging buffer (symmetric memory) and stores, for each of its
//               assignments, the entry (round, source, row index) into the owner's row table at the assignment's row;
//               the last CTA to finish publishes the ARR flag at every peer.
//   4. land     the owner waits for all ARR flags and pulls every row of its used tiles from the staging buffer its
//               table entry names, into a private buffer; rows without an entry of this round (the tail of an
//               expert's last tile) become zero.  The grouped GEMMs run on that buffer; the last one writes into the
//               owner's output slab, then the owner publishes DONE at every peer.
//   5. pull     after all DONE flags a source reads its rows back from the owners' output slabs.
// The backward pass is the same round on a second set of buffers and flags (offer of output gradients, pull of input
// gradients); the layout of step 2 is reused.
//
// Flags hold the round number (monotonic), table entries carry it, so nothing is ever reset.  Every wait is bounded;
// on expiry the status word is set and the kernel goes on (the step's result is wrong and the host raises when it
// reads the status).  A buffer is rewritten only after every reader finished with it: a rank starts round n + 1 after
// its pull of round n, the pull follows the DONE flags of all owners, and an owner publishes DONE only after its own
// reads of round n.
// Included by lme_cuda.cu.

namespace lme {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_MAX_E = 1024;
// words of one direction's flag block inside a rank's int32 pad
constexpr int EP_CNT = 0;    // [8] counts of source s have arrived
constexpr int EP_ARR = 8;    // [8] rows of source s have arrived
constexpr int EP_DONE = 16;  // [8] owner r's output slab is ready
constexpr int EP_WORDS = 24;

struct EpPtrs {
    uint8_t* p[EP_MAX_RANKS];
};

__global__ void __launch_bounds__(256)
ep_publish_counts_kernel(const long long* __restrict__ freq, EpPtrs counts, EpPtrs pads, int rank, int world, int E,
                         int seq) {
    const int p = blockIdx.x;
    int* dst = reinterpret_cast<int*>(counts.p[p]) + static_cast<long long>(rank) * E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = static_cast<int>(freq[e]);
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(reinterpret_cast<int*>(pads.p[p]) + EP_CNT + rank, seq);
}

// One CTA.  counts: [world][E] (this rank's table, filled by the peers).  Outputs: base[e] = first row at e's owner
// of this rank's tokens for expert e; for the rank's own experts k0 / kb / rows (= real rows) and the tile table.
__global__ void __launch_bounds__(1024)
ep_bases_kernel(const int* __restrict__ counts, const int* __restrict__ pad, int rank, int world, int E, int seq,
                int cap, int* __restrict__ base, int* __restrict__ k0_own, int* __restrict__ kb_own,
                int* __restrict__ rows_own, int* __restrict__ tile_group) {
    __shared__ int s_pad[EP_MAX_E];
    __shared__ int s_k0[EP_MAX_E];
    if (threadIdx.x < world) wait_flag_sys(pad + EP_CNT + threadIdx.x, seq, 1100 + threadIdx.x);
    __syncthreads();
    const int Le = E / world, ntiles = cap / 128;
    const int e = threadIdx.x;                              // E <= 1024 = blockDim.x
    int tot = 0, before = 0;
    if (e < E) {
        for (int s = 0; s < world; ++s) {
            const int c = counts[s * E + e];
            tot += c;
            if (s < rank) before += c;
        }
        s_pad[e] = (tot + 127) / 128 * 128;
    }
    __syncthreads();
    if (e < E) {
        const int first = e / Le * Le;
        int k0 = 0;
        for (int j = first; j < e; ++j) k0 += s_pad[j];
        s_k0[e] = k0;
        base[e] = k0 + before;
        if (e % Le == Le - 1 && k0 + s_pad[e] > cap) report_error(STATUS_BOUNDS, 1200 + e / Le);
        if (e / Le == rank) {
            const int le = e - first;
            const int end = min(k0 + s_pad[e], cap);
            const int start = min(k0, end);
            k0_own[le] = start;
            kb_own[le] = (end - start) / 64;
            rows_own[le] = min(tot, end - start);
            for (int tile = start / 128; tile < end / 128; ++tile) tile_group[tile] = le;
        }
    }
    __syncthreads();
    const int last = rank * Le + Le - 1;
    const int used = min(s_k0[last] + s_pad[last], cap);
    for (int tile = used / 128 + threadIdx.x; tile < ntiles; tile += blockDim.x) tile_group[tile] = -1;
}

// dest[a] = (owner, row at the owner) of assignment a; row < 0: dropped (expert id out of range, or past the capacity,
// which the bases kernel has reported).
__global__ void __launch_bounds__(256)
ep_dest_kernel(const long long* __restrict__ sel, const int* __restrict__ slot, const int* __restrict__ k0_local,
               const int* __restrict__ base, int A, int E, int Le, int cap, int2* __restrict__ dest) {
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= A) return;
    const long long e = sel[a];
    int2 d = make_int2(0, -1);
    if (e >= 0 && e < E) {
        const int row = base[e] + slot[a] - k0_local[e];
        if (row >= 0 && row < cap) d = make_int2(static_cast<int>(e) / Le, row);
    }
    dest[a] = d;
}

// Table entry of a landing row: x = round * 8 + source rank, y = index of the source's staged row.
// One thread per assignment stores its entry at the owner; the last CTA publishes the arrival flag everywhere.
__global__ void __launch_bounds__(256)
ep_offer_rows_kernel(const int2* __restrict__ dest, EpPtrs tables, EpPtrs pads, int A, unsigned int* __restrict__ counter,
                     int rank, int world, int seq) {
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a < A) {
        const int2 d = dest[a];
        if (d.y >= 0) reinterpret_cast<int2*>(tables.p[d.x])[d.y] = make_int2(seq * 8 + rank, a);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int arrived = atomicAdd(counter, 1u);
        if (arrived == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            for (int p = 0; p < world; ++p) st_release_sys(reinterpret_cast<int*>(pads.p[p]) + EP_ARR + rank, seq);
        }
    }
}

// Owner: rows of tiles that belong to an expert are fetched from the staging buffer their table entry names (staged
// row = entry.y / rep), rows without an entry of round `seq` are zeroed, tiles without an expert are left alone.
// Each CTA takes LAND_ROWS consecutive rows.
constexpr int LAND_ROWS = 4;
__global__ void __launch_bounds__(256)
ep_land_rows_kernel(EpPtrs stages, const int2* __restrict__ table, const int* __restrict__ tile_group,
                    __nv_bfloat16* __restrict__ out, int H, int rep, int seq) {
    const int row0 = blockIdx.x * LAND_ROWS;
    if (tile_group[row0 / 128] < 0) return;
#pragma unroll
    for (int i = 0; i < LAND_ROWS; ++i) {
        const int row = row0 + i;
        const int2 e = table[row];
        uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(row) * H);
        if ((e.x >> 3) == seq) {
            const uint4* src = reinterpret_cast<const uint4*>(stages.p[e.x & 7]) +
                               static_cast<long long>(e.y / rep) * (H / 8);
            for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = ld_peer_v4(src + c);
        } else {
            for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = make_uint4(0, 0, 0, 0);
        }
    }
}

__global__ void ep_wait_kernel(const int* pad, int word0, int world, int seq, unsigned int id) {
    if (threadIdx.x < world) wait_flag_sys(pad + word0 + threadIdx.x, seq, id + threadIdx.x);
}

__global__ void ep_signal_kernel(EpPtrs pads, int word, int world, int seq) {
    __threadfence_system();
    if (threadIdx.x < world) st_release_sys(reinterpret_cast<int*>(pads.p[threadIdx.x]) + word, seq);
}

// reduce == 0: out[t * K + k] = row dest[t * K + k] of its owner's slab (zero when dropped);
// reduce != 0: out[t] = sum over k of those rows (fp32 accumulation).
__global__ void __launch_bounds__(256)
ep_pull_rows_kernel(EpPtrs slabs, const int2* __restrict__ dest, __nv_bfloat16* __restrict__ out, int K, int H,
                    int reduce) {
    const long long t = blockIdx.x;
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < K; ++k) {
            const int2 d = dest[t * K + k];
            uint4 v = make_uint4(0, 0, 0, 0);
            if (d.y >= 0)
                v = ld_peer_v4(reinterpret_cast<const uint4*>(slabs.p[d.x]) + static_cast<long long>(d.y) * (H / 8) + c);
            if (!reduce) {
                reinterpret_cast<uint4*>(out + (t * K + k) * H)[c] = v;
            } else {
                float2 f;
                f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
                f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
                f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
                f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
            }
        }
        if (reduce) {
            uint4 v;
            v.x = pack_bf16x2(acc[0], acc[1]);
            v.y = pack_bf16x2(acc[2], acc[3]);
            v.z = pack_bf16x2(acc[4], acc[5]);
            v.w = pack_bf16x2(acc[6], acc[7]);
            reinterpret_cast<uint4*>(out + t * H)[c] = v;
        }
    }
}

static EpPtrs ep_ptrs(void* const* arr, int world, long long byte_off = 0) {
    EpPtrs r{};
    for (int i = 0; i < world; ++i) r.p[i] = static_cast<uint8_t*>(arr[i]) + byte_off;
    return r;
}

}  // namespace lme

using namespace lme;

static bool ep_world_ok(int rank, int world) { return world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world; }

// pads[r]: rank r's flag block of this direction (EP_WORDS int32 words).  counts[r]: rank r's [world][E] int32 table.
extern "C" int lme_ep_publish_counts(const long long* freq, void* const* counts, void* const* pads, int rank,
                                     int world, int E, int seq, void* stream) {
    if (!ep_world_ok(rank, world) || E <= 0 || E > EP_MAX_E || E % world) return LME_ERR_SHAPE;
    ep_publish_counts_kernel<<<world, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        freq, ep_ptrs(counts, world), ep_ptrs(pads, world), rank, world, E, seq);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_ep_bases(const int* counts, const int* pad, int rank, int world, int E, int seq, int cap, int* base,
                            int* k0_own, int* kb_own, int* rows_own, int* tile_group, void* stream) {
    if (!ep_world_ok(rank, world) || E <= 0 || E > EP_MAX_E || E % world || cap <= 0 || cap % 128)
        return LME_ERR_SHAPE;
    ep_bases_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(counts, pad, rank, world, E, seq, cap, base,
                                                                       k0_own, kb_own, rows_own, tile_group);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_ep_dest(const long long* sel, const int* slot, const int* k0_local, const int* base, int A, int E,
                           int world, int cap, void* dest, void* stream) {
    if (A <= 0 || E <= 0 || world <= 0 || E % world) return LME_ERR_SHAPE;
    ep_dest_kernel<<<(A + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(sel, slot, k0_local, base, A, E,
                                                                                  E / world, cap,
                                                                                  static_cast<int2*>(dest));
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

// Stores this rank's table entries for its A assignments (dest: int32 [A][2]) into the owners' row tables and
// publishes the arrival flag; counter: one zeroed word of this rank.  The staged rows must be complete in stream order.
extern "C" int lme_ep_offer_rows(const void* dest, void* const* tables, void* const* pads, int A,
                                 unsigned int* counter, int rank, int world, int seq, void* stream) {
    if (!ep_world_ok(rank, world) || A <= 0 || seq <= 0 || seq >= (1 << 27)) return LME_ERR_SHAPE;
    ep_offer_rows_kernel<<<(A + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int2*>(dest), ep_ptrs(tables, world), ep_ptrs(pads, world), A, counter, rank, world, seq);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

// stages[r]: rank r's staging buffer (rows of H bf16); table: this rank's row table (int32 [cap][2]); out [cap][H].
extern "C" int lme_ep_land_rows(void* const* stages, const void* table, const int* tile_group, void* out, int cap,
                                int H, int rep, int seq, int world, void* stream) {
    if (world <= 0 || world > EP_MAX_RANKS || cap <= 0 || cap % 128 || H <= 0 || H % 8 || rep <= 0)
        return LME_ERR_SHAPE;
    ep_land_rows_kernel<<<cap / LAND_ROWS, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        ep_ptrs(stages, world), static_cast<const int2*>(table), tile_group, static_cast<__nv_bfloat16*>(out), H, rep,
        seq);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

// which: 0 = rows arrived (ARR), 1 = output ready (DONE)
extern "C" int lme_ep_wait(const int* pad, int which, int world, int seq, void* stream) {
    if (world <= 0 || world > EP_MAX_RANKS) return LME_ERR_SHAPE;
    ep_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pad, which ? EP_DONE : EP_ARR, world, seq,
                                                                    which ? 1400u : 1300u);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_ep_signal_done(void* const* pads, int rank, int world, int seq, void* stream) {
    if (!ep_world_ok(rank, world)) return LME_ERR_SHAPE;
    ep_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ep_ptrs(pads, world), EP_DONE + rank, world, seq);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_ep_pull_rows(void* const* slabs, const void* dest, void* out, int T, int K, int H, int reduce,
                                int world, void* stream) {
    if (world <= 0 || world > EP_MAX_RANKS || T <= 0 || K <= 0 || H <= 0 || H % 8) return LME_ERR_SHAPE;
    ep_pull_rows_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        ep_ptrs(slabs, world), static_cast<const int2*>(dest), static_cast<__nv_bfloat16*>(out), K, H, reduce);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_ep_flag_words(void) { return EP_WORDS; }
