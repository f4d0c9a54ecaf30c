// Router kernels of the mixture-of-experts layer: top-k selection fused with the softmax (forward and backward), and
// the padded per-expert row layout computed straight from the unsorted selection (a stable counting sort: histogram
// per CTA, one scan CTA, rank per CTA) so the layer needs no sort, no search and no host round trip.
// Included by lme_cuda.cu.

namespace lme {

constexpr int ROUTE_CHUNK = 2048;     // assignments ranked by one CTA
constexpr int ROUTE_MAX_E = 1024;
constexpr int TOPK_MAX_PER_LANE = 16; // experts held by one lane -> at most 512 experts

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// One warp per token.  NORMALIZED: weights = softmax over the k selected logits; else weights = softmax over all
// experts, read at the selected ones (lse keeps the row's log-sum-exp for the backward pass).  Selection is in
// descending order, the lower index first among equal values.
template <bool NORMALIZED>
__global__ void __launch_bounds__(256)
moe_topk_softmax_fwd_kernel(const __nv_bfloat16* __restrict__ logits, int T, int E, int K,
                            __nv_bfloat16* __restrict__ weights, long long* __restrict__ selected,
                            float* __restrict__ lse) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const __nv_bfloat16* row = logits + static_cast<long long>(t) * E;
    float v[TOPK_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < TOPK_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? __bfloat162float(row[e]) : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    float denom = 0.f;
    if (!NORMALIZED) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
        for (int i = 0; i < TOPK_MAX_PER_LANE; ++i) denom += (lane + 32 * i < E) ? __expf(v[i] - mx) : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
        if (lane == 0 && lse) lse[t] = mx + __logf(denom);
    }
    float mine = 0.f;       // lane k keeps the k-th selected logit
    int mine_idx = 0;
    float top = 0.f;
    for (int k = 0; k < K; ++k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < TOPK_MAX_PER_LANE; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (v[i] > bv || (v[i] == bv && e < bi))) { bv = v[i]; bi = e; }
        }
        warp_argmax(bv, bi);
        if (k == 0) top = bv;
        if (lane == k) { mine = bv; mine_idx = bi; }
#pragma unroll
        for (int i = 0; i < TOPK_MAX_PER_LANE; ++i)
            if (lane + 32 * i == bi) v[i] = -INFINITY;
    }
    float w;
    if (NORMALIZED) {
        float ex = lane < K ? __expf(mine - top) : 0.f;
        float s = ex;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        w = ex / s;
    } else {
        w = __expf(mine - mx) / denom;
    }
    if (lane < K) {
        weights[static_cast<long long>(t) * K + lane] = __float2bfloat16(w);
        selected[static_cast<long long>(t) * K + lane] = mine_idx;
    }
}

template <bool NORMALIZED>
__global__ void __launch_bounds__(256)
moe_topk_softmax_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ selected,
                            const __nv_bfloat16* __restrict__ dw, const float* __restrict__ lse, int T, int E, int K,
                            __nv_bfloat16* __restrict__ dlogits) {
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const __nv_bfloat16* row = logits + static_cast<long long>(t) * E;
    __nv_bfloat16* drow = dlogits + static_cast<long long>(t) * E;
    const int sel = lane < K ? static_cast<int>(selected[static_cast<long long>(t) * K + lane]) : 0;
    const float l = lane < K ? __bfloat162float(row[sel]) : -INFINITY;
    const float g = lane < K ? __bfloat162float(dw[static_cast<long long>(t) * K + lane]) : 0.f;
    float p;
    if (NORMALIZED) {
        float mx = l;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float ex = lane < K ? __expf(l - mx) : 0.f;
        float s = ex;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        p = ex / s;
    } else {
        p = lane < K ? __expf(l - lse[t]) : 0.f;
    }
    float dot = p * g;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    for (int e = lane; e < E; e += 32)
        drow[e] = __float2bfloat16(NORMALIZED ? 0.f : -__expf(__bfloat162float(row[e]) - lse[t]) * dot);
    __syncwarp();
    if (lane < K) drow[sel] = __float2bfloat16(p * (g - dot));
}

// ---- padded per-expert layout from the unsorted selection ---------------------------------------------------------

__global__ void __launch_bounds__(256)
moe_route_count_kernel(const long long* __restrict__ sel, int total, int E, int* __restrict__ cta_counts) {
    __shared__ int hist[ROUTE_MAX_E];
    for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int base = blockIdx.x * ROUTE_CHUNK;
    const int end = min(total, base + ROUTE_CHUNK);
    for (int i = base + threadIdx.x; i < end; i += blockDim.x) {
        const long long e = sel[i];
        if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cta_counts[blockIdx.x * E + e] = hist[e];
}

// One CTA: per-expert totals, the CTAs' counts turned into exclusive prefixes in place, row ranges rounded up to the
// 128-row tile, and the tile -> expert table (-1 past the last expert).
__global__ void __launch_bounds__(1024)
moe_route_scan_kernel(int* __restrict__ cta_counts, int G, int E, int ntiles, long long* __restrict__ freq,
                      int* __restrict__ k0, int* __restrict__ kb, int* __restrict__ tile_group) {
    __shared__ int s_pad[ROUTE_MAX_E];
    __shared__ int s_start[ROUTE_MAX_E + 1];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int run = 0;
        for (int b = 0; b < G; ++b) {
            const int c = cta_counts[b * E + e];
            cta_counts[b * E + e] = run;
            run += c;
        }
        freq[e] = run;
        s_pad[e] = (run + 127) / 128 * 128;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        int carry = 0;
        for (int c = 0; c < E; c += 32) {
            const int e = c + threadIdx.x;
            const int v = e < E ? s_pad[e] : 0;
            int incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (threadIdx.x >= o) incl += up;
            }
            if (e < E) s_start[e] = carry + incl - v;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (threadIdx.x == 0) s_start[E] = carry;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        k0[e] = s_start[e];
        kb[e] = s_pad[e] / 64;
        const int first = s_start[e] / 128, last = min(ntiles, (s_start[e] + s_pad[e]) / 128);
        for (int tile = first; tile < last; ++tile) tile_group[tile] = e;
    }
    for (int tile = s_start[E] / 128 + threadIdx.x; tile < ntiles; tile += blockDim.x) tile_group[tile] = -1;
}

// slot[i] = first row of the expert + assignments of that expert in earlier CTAs + rank inside this CTA, ranks taken
// in index order (stable), so the result does not depend on scheduling.
__global__ void __launch_bounds__(256)
moe_route_slot_kernel(const long long* __restrict__ sel, int total, int E, const int* __restrict__ cta_prefix,
                      const int* __restrict__ k0, int* __restrict__ slot) {
    __shared__ int running[ROUTE_MAX_E];
    for (int e = threadIdx.x; e < E; e += blockDim.x) running[e] = k0[e] + cta_prefix[blockIdx.x * E + e];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int base = blockIdx.x * ROUTE_CHUNK;
    const int end = min(total, base + ROUTE_CHUNK);
    for (int off = base; off < end; off += blockDim.x) {
        const int i = off + threadIdx.x;
        const long long e64 = i < end ? sel[i] : -1;
        const bool valid = e64 >= 0 && e64 < E;
        const int e = valid ? static_cast<int>(e64) : -1 - lane;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int leader = __ffs(same) - 1;
        const int rank = __popc(same & ((1u << lane) - 1u));
        int first = 0;
        for (int w = 0; w < 8; ++w) {
            if (warp == w) {
                if (valid && lane == leader) {
                    first = running[e];
                    running[e] = first + __popc(same);
                }
                first = __shfl_sync(0xffffffffu, first, leader);
            }
            __syncthreads();
        }
        if (i < end) slot[i] = valid ? first + rank : -1;
    }
}

}  // namespace lme

using namespace lme;

extern "C" int lme_moe_topk_softmax_fwd(const void* logits, int T, int E, int K, int normalized, void* weights,
                                        long long* selected, float* lse, void* stream) {
    if (T < 0 || E <= 0 || K <= 0 || K > 32 || K > E || E > 32 * TOPK_MAX_PER_LANE) return LME_ERR_SHAPE;
    if (!normalized && !lse) return LME_ERR_SHAPE;
    if (T == 0) return LME_OK;
    auto st = static_cast<cudaStream_t>(stream);
    const int blocks = (T + 7) / 8;
    if (normalized)
        moe_topk_softmax_fwd_kernel<true><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), T, E, K,
                                                                 static_cast<__nv_bfloat16*>(weights), selected, lse);
    else
        moe_topk_softmax_fwd_kernel<false><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), T, E, K,
                                                                  static_cast<__nv_bfloat16*>(weights), selected, lse);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_moe_topk_softmax_bwd(const void* logits, const long long* selected, const void* dw,
                                        const float* lse, int T, int E, int K, int normalized, void* dlogits,
                                        void* stream) {
    if (T < 0 || E <= 0 || K <= 0 || K > 32 || K > E) return LME_ERR_SHAPE;
    if (!normalized && !lse) return LME_ERR_SHAPE;
    if (T == 0) return LME_OK;
    auto st = static_cast<cudaStream_t>(stream);
    const int blocks = (T + 7) / 8;
    if (normalized)
        moe_topk_softmax_bwd_kernel<true><<<blocks, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(logits), selected, static_cast<const __nv_bfloat16*>(dw), lse, T, E, K,
            static_cast<__nv_bfloat16*>(dlogits));
    else
        moe_topk_softmax_bwd_kernel<false><<<blocks, 256, 0, st>>>(
            static_cast<const __nv_bfloat16*>(logits), selected, static_cast<const __nv_bfloat16*>(dw), lse, T, E, K,
            static_cast<__nv_bfloat16*>(dlogits));
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_moe_route_chunks(int total) { return (total + ROUTE_CHUNK - 1) / ROUTE_CHUNK; }

// scratch: lme_moe_route_chunks(total) * E ints.  tile_group has ntiles entries (capacity / 128).
extern "C" int lme_moe_route_layout(const long long* selected, int total, int E, int* scratch, long long* freq,
                                    int* k0, int* kb, int* tile_group, int ntiles, int* slot, void* stream) {
    if (total <= 0 || E <= 0 || E > ROUTE_MAX_E || ntiles <= 0) return LME_ERR_SHAPE;
    if (static_cast<long long>(ntiles) * 128 < static_cast<long long>(total) + static_cast<long long>(E) * 127)
        return LME_ERR_SHAPE;
    auto st = static_cast<cudaStream_t>(stream);
    const int G = lme_moe_route_chunks(total);
    moe_route_count_kernel<<<G, 256, 0, st>>>(selected, total, E, scratch);
    moe_route_scan_kernel<<<1, 1024, 0, st>>>(scratch, G, E, ntiles, freq, k0, kb, tile_group);
    moe_route_slot_kernel<<<G, 256, 0, st>>>(selected, total, E, scratch, k0, slot);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
