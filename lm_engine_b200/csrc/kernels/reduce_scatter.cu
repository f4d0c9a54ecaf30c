// Gradient reduce-scatter over NVLink fused with the mean, the write (or accumulation) of the gradient shard and the
// partial sums of squares of the gradient norm: the data-parallel gradient path of ZeRO-1/2/3 in ONE kernel, with no
// library collective on the data plane (the reference runs FSDP-2's reduce-scatter through NCCL and a separate
// clip_grad_norm_, lm_engine/distributed.py:326-344, lm_engine/train.py:211).
//
// Every rank's unreduced gradient buffer lives in symmetric memory.  Rank r owns elements [r * n, (r + 1) * n) of
// the buffer; its kernel reads that slice from every rank (its own from local memory, the others' with plain
// 16-byte loads over NVLink, or all of them at once with multimem.ld_reduce through the switch), sums in fp32 in
// rank order, multiplies by `scale`, adds the previous shard when accumulating, writes the shard in the gradient
// dtype and leaves one partial sum of squares of what it wrote per CTA.
//
// The kernel needs no shared-memory tiles and few registers, so its CTAs become resident NEXT TO the persistent
// GEMM CTAs of the backward pass instead of displacing them (a collective kernel that takes whole SMs delays the
// GEMM CTAs of those SMs, and a persistent GEMM with a static tile schedule is as slow as its latest CTA).
//
// Cross-rank protocol (pads are the 16-word int32 signal pads of gather.cuh, `seq` grows by one per call):
//   sig[rank] := seq in every peer's pad when the kernel starts: "my buffer for call seq is complete" (stream order
//                puts the kernel behind the backward pass that filled it, and behind this rank's reads of call seq-1)
//   wait sig[p] >= seq for every peer p (bounded), then read.
// A rank may overwrite a buffer once its own NEXT call has finished: that call saw every peer's sig for seq + 1,
// which a peer sends only after its reads of call seq.
#include "common.cuh"
#include "../lme_api.h"

#include "gather.cuh"

namespace lme {

struct RsPeerArgs {
    const void* src[GATHER_MAX_RANKS];   // this rank's slice inside every rank's buffer ([rank] = local memory)
    int* pad[GATHER_MAX_RANKS];
    const void* mc_src;                  // multicast address of the slice (NVLS variant), else null
    int rank, world, seq;
    void* out;
    long long n;
    float scale;
    int accumulate;
    float* partials;                     // [gridDim.x], may be null
};

__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
// sum over every device bound to the multicast object, added inside the switch (fp32 accumulation for bf16 pairs)
__device__ __forceinline__ uint4 ld_reduce_bf16x8(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_reduce_f32x4(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

template <bool BF16>
__device__ __forceinline__ void add_vec(float (&acc)[8], const uint4& v) {
    if constexpr (BF16) {
        float2 f;
        f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
        f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
        f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
        f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
    } else {
        acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
        acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
    }
}

// BF16: gradient dtype (else fp32).  MC: one multimem.ld_reduce per vector instead of `world` loads.
// U vectors of 16 bytes per thread and source are in flight at once; MAXR bounds the number of ranks, so that a
// small group spends its registers on more vectors per source (U * MAXR = 16 loads in flight per thread).
template <bool BF16, bool MC, int U, int MAXR>
__global__ void __launch_bounds__(256) reduce_scatter_peers_kernel(const __grid_constant__ RsPeerArgs a) {
    __shared__ float red[32];
    __shared__ int ok_s;
    constexpr int VEC = BF16 ? 8 : 4;
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) {
            __threadfence_system();
            for (int p = 0; p < a.world; ++p)
                if (p != a.rank) st_release_sys(&a.pad[p][PAD_SIG + a.rank], a.seq);
        }
        int ok = 1;
        for (int i = 1; i < a.world && ok; ++i) {
            const int p = (a.rank + i) % a.world;
            ok = wait_flag_sys(&a.pad[a.rank][PAD_SIG + p], a.seq, 860 + p) ? 1 : 0;
        }
        ok_s = ok;
    }
    __syncthreads();
    if (!ok_s) {   // a peer never announced its buffer: the status word is set, nothing is read or written
        if (threadIdx.x == 0 && a.partials != nullptr) a.partials[blockIdx.x] = 0.f;
        return;
    }
    const long long nvec = a.n / VEC;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    float ss = 0.f;
    for (long long base = tid; base < nvec; base += nthreads * U) {
        float acc[U][8];
#pragma unroll
        for (int j = 0; j < U; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
        if constexpr (MC) {
            uint4 v[U];
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const long long i = base + j * nthreads;
                if (i < nvec) {
                    const uint8_t* p = static_cast<const uint8_t*>(a.mc_src) + i * 16;
                    v[j] = BF16 ? ld_reduce_bf16x8(p) : ld_reduce_f32x4(p);
                } else {
                    v[j] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (int j = 0; j < U; ++j) add_vec<BF16>(acc[j], v[j]);
        } else {
            uint4 v[U][MAXR];
#pragma unroll
            for (int j = 0; j < U; ++j) {
                const long long i = base + j * nthreads;
#pragma unroll
                for (int r = 0; r < MAXR; ++r) {
                    if (r < a.world && i < nvec)
                        v[j][r] = ld_peer_v4(static_cast<const uint8_t*>(a.src[r]) + i * 16);
                    else
                        v[j][r] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (int j = 0; j < U; ++j)
#pragma unroll
                for (int r = 0; r < MAXR; ++r)   // rank order: the sum does not depend on timing
                    if (r < a.world) add_vec<BF16>(acc[j], v[j][r]);
        }
#pragma unroll
        for (int j = 0; j < U; ++j) {
            const long long i = base + j * nthreads;
            if (i >= nvec) continue;
            float f[8];
#pragma unroll
            for (int e = 0; e < VEC; ++e) f[e] = acc[j][e] * a.scale;
            if constexpr (BF16) {
                __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.out) + i * 8;
                if (a.accumulate) {
                    const uint4 old = *reinterpret_cast<const uint4*>(o);
                    float2 g;
                    g = unpack_bf16x2(old.x); f[0] += g.x; f[1] += g.y;
                    g = unpack_bf16x2(old.y); f[2] += g.x; f[3] += g.y;
                    g = unpack_bf16x2(old.z); f[4] += g.x; f[5] += g.y;
                    g = unpack_bf16x2(old.w); f[6] += g.x; f[7] += g.y;
                }
                uint4 w;
                w.x = pack_bf16x2(f[0], f[1]); w.y = pack_bf16x2(f[2], f[3]);
                w.z = pack_bf16x2(f[4], f[5]); w.w = pack_bf16x2(f[6], f[7]);
                *reinterpret_cast<uint4*>(o) = w;
                // the norm is taken of the values that the optimizer will read (after rounding)
                float2 g;
                g = unpack_bf16x2(w.x); ss += g.x * g.x + g.y * g.y;
                g = unpack_bf16x2(w.y); ss += g.x * g.x + g.y * g.y;
                g = unpack_bf16x2(w.z); ss += g.x * g.x + g.y * g.y;
                g = unpack_bf16x2(w.w); ss += g.x * g.x + g.y * g.y;
            } else {
                float* o = static_cast<float*>(a.out) + i * 4;
                if (a.accumulate) {
                    const float4 old = *reinterpret_cast<const float4*>(o);
                    f[0] += old.x; f[1] += old.y; f[2] += old.z; f[3] += old.w;
                }
                *reinterpret_cast<float4*>(o) = make_float4(f[0], f[1], f[2], f[3]);
                ss += f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
            }
        }
    }
    if (a.partials != nullptr) {
        ss = block_sum(ss, red);
        if (threadIdx.x == 0) a.partials[blockIdx.x] = ss;
    }
}

}  // namespace lme

using namespace lme;

// n (elements of this rank's shard) must be a multiple of 8 (bf16) / 4 (fp32); every pointer 16-byte aligned.
// src[r] / pads[r]: rank r's copy of the slice / signal pad as mapped into this process ([rank] local).
// mc_src: multicast mapping of the slice or null.  partials: `ctas` floats or null.  ctas <= 1184.
extern "C" int lme_reduce_scatter_peers(const void* const* src, int* const* pads, const void* mc_src, int rank,
                                        int world, int seq, void* out, long long n, int is_bf16, float scale,
                                        int accumulate, float* partials, int ctas, void* stream) {
    if (world < 1 || world > GATHER_MAX_RANKS || rank < 0 || rank >= world || n < 0 || (n % (is_bf16 ? 8 : 4)))
        return LME_ERR_SHAPE;
    if (ctas < 1 || ctas > 1184) return LME_ERR_SHAPE;
    RsPeerArgs a;
    for (int r = 0; r < GATHER_MAX_RANKS; ++r) {
        a.src[r] = r < world ? src[r] : nullptr;
        a.pad[r] = r < world ? pads[r] : nullptr;
        if (r < world && (reinterpret_cast<uintptr_t>(src[r]) & 15)) return LME_ERR_ALIGN;
    }
    if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(mc_src)) & 15) return LME_ERR_ALIGN;
    a.mc_src = mc_src;
    a.rank = rank; a.world = world; a.seq = seq;
    a.out = out; a.n = n; a.scale = scale; a.accumulate = accumulate; a.partials = partials;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LME_RS_LAUNCH(MC_, U_, R_)                                                                      \
    do {                                                                                                \
        if (is_bf16) reduce_scatter_peers_kernel<true, MC_, U_, R_><<<ctas, 256, 0, st>>>(a);           \
        else reduce_scatter_peers_kernel<false, MC_, U_, R_><<<ctas, 256, 0, st>>>(a);                  \
    } while (0)
    if (mc_src != nullptr) LME_RS_LAUNCH(true, 8, 1);
    else if (world <= 2) LME_RS_LAUNCH(false, 8, 2);
    else if (world <= 4) LME_RS_LAUNCH(false, 4, 4);
    else LME_RS_LAUNCH(false, 2, 8);
#undef LME_RS_LAUNCH
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

// out[0] (+)= sum(partials[0 .. n)) in a fixed order (one CTA)
extern "C" int lme_sum_partials(const float* partials, int n, float* out, int accumulate, void* stream) {
    if (n < 0) return LME_ERR_SHAPE;
    sum_partials_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(partials, n, out, accumulate);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

// Limit of the waits on words that ANOTHER GPU writes (default 2 s).  A training job raises it: ranks drift apart by
// more than that around evaluation, checkpoints and first-step allocations.
extern "C" int lme_set_peer_wait_limit_ms(long long ms) {
    if (ms < 1) return LME_ERR_SHAPE;
    const unsigned long long ns = static_cast<unsigned long long>(ms) * 1000000ull;
    return cudaMemcpyToSymbol(lme_peer_wait_ns, &ns, sizeof(ns)) == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
