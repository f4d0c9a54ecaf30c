// Token movement of mixture-of-experts layers, all in terms of slot[t, k] = row of the padded per-expert layout that
// holds the k-th expert assignment of token t.  Every padded row is written by exactly one (t, k), every token reads
// its own k rows, so neither direction needs atomics and both are deterministic.
//
//   scatter_rows   : dst[slot[t, k]] = (w ? w[t, k] : 1) * src[t]             dispatch; backward of combine
//   gather_reduce  : dst[t] = sum_k (w ? w[t, k] : 1) * src[slot[t, k]]       combine;  backward of dispatch
//   row_dots       : out[t, k] = <a[slot[t, k]], b[t]>                        gradient of the combine weights
//
// bf16 rows of H elements (H % 8 == 0), fp32 accumulation; one thread block per token.
// Role of ScatterMoE's fused gather / scatter-combine in the reference
// (lm_engine/modeling_utils/mlp_blocks/moe/experts.py:137-149,212-225); here the GEMM stays separate and reads the
// padded layout with TMA.
namespace lme {

__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ slot,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ dst, int H, int K) {
    const int t = blockIdx.x;
    const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<long long>(t) * H);
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        const uint4 v = s[c];
        const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
        for (int k = 0; k < K; ++k) {
            const int row = __ldg(&slot[t * K + k]);
            if (row < 0) continue;
            uint4 o = v;
            if (w != nullptr) {
                const float g = __bfloat162float(w[t * K + k]);
                o.x = pack_bf16x2(f0.x * g, f0.y * g); o.y = pack_bf16x2(f1.x * g, f1.y * g);
                o.z = pack_bf16x2(f2.x * g, f2.y * g); o.w = pack_bf16x2(f3.x * g, f3.y * g);
            }
            reinterpret_cast<uint4*>(dst + static_cast<long long>(row) * H)[c] = o;
        }
    }
}

__global__ void __launch_bounds__(256)
moe_gather_reduce_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ slot,
                         const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ dst, int H, int K) {
    const int t = blockIdx.x;
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < K; ++k) {
            const int row = __ldg(&slot[t * K + k]);
            if (row < 0) continue;
            const float g = w != nullptr ? __bfloat162float(w[t * K + k]) : 1.0f;
            const uint4 v = reinterpret_cast<const uint4*>(src + static_cast<long long>(row) * H)[c];
            float2 f;
            f = unpack_bf16x2(v.x); acc[0] += g * f.x; acc[1] += g * f.y;
            f = unpack_bf16x2(v.y); acc[2] += g * f.x; acc[3] += g * f.y;
            f = unpack_bf16x2(v.z); acc[4] += g * f.x; acc[5] += g * f.y;
            f = unpack_bf16x2(v.w); acc[6] += g * f.x; acc[7] += g * f.y;
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(dst + static_cast<long long>(t) * H)[c] = o;
    }
}

__global__ void __launch_bounds__(256)
moe_row_dots_kernel(const __nv_bfloat16* __restrict__ a, const int* __restrict__ slot,
                    const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ out, int H, int K) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const uint4* bt = reinterpret_cast<const uint4*>(b + static_cast<long long>(t) * H);
    for (int k = 0; k < K; ++k) {
        const int row = __ldg(&slot[t * K + k]);
        float acc = 0.f;
        if (row >= 0) {
            const uint4* ar = reinterpret_cast<const uint4*>(a + static_cast<long long>(row) * H);
            for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
                const uint4 x = ar[c], y = bt[c];
                float2 p, q;
                p = unpack_bf16x2(x.x); q = unpack_bf16x2(y.x); acc += p.x * q.x + p.y * q.y;
                p = unpack_bf16x2(x.y); q = unpack_bf16x2(y.y); acc += p.x * q.x + p.y * q.y;
                p = unpack_bf16x2(x.z); q = unpack_bf16x2(y.z); acc += p.x * q.x + p.y * q.y;
                p = unpack_bf16x2(x.w); q = unpack_bf16x2(y.w); acc += p.x * q.x + p.y * q.y;
            }
        }
        acc = block_sum(acc, red);
        if (threadIdx.x == 0) out[t * K + k] = __float2bfloat16(acc);
    }
}

}  // namespace lme

using namespace lme;

static int moe_check(const void* a, const void* b, int T, int H, int K) {
    if (T < 0 || K <= 0 || H <= 0 || (H % 8)) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) return LME_ERR_ALIGN;
    return LME_OK;
}

extern "C" int lme_moe_scatter_rows(const void* src, const int* slot, const void* w, void* dst, int T, int H, int K,
                                    void* stream) {
    int rc = moe_check(src, dst, T, H, K);
    if (rc || T == 0) return rc;
    moe_scatter_rows_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(src), slot, static_cast<const __nv_bfloat16*>(w),
        static_cast<__nv_bfloat16*>(dst), H, K);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_moe_gather_reduce(const void* src, const int* slot, const void* w, void* dst, int T, int H, int K,
                                     void* stream) {
    int rc = moe_check(src, dst, T, H, K);
    if (rc || T == 0) return rc;
    moe_gather_reduce_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(src), slot, static_cast<const __nv_bfloat16*>(w),
        static_cast<__nv_bfloat16*>(dst), H, K);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_moe_row_dots(const void* a, const int* slot, const void* b, void* out, int T, int H, int K,
                                void* stream) {
    int rc = moe_check(a, b, T, H, K);
    if (rc || T == 0) return rc;
    moe_row_dots_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(a), slot, static_cast<const __nv_bfloat16*>(b),
        static_cast<__nv_bfloat16*>(out), H, K);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
