// Mamba-2 SSD, intra-chunk part: y[l] = sum_{s <= l} exp(cum[l] - cum[s]) (C_l . B_s) xdt[s] per head and chunk.
//
//   ssd_decay_matrix : M[b,c,n,l,s] = CB[b,c,g(n),l,s] * exp(cum[b,c,n,l] - cum[b,c,n,s]) for s <= l, else 0   (bf16)
//                      -- one pass that replaces the difference / mask / exp / repeat / multiply chain over
//                      [chunks, heads, L, L] fp32 tensors; y = M @ xdt then runs on the tensor cores as a batched GEMM
//   ssd_dcb          : dCB[b,c,g,l,s] = sum_{n in g} dM[b,c,n,l,s] * exp(cum[n,l] - cum[n,s]) for s <= l
//                      -- one warp per (b, c, g, l) row loops over the heads of the group: no atomics
// The gradient with respect to cum needs no L x L pass: sum_s dM[l,s] M[l,s] = dy[l] . y[l] and
// sum_l dM[l,s] M[l,s] = xdt[s] . dxdt[s] (both are products of the same three factors), evaluated by the caller.
// Role of the chunk-scan kernels of mamba_ssm used by the reference
// (lm_engine/modeling_utils/sequence_mixer_blocks/mamba2/op.py:385-457).
namespace lme {

// grid.x covers (b*c*n) * L rows * (L/8) vectors
__global__ void __launch_bounds__(256)
ssd_decay_matrix_kernel(const __nv_bfloat16* __restrict__ cb, const float* __restrict__ cum,
                        __nv_bfloat16* __restrict__ m, long long heads_total, int N, int G, int L) {
    const int vec_per_row = L / 8;
    const long long total = heads_total * L * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int v = static_cast<int>(i % vec_per_row);
        long long rest = i / vec_per_row;
        const int l = static_cast<int>(rest % L);
        const long long head = rest / L;                 // (b*nc + c) * N + n
        const int n = static_cast<int>(head % N);
        const long long bc = head / N;
        const int s0 = v * 8;
        float out[8];
        if (s0 > l) {
#pragma unroll
            for (int j = 0; j < 8; ++j) out[j] = 0.f;
        } else {
            const int g = n / (N / G);
            float c8[8];
            load8(cb + ((bc * G + g) * L + l) * L + s0, c8);
            const float* cu = cum + head * L;
            const float cl = cu[l];
            const float4 a = *reinterpret_cast<const float4*>(cu + s0);
            const float4 b = *reinterpret_cast<const float4*>(cu + s0 + 4);
            const float cs[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) out[j] = (s0 + j <= l) ? c8[j] * __expf(cl - cs[j]) : 0.f;
        }
        store8(m + (head * L + l) * L + s0, out);
    }
}

// one warp per (bc, g, l); block = 8 warps
template <int MAXV>
__global__ void __launch_bounds__(256)
ssd_dcb_kernel(const __nv_bfloat16* __restrict__ dm, const float* __restrict__ cum, __nv_bfloat16* __restrict__ dcb,
               long long rows_total, int N, int G, int L) {
    const int lane = threadIdx.x & 31;
    const long long row = blockIdx.x * 8ll + (threadIdx.x >> 5);   // (bc * G + g) * L + l
    if (row >= rows_total) return;
    const int l = static_cast<int>(row % L);
    const long long bcg = row / L;
    const int g = static_cast<int>(bcg % G);
    const long long bc = bcg / G;
    const int rep = N / G;
    const int nvec = L / 8;
    float acc[MAXV][8];
#pragma unroll
    for (int k = 0; k < MAXV; ++k)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
    for (int r = 0; r < rep; ++r) {
        const long long head = bc * N + g * rep + r;
        const float* cu = cum + head * L;
        const float cl = cu[l];
        const __nv_bfloat16* drow = dm + (head * L + l) * L;
#pragma unroll
        for (int k = 0; k < MAXV; ++k) {
            const int v = lane + 32 * k;
            const int s0 = v * 8;
            if (v < nvec && s0 <= l) {
                float d8[8];
                load8(drow + s0, d8);
                const float4 a = *reinterpret_cast<const float4*>(cu + s0);
                const float4 b = *reinterpret_cast<const float4*>(cu + s0 + 4);
                const float cs[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (s0 + j <= l) acc[k][j] += d8[j] * __expf(cl - cs[j]);
            }
        }
    }
    __nv_bfloat16* orow = dcb + row * L;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
        const int v = lane + 32 * k;
        if (v < nvec) store8(orow + v * 8, acc[k]);
    }
}

}  // namespace lme

using namespace lme;

// cb [BC, G, L, L] bf16, cum [BC, N, L] fp32 (inclusive cumulative sums of dt * A inside the chunk) -> m [BC, N, L, L]
extern "C" int lme_ssd_decay_matrix(const void* cb, const float* cum, void* m, long long BC, int N, int G, int L,
                                    void* stream) {
    if (BC <= 0) return LME_OK;
    if (L % 8 || N % G || L > 1024) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(cb) | reinterpret_cast<uintptr_t>(cum) | reinterpret_cast<uintptr_t>(m)) & 15)
        return LME_ERR_ALIGN;
    const long long heads = BC * N;
    const long long total = heads * L * (L / 8);
    ssd_decay_matrix_kernel<<<grid_for(total, 256, 148 * 32), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(cb), cum, static_cast<__nv_bfloat16*>(m), heads, N, G, L);
    return LME_LAUNCH_OK();
}

// dm [BC, N, L, L] bf16, cum [BC, N, L] fp32 -> dcb [BC, G, L, L] bf16
extern "C" int lme_ssd_dcb(const void* dm, const float* cum, void* dcb, long long BC, int N, int G, int L,
                           void* stream) {
    if (BC <= 0) return LME_OK;
    if (L % 8 || N % G || L > 1024) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(dm) | reinterpret_cast<uintptr_t>(cum) | reinterpret_cast<uintptr_t>(dcb)) & 15)
        return LME_ERR_ALIGN;
    const long long rows = BC * G * L;
    const unsigned int grid = static_cast<unsigned int>((rows + 7) / 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto DM = static_cast<const __nv_bfloat16*>(dm);
    auto DC = static_cast<__nv_bfloat16*>(dcb);
    if (L <= 256) ssd_dcb_kernel<1><<<grid, 256, 0, st>>>(DM, cum, DC, rows, N, G, L);
    else if (L <= 512) ssd_dcb_kernel<2><<<grid, 256, 0, st>>>(DM, cum, DC, rows, N, G, L);
    else ssd_dcb_kernel<4><<<grid, 256, 0, st>>>(DM, cum, DC, rows, N, G, L);
    return LME_LAUNCH_OK();
}
