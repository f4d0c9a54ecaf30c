// Depthwise causal convolution over channel-last activations (Mamba-2 / gated delta net short convolutions):
//   z[b, t, c] = bias[c] + sum_j w[c, j] * x[b, t - (K-1) + j, c],   y = silu(z) or z,   K <= 8
// with x[b, t < 0, c] taken from init[b, c, K-1+t] (or 0).  One thread owns 8 channels (one 16-byte vector) and a
// run of CHUNK time steps and slides a register window over it, so every x element is read once (+ K-1 halo rows per
// chunk) and consecutive threads touch consecutive channels (fully coalesced rows).
// Backward recomputes z (nothing but x is saved), forms dz = dy * act'(z), and produces dx (needs dz of the next K-1
// steps: a forward halo), the gradient of the initial state, and per-thread partial sums of dw / dbias that are
// added atomically into fp32 accumulators.
// Role of causal_conv1d_fn / causal_conv1d_update in the reference
// (lm_engine/modeling_utils/depthwise_causal_convolution.py:110-206).
namespace lme {

static constexpr int CONV_MAX_K = 8;
static constexpr int CONV_CHUNK = 32;

__device__ __forceinline__ void conv_load_row(const __nv_bfloat16* x, const __nv_bfloat16* init, long long b, int t,
                                              int S, int C, int K, int c, float (&out)[8]) {
    if (t >= 0) {
        if (t < S) load8(x + (b * S + t) * C + c, out);
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] = 0.f;
        }
    } else if (init != nullptr) {
        // init [B, C, K-1]: element (c + i, K-1+t)
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = __bfloat162float(init[(b * C + c + i) * (K - 1) + (K - 1 + t)]);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = 0.f;
    }
}

// EXACT: the filter has exactly KM taps, so every `j < K` test and tap select below folds at compile time
template <int KM, bool EXACT>
__global__ void __launch_bounds__(128)
causal_conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ init,
                         __nv_bfloat16* __restrict__ y, int B, int S, int C, int K_, int silu) {
    const int K = EXACT ? KM : K_;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int t0 = blockIdx.y * CONV_CHUNK;
    const long long b = blockIdx.z;
    float wv[KM][8], bv[8], win[KM][8];
#pragma unroll
    for (int j = 0; j < KM; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[j][i] = j < K ? __bfloat162float(w[(c + i) * K + j]) : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) bv[i] = bias != nullptr ? __bfloat162float(bias[c + i]) : 0.f;
    // window slots 0 .. K-2 hold x[t - (K-1)] .. x[t - 1]
#pragma unroll
    for (int j = 0; j < KM - 1; ++j)
        if (j < K - 1) conv_load_row(x, init, b, t0 - (K - 1) + j, S, C, K, c, win[j]);
    const int t1 = min(t0 + CONV_CHUNK, S);
    for (int t = t0; t < t1; ++t) {
        float cur[8], z[8];
        load8(x + (b * S + t) * C + c, cur);
#pragma unroll
        for (int i = 0; i < 8; ++i) z[i] = bv[i];
#pragma unroll
        for (int j = 0; j < KM - 1; ++j)
            if (j < K - 1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) z[i] += wv[j][i] * win[j][i];
            }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float wk = 0.f;
#pragma unroll
            for (int j = 0; j < KM; ++j) wk = (j == K - 1) ? wv[j][i] : wk;
            z[i] += wk * cur[i];
            if (silu) z[i] = silu_f(z[i]);
        }
        store8(y + (b * S + t) * C + c, z);
#pragma unroll
        for (int j = 0; j < KM - 2; ++j)
            if (j < K - 2) {
#pragma unroll
                for (int i = 0; i < 8; ++i) win[j][i] = win[j + 1][i];
            }
#pragma unroll
        for (int j = 0; j < KM - 1; ++j)
            if (j == K - 2) {
#pragma unroll
                for (int i = 0; i < 8; ++i) win[j][i] = cur[i];
            }
    }
}

// dz at time t for the thread's 8 channels (0 outside [0, S))
template <int KM>
__device__ __forceinline__ void conv_dz(const __nv_bfloat16* x, const __nv_bfloat16* init, const __nv_bfloat16* dy,
                                        const float (&wv)[KM][8], const float (&bv)[8], long long b, int t,
                                        int S, int C, int K, int c, int silu, float (&dz)[8]) {
    if (t < 0 || t >= S) {
#pragma unroll
        for (int i = 0; i < 8; ++i) dz[i] = 0.f;
        return;
    }
    float z[8], g[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) z[i] = bv[i];
    for (int j = 0; j < K; ++j) {
        float xr[8];
        conv_load_row(x, init, b, t - (K - 1) + j, S, C, K, c, xr);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float wj = 0.f;
#pragma unroll
            for (int jj = 0; jj < KM; ++jj) wj = (jj == j) ? wv[jj][i] : wj;
            z[i] += wj * xr[i];
        }
    }
    load8(dy + (b * S + t) * C + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (silu) {
            const float sg = 1.f / (1.f + __expf(-z[i]));
            dz[i] = g[i] * sg * (1.f + z[i] * (1.f - sg));
        } else {
            dz[i] = g[i];
        }
    }
}

template <int KM, bool EXACT>
__global__ void __launch_bounds__(128)
causal_conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ init,
                         const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                         float* __restrict__ dw, float* __restrict__ dbias, float* __restrict__ dinit, int B, int S,
                         int C, int K_, int silu) {
    const int K = EXACT ? KM : K_;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int t0 = blockIdx.y * CONV_CHUNK;
    const long long b = blockIdx.z;
    float wv[KM][8], bv[8];
#pragma unroll
    for (int j = 0; j < KM; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[j][i] = j < K ? __bfloat162float(w[(c + i) * K + j]) : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) bv[i] = bias != nullptr ? __bfloat162float(bias[c + i]) : 0.f;
    float dwacc[KM][8], dbacc[8];
#pragma unroll
    for (int j = 0; j < KM; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) dbacc[i] = 0.f;
    // dzw slot j holds dz[t + j]; dx[t] = sum_j w[K-1-j] * dz[t + j]
    float dzw[KM][8];
#pragma unroll
    for (int j = 0; j < KM; ++j)
        if (j < K) conv_dz<KM>(x, init, dy, wv, bv, b, t0 + j, S, C, K, c, silu, dzw[j]);
    const int t1 = min(t0 + CONV_CHUNK, S);
    for (int t = t0; t < t1; ++t) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = 0.f;
#pragma unroll
        for (int j = 0; j < KM; ++j)
            if (j < K) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float wr = 0.f;
#pragma unroll
                    for (int jj = 0; jj < KM; ++jj) wr = (jj == K - 1 - j) ? wv[jj][i] : wr;
                    o[i] += wr * dzw[j][i];
                }
            }
        store8(dx + (b * S + t) * C + c, o);
        // weight / bias gradients of output step t (dz[t] = slot 0) against its K inputs
        for (int j = 0; j < K; ++j) {
            float xr[8];
            conv_load_row(x, init, b, t - (K - 1) + j, S, C, K, c, xr);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int jj = 0; jj < KM; ++jj)
                    if (jj == j) dwacc[jj][i] += dzw[0][i] * xr[i];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) dbacc[i] += dzw[0][i];
        // slide: slot j <- slot j + 1, new last slot = dz[t + K]
#pragma unroll
        for (int j = 0; j < KM - 1; ++j)
            if (j < K - 1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) dzw[j][i] = dzw[j + 1][i];
            }
        float nxt[8];
        conv_dz<KM>(x, init, dy, wv, bv, b, t + K, S, C, K, c, silu, nxt);
#pragma unroll
        for (int j = 0; j < KM; ++j)
            if (j == K - 1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) dzw[j][i] = nxt[i];
            }
    }
    for (int j = 0; j < K; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float v = 0.f;
#pragma unroll
            for (int jj = 0; jj < KM; ++jj) v = (jj == j) ? dwacc[jj][i] : v;
            atomicAdd(&dw[(c + i) * K + j], v);
        }
    if (dbias != nullptr)
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(&dbias[c + i], dbacc[i]);
    // gradient of the initial state: x at time s = i - (K-1) (i = 0 .. K-2) feeds output t = s + (K-1) - j, t >= 0
    if (dinit != nullptr && blockIdx.y == 0) {
        for (int i = 0; i < K - 1; ++i) {
            float acc[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[q] = 0.f;
            for (int j = 0; j <= i; ++j) {
                float dz[8];
                conv_dz<KM>(x, init, dy, wv, bv, b, i - j, S, C, K, c, silu, dz);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float wj = 0.f;
#pragma unroll
                    for (int jj = 0; jj < KM; ++jj) wj = (jj == j) ? wv[jj][q] : wj;
                    acc[q] += wj * dz[q];
                }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q) dinit[(b * C + c + q) * (K - 1) + i] = acc[q];
        }
    }
}

}  // namespace lme

using namespace lme;

extern "C" int lme_causal_conv1d_fwd(const void* x, const void* w, const void* bias, const void* init, void* y, int B,
                                     int S, int C, int K, int silu, void* stream) {
    if (B <= 0 || S <= 0 || C <= 0) return LME_OK;
    if (C % 8 || K < 1 || K > CONV_MAX_K) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) return LME_ERR_ALIGN;
    dim3 grid((C / 8 + 127) / 128, (S + CONV_CHUNK - 1) / CONV_CHUNK, B);
    auto X = static_cast<const __nv_bfloat16*>(x);
    auto W = static_cast<const __nv_bfloat16*>(w);
    auto BI = static_cast<const __nv_bfloat16*>(bias);
    auto IN = static_cast<const __nv_bfloat16*>(init);
    auto Y = static_cast<__nv_bfloat16*>(y);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K == 4) causal_conv1d_fwd_kernel<4, true><<<grid, 128, 0, st>>>(X, W, BI, IN, Y, B, S, C, K, silu);
    else if (K < 4) causal_conv1d_fwd_kernel<4, false><<<grid, 128, 0, st>>>(X, W, BI, IN, Y, B, S, C, K, silu);
    else causal_conv1d_fwd_kernel<CONV_MAX_K, false><<<grid, 128, 0, st>>>(X, W, BI, IN, Y, B, S, C, K, silu);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

// dw [C, K], dbias [C] (may be null), dinit [B, C, K-1] (may be null) are fp32; dw / dbias must be zeroed by the caller
// (they are accumulated atomically), dinit is written.
extern "C" int lme_causal_conv1d_bwd(const void* x, const void* w, const void* bias, const void* init, const void* dy,
                                     void* dx, float* dw, float* dbias, float* dinit, int B, int S, int C, int K,
                                     int silu, void* stream) {
    if (B <= 0 || S <= 0 || C <= 0) return LME_OK;
    if (C % 8 || K < 1 || K > CONV_MAX_K) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15)
        return LME_ERR_ALIGN;
    dim3 grid((C / 8 + 127) / 128, (S + CONV_CHUNK - 1) / CONV_CHUNK, B);
    auto X = static_cast<const __nv_bfloat16*>(x);
    auto W = static_cast<const __nv_bfloat16*>(w);
    auto BI = static_cast<const __nv_bfloat16*>(bias);
    auto IN = static_cast<const __nv_bfloat16*>(init);
    auto DY = static_cast<const __nv_bfloat16*>(dy);
    auto DX = static_cast<__nv_bfloat16*>(dx);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K == 4)
        causal_conv1d_bwd_kernel<4, true><<<grid, 128, 0, st>>>(X, W, BI, IN, DY, DX, dw, dbias, dinit, B, S, C, K, silu);
    else if (K < 4)
        causal_conv1d_bwd_kernel<4, false><<<grid, 128, 0, st>>>(X, W, BI, IN, DY, DX, dw, dbias, dinit, B, S, C, K, silu);
    else
        causal_conv1d_bwd_kernel<CONV_MAX_K, false><<<grid, 128, 0, st>>>(X, W, BI, IN, DY, DX, dw, dbias, dinit, B, S, C,
                                                                          K, silu);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
