// Tensor-wise dynamically scaled FP8 casts for the 8-bit GEMM path.
//
//   amax      : max |x| over a bf16 tensor, accumulated with an integer atomicMax (non-negative floats order like
//               their bit patterns), so several tensors / launches can share one cell
//   quantize  : q = sat(x * fmax / amax) as e4m3 (fmax 448) or e5m2 (fmax 57344), row-major and, optionally, its
//               transpose in the same pass (the backward GEMMs contract over the other axis and the tensor core
//               reads 8-bit operands K-major only); also writes the de-quantisation scale amax / fmax
//
// Plays the role of torchao's tensor-wise dynamic casts used by the reference (lm_engine/fp8.py:53-75).
#include <cuda_fp8.h>

namespace lme {

__global__ void fp8_amax_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ amax) {
    __shared__ float red[32];
    float m = 0.f;
    const long long n8 = n / 8;
    const uint4* x8 = reinterpret_cast<const uint4*>(x);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        uint4 v = x8[i];
        float2 f;
        f = unpack_bf16x2(v.x); m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
        f = unpack_bf16x2(v.y); m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
        f = unpack_bf16x2(v.z); m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
        f = unpack_bf16x2(v.w); m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (long long i = n8 * 8; i < n; ++i) m = fmaxf(m, fabsf(__bfloat162float(x[i])));
    m = block_max(m, red);
    if (threadIdx.x == 0 && m > 0.f && isfinite(m)) atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));
}

template <bool E5M2>
__device__ __forceinline__ uint32_t cvt4(float a, float b, float c, float d) {
    constexpr __nv_fp8_interpretation_t kind = E5M2 ? __NV_E5M2 : __NV_E4M3;
    uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
    uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, kind);
    return lo | (hi << 16);
}

// One block = one 64 x 64 tile; thread t handles row t / 4, columns (t % 4) * 16 .. + 16.
template <bool E5M2, bool TRANSPOSE>
__global__ void __launch_bounds__(256)
fp8_quantize_kernel(const __nv_bfloat16* __restrict__ x, int rows, int cols, long long ldx,
                    const float* __restrict__ amax, uint8_t* __restrict__ q, long long ldq,
                    uint8_t* __restrict__ qt, long long ldqt, float* __restrict__ scale_inv) {
    __shared__ __align__(16) uint8_t tile[64][64 + 16];
    constexpr float FMAX = E5M2 ? 57344.f : 448.f;
    const float a = fmaxf(__ldg(amax), 1e-12f);
    const float scale = FMAX / a;
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *scale_inv = a / FMAX;
    const int r = blockIdx.y * 64 + (threadIdx.x >> 2);
    const int c = blockIdx.x * 64 + (threadIdx.x & 3) * 16;
    uint4 out = make_uint4(0, 0, 0, 0);
    if (r < rows && c < cols) {   // cols % 16 == 0: a 16-wide segment is entirely inside or outside
        const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ldx + c);
        uint4 v0 = src[0], v1 = src[1];
        float2 f0, f1;
        f0 = unpack_bf16x2(v0.x); f1 = unpack_bf16x2(v0.y);
        out.x = cvt4<E5M2>(f0.x * scale, f0.y * scale, f1.x * scale, f1.y * scale);
        f0 = unpack_bf16x2(v0.z); f1 = unpack_bf16x2(v0.w);
        out.y = cvt4<E5M2>(f0.x * scale, f0.y * scale, f1.x * scale, f1.y * scale);
        f0 = unpack_bf16x2(v1.x); f1 = unpack_bf16x2(v1.y);
        out.z = cvt4<E5M2>(f0.x * scale, f0.y * scale, f1.x * scale, f1.y * scale);
        f0 = unpack_bf16x2(v1.z); f1 = unpack_bf16x2(v1.w);
        out.w = cvt4<E5M2>(f0.x * scale, f0.y * scale, f1.x * scale, f1.y * scale);
        if (q != nullptr) *reinterpret_cast<uint4*>(q + (long long)r * ldq + c) = out;
    }
    if (TRANSPOSE) {
        *reinterpret_cast<uint4*>(&tile[threadIdx.x >> 2][(threadIdx.x & 3) * 16]) = out;
        __syncthreads();
        // thread t writes transposed row (t / 4) = source column, 16 source rows starting at (t % 4) * 16
        const int tc = threadIdx.x >> 2, tr0 = (threadIdx.x & 3) * 16;
        const int oc = blockIdx.x * 64 + tc;        // row of the transposed output
        const int orow0 = blockIdx.y * 64 + tr0;    // column of the transposed output
        if (oc < cols && orow0 < rows) {            // rows % 16 == 0 is enforced on the host
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w[j] = (uint32_t)tile[tr0 + 4 * j][tc] | ((uint32_t)tile[tr0 + 4 * j + 1][tc] << 8) |
                       ((uint32_t)tile[tr0 + 4 * j + 2][tc] << 16) | ((uint32_t)tile[tr0 + 4 * j + 3][tc] << 24);
            }
            *reinterpret_cast<uint4*>(qt + (long long)oc * ldqt + orow0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

}  // namespace lme

using namespace lme;

// amax must hold 0 (or the running maximum of earlier tensors sharing the cell) on entry
extern "C" int lme_fp8_amax(const void* x, long long n, float* amax, void* stream) {
    if (n <= 0) return LME_OK;
    if (reinterpret_cast<uintptr_t>(x) & 15) return LME_ERR_ALIGN;
    long long blocks = (n / 8 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
    fp8_amax_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), n, amax);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

// fmt: 0 = e4m3, 1 = e5m2.  q ([rows, cols], pitch ldq) and / or qt ([cols, rows], pitch ldqt) may be null.
extern "C" int lme_fp8_quantize(const void* x, int rows, int cols, long long ldx, const float* amax, int fmt, void* q,
                                long long ldq, void* qt, long long ldqt, float* scale_inv, void* stream) {
    if (rows <= 0 || cols <= 0) return LME_OK;
    if ((cols % 16) || (ldx % 8) || (q && (ldq % 16)) || (qt && ((rows % 16) || (ldqt % 16)))) return LME_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(qt)) & 15)
        return LME_ERR_ALIGN;
    dim3 grid((cols + 63) / 64, (rows + 63) / 64);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto X = static_cast<const __nv_bfloat16*>(x);
    auto Q = static_cast<uint8_t*>(q);
    auto QT = static_cast<uint8_t*>(qt);
#define LME_Q(E, T) fp8_quantize_kernel<E, T><<<grid, 256, 0, st>>>(X, rows, cols, ldx, amax, Q, ldq, QT, ldqt, scale_inv)
    if (fmt == 1) { if (qt) LME_Q(true, true); else LME_Q(true, false); }
    else { if (qt) LME_Q(false, true); else LME_Q(false, false); }
#undef LME_Q
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
