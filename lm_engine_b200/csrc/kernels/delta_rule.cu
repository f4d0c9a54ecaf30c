// Inter-chunk chain of the gated delta rule (forward and backward): the only sequential part of the chunk-parallel
// algorithm.  With the per-chunk operands prepared for all chunks at once (W_k, W_v from the unit-triangular solve,
// the decayed queries Q_e, the decayed keys K_e, the masked decayed Q K^T, the chunk decay a), the state h [K, V]
// obeys
//     U_c     = W_v,c - W_k,c h_c                     [L, V]
//     y_c     = Q_e,c h_c + QK_c U_c                  [L, V]
//     h_{c+1} = a_c h_c + K_e,c^T U_c                 [K, V]
// and the reverse chain for the gradients
//     dU_c = QK_c^T dy_c + K_e,c dh_{c+1}             dh_c = a_c dh_{c+1} + Q_e,c^T dy_c - W_k,c^T dU_c
// (the parameter gradients are batched GEMMs over all chunks on what the two kernels leave behind: U_c, dU_c, the
// state entering each chunk and the gradient leaving it).
//
// The columns of h are independent, so a CTA owns VS = 64 (or 32, when that is needed to fill the GPU) columns of one
// (batch, head) and walks the chunks alone.  The
// state lives in mma.sync accumulator registers in fp32 for the whole sequence (8 warps x K/8 rows x VS columns);
// per chunk it is rounded to bf16 once into shared memory as the B operand of the products that read it.  All
// products are mma.sync m16n8k16 (bf16 in, fp32 accumulate) on operands staged by cp.async; the operands of the next
// chunk are fetched while the current one is multiplied.  tcgen05 is deliberately not used: a chunk is four products
// of 64..256 rows in a dependent chain of S / 64 links, so the latency of a link decides, not the tensor throughput
// (the same reasoning as for the M2RNN / RNN scans).
//
// Role of fla's chunk_gated_delta_rule as called by the reference
// (lm_engine/modeling_utils/sequence_mixer_blocks/gated_deltanet/module.py:193-222).
// Included by lme_cuda.cu after m2rnn.cu (shares its mma / cp.async helpers).

namespace lme {
namespace dr {

using m2::cp16;
using m2::cp_commit;
using m2::cp_wait;
using m2::mma16816;
using m2::pack2;

constexpr int L = 64;    // rows of a chunk
constexpr int PADE = 8;  // bf16 elements appended to every shared-memory row (spreads the rows over the banks)

// C[16 x 8 NT] += A[m0 .. m0 + 16)[0 .. kd) * B[n0 .. n0 + 8 NT)[0 .. kd)^T; A row-major (lda), B n-major (ldb).
// NEG: the product is subtracted (the sign bits of the A fragments are flipped on the way to the tensor core).
template <int NT, bool NEG = false>
__device__ __forceinline__ void warp_mma(float (&acc)[NT][4], const __nv_bfloat16* A, int lda, int m0,
                                         const __nv_bfloat16* B, int ldb, int n0, int kd, int g, int t) {
    for (int k0 = 0; k0 < kd; k0 += 16) {
        uint32_t a[4];
        const __nv_bfloat16* ap = A + (m0 + g) * lda + k0 + 2 * t;
        a[0] = *reinterpret_cast<const uint32_t*>(ap);
        a[1] = *reinterpret_cast<const uint32_t*>(ap + 8 * lda);
        a[2] = *reinterpret_cast<const uint32_t*>(ap + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(ap + 8 * lda + 8);
        if (NEG) {
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] ^= 0x80008000u;
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const __nv_bfloat16* bp = B + (n0 + nt * 8 + g) * ldb + k0 + 2 * t;
            mma16816(acc[nt], a, *reinterpret_cast<const uint32_t*>(bp), *reinterpret_cast<const uint32_t*>(bp + 8));
        }
    }
}

// rows x cols bf16 tile, contiguous rows in global memory (row pitch = cols) -> shared rows of cols + PADE
__device__ __forceinline__ void stage_tile(__nv_bfloat16* dst, const __nv_bfloat16* src, int rows, int cols) {
    const int per_row = cols / 8;
    for (int i = threadIdx.x; i < rows * per_row; i += blockDim.x) {
        const int r = i / per_row, c = (i % per_row) * 8;
        cp16(dst + r * (cols + PADE) + c, src + static_cast<long long>(r) * cols + c);
    }
}

struct FwdArgs {
    const __nv_bfloat16 *wk, *qe, *ket, *qk;   // [BN][nc][L][K], [BN][nc][L][K], [BN][nc][K][L], [BN][nc][L][L]
    const float *wv, *a, *h0;                       // [BN][nc][L][V], [BN][nc], [BN][K][V] or null
    float* y;                                       // [BN][nc][L][V]
    __nv_bfloat16 *u_all, *h_all;                   // [BN][nc][L][V], [BN][nc][K][V] (state entering the chunk)
    float* h_final;                                 // [BN][K][V]
    int nc, V;
};

struct BwdArgs {
    const __nv_bfloat16 *qkt, *ke, *qet, *wkt;  // [BN][nc][L][L], [BN][nc][L][K], [BN][nc][K][L], [BN][nc][K][L]
    const float *dy, *a, *dh_final;                 // [BN][nc][L][V], [BN][nc], [BN][K][V] or null
    __nv_bfloat16 *du_all, *dh_all;                 // [BN][nc][L][V], [BN][nc][K][V] (gradient leaving the chunk)
    float* dh0;                                     // [BN][K][V]
    int nc, V;
};

// state fragment (mt, nt, i) of warp w, lane (g, t): row = w * (K / 8) + mt * 16 + g + 8 * (i >> 1), col = nt * 8 + 2 t + (i & 1)
template <int K, int VS>
__device__ __forceinline__ void state_to_smem_and_global(const float (&h)[K / 128][VS / 8][4], __nv_bfloat16* sB,
                                                         __nv_bfloat16* gdst, int V, int warp, int g, int t) {
#pragma unroll
    for (int mt = 0; mt < K / 128; ++mt)
#pragma unroll
        for (int nt = 0; nt < VS / 8; ++nt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = warp * (K / 8) + mt * 16 + g + 8 * half, col = nt * 8 + 2 * t;
                const float x0 = h[mt][nt][2 * half], x1 = h[mt][nt][2 * half + 1];
                sB[col * (K + PADE) + row] = __float2bfloat16(x0);
                sB[(col + 1) * (K + PADE) + row] = __float2bfloat16(x1);
                *reinterpret_cast<uint32_t*>(gdst + static_cast<long long>(row) * V + col) = pack2(x0, x1);
            }
}

template <int K, int VS>
__global__ void __launch_bounds__(256, 1) delta_chain_fwd_kernel(FwdArgs p) {
    constexpr int NTL = VS / 16;   // 8-column tiles of an [L, VS] product per warp (two warps share a 16-row block)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sWk = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sQe = sWk + L * (K + PADE);
    __nv_bfloat16* sKet = sQe + L * (K + PADE);
    __nv_bfloat16* sQk = sKet + K * (L + PADE);
    __nv_bfloat16* sH = sQk + L * (L + PADE);
    __nv_bfloat16* sU = sH + VS * (K + PADE);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int mi = warp & 3, nh = warp >> 2;                 // 16-row block and column half of an [L, VS] product
    const long long bn = blockIdx.y;
    const int v0 = blockIdx.x * VS, V = p.V, nc = p.nc;

    float h[K / 128][VS / 8][4];
#pragma unroll
    for (int mt = 0; mt < K / 128; ++mt)
#pragma unroll
        for (int nt = 0; nt < VS / 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = warp * (K / 8) + mt * 16 + g + 8 * (i >> 1), col = nt * 8 + 2 * t + (i & 1);
                h[mt][nt][i] = p.h0 ? p.h0[(bn * K + row) * V + v0 + col] : 0.f;
            }

    auto stage_first = [&](int c) {      // operands of the products with the state
        const long long o = (bn * nc + c) * L * K;
        if (p.wk) stage_tile(sWk, p.wk + o, L, K);     // null: no correction term (linear attention)
        stage_tile(sQe, p.qe + o, L, K);
        cp_commit();
    };
    auto stage_second = [&](int c) {     // operands of the products with U
        stage_tile(sKet, p.ket + (bn * nc + c) * K * L, K, L);
        stage_tile(sQk, p.qk + (bn * nc + c) * L * L, L, L);
        cp_commit();
    };
    stage_first(0);
    stage_second(0);
    // W_v fragments (fp32, the initial value of the U accumulators) are fetched one chunk ahead into registers
    float wv_next[NTL][4];
    auto fetch_wv = [&](int c) {
        const float* wv = p.wv + (bn * nc + c) * L * V + v0;
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) {
            const int col = nh * (VS / 2) + nt * 8 + 2 * t;
            const float2 lo = *reinterpret_cast<const float2*>(wv + static_cast<long long>(mi * 16 + g) * V + col);
            const float2 hi = *reinterpret_cast<const float2*>(wv + static_cast<long long>(mi * 16 + g + 8) * V + col);
            wv_next[nt][0] = lo.x; wv_next[nt][1] = lo.y; wv_next[nt][2] = hi.x; wv_next[nt][3] = hi.y;
        }
    };
    fetch_wv(0);

    for (int c = 0; c < nc; ++c) {
        const long long chunk = bn * nc + c;
        cp_wait<1>();                                        // W_k, Q_e of this chunk have landed (for this thread)
        state_to_smem_and_global<K, VS>(h, sH, p.h_all + chunk * K * V + v0, V, warp, g, t);
        __syncthreads();
        // U = W_v - W_k h,  y = Q_e h (+ QK U below)
        float accU[NTL][4], accY[NTL][4];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                accU[nt][i] = wv_next[nt][i];
                accY[nt][i] = 0.f;
            }
        if (c + 1 < nc) fetch_wv(c + 1);
        if (p.wk) warp_mma<NTL, true>(accU, sWk, K + PADE, mi * 16, sH, K + PADE, nh * (VS / 2), K, g, t);
        warp_mma<NTL>(accY, sQe, K + PADE, mi * 16, sH, K + PADE, nh * (VS / 2), K, g, t);
        __nv_bfloat16* ug = p.u_all + chunk * L * V + v0;
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mi * 16 + g + 8 * half, col = nh * (VS / 2) + nt * 8 + 2 * t;
                const float x0 = accU[nt][2 * half], x1 = accU[nt][2 * half + 1];
                sU[col * (L + PADE) + row] = __float2bfloat16(x0);
                sU[(col + 1) * (L + PADE) + row] = __float2bfloat16(x1);
                *reinterpret_cast<uint32_t*>(ug + static_cast<long long>(row) * V + col) = pack2(x0, x1);
            }
        __syncthreads();                                     // U complete; W_k, Q_e and the state copy are free
        if (c + 1 < nc) stage_first(c + 1); else cp_commit();
        cp_wait<1>();                                        // K_e^T, QK of this chunk have landed
        __syncthreads();
        warp_mma<NTL>(accY, sQk, L + PADE, mi * 16, sU, L + PADE, nh * (VS / 2), L, g, t);
        float* yg = p.y + chunk * L * V + v0;
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) {
            const int col = nh * (VS / 2) + nt * 8 + 2 * t;
            *reinterpret_cast<float2*>(yg + static_cast<long long>(mi * 16 + g) * V + col) =
                make_float2(accY[nt][0], accY[nt][1]);
            *reinterpret_cast<float2*>(yg + static_cast<long long>(mi * 16 + g + 8) * V + col) =
                make_float2(accY[nt][2], accY[nt][3]);
        }
        // h = a h + K_e^T U
        const float a = p.a[chunk];
#pragma unroll
        for (int mt = 0; mt < K / 128; ++mt) {
#pragma unroll
            for (int nt = 0; nt < VS / 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) h[mt][nt][i] *= a;
            warp_mma<VS / 8>(h[mt], sKet, L + PADE, warp * (K / 8) + mt * 16, sU, L + PADE, 0, L, g, t);
        }
        __syncthreads();                                     // K_e^T, QK, U are free
        if (c + 1 < nc) stage_second(c + 1); else cp_commit();
    }
    cp_wait<0>();
#pragma unroll
    for (int mt = 0; mt < K / 128; ++mt)
#pragma unroll
        for (int nt = 0; nt < VS / 8; ++nt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = warp * (K / 8) + mt * 16 + g + 8 * half, col = nt * 8 + 2 * t;
                *reinterpret_cast<float2*>(p.h_final + (bn * K + row) * V + v0 + col) =
                    make_float2(h[mt][nt][2 * half], h[mt][nt][2 * half + 1]);
            }
}

template <int K, int VS>
__global__ void __launch_bounds__(256, 1) delta_chain_bwd_kernel(BwdArgs p) {
    constexpr int NTL = VS / 16;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* sQkt = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sKe = sQkt + L * (L + PADE);
    __nv_bfloat16* sQet = sKe + L * (K + PADE);
    __nv_bfloat16* sWkt = sQet + K * (L + PADE);
    __nv_bfloat16* sDy = sWkt + K * (L + PADE);
    __nv_bfloat16* sDu = sDy + VS * (L + PADE);
    __nv_bfloat16* sDh = sDu + VS * (L + PADE);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int mi = warp & 3, nh = warp >> 2;
    const long long bn = blockIdx.y;
    const int v0 = blockIdx.x * VS, V = p.V, nc = p.nc;

    float dh[K / 128][VS / 8][4];
#pragma unroll
    for (int mt = 0; mt < K / 128; ++mt)
#pragma unroll
        for (int nt = 0; nt < VS / 8; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = warp * (K / 8) + mt * 16 + g + 8 * (i >> 1), col = nt * 8 + 2 * t + (i & 1);
                dh[mt][nt][i] = p.dh_final ? p.dh_final[(bn * K + row) * V + v0 + col] : 0.f;
            }

    auto stage_first = [&](int c) {      // operands of dU
        stage_tile(sQkt, p.qkt + (bn * nc + c) * L * L, L, L);
        stage_tile(sKe, p.ke + (bn * nc + c) * L * K, L, K);
        cp_commit();
    };
    auto stage_second = [&](int c) {     // operands of the state-gradient update
        const long long o = (bn * nc + c) * K * L;
        stage_tile(sQet, p.qet + o, K, L);
        if (p.wkt) stage_tile(sWkt, p.wkt + o, K, L);
        cp_commit();
    };
    stage_first(nc - 1);
    stage_second(nc - 1);
    // the fp32 dy tile of a chunk is fetched one chunk ahead into registers (L * VS / 256 = 16 values per thread)
    float dy_next[L * VS / 256];
    auto fetch_dy = [&](int c) {
        const float* dyg = p.dy + (bn * nc + c) * L * V + v0;
#pragma unroll
        for (int j = 0; j < L * VS / 256; ++j) {
            const int i = threadIdx.x + j * 256;
            dy_next[j] = dyg[static_cast<long long>(i / VS) * V + i % VS];
        }
    };
    fetch_dy(nc - 1);

    for (int c = nc - 1; c >= 0; --c) {
        const long long chunk = bn * nc + c;
        cp_wait<1>();
        state_to_smem_and_global<K, VS>(dh, sDh, p.dh_all + chunk * K * V + v0, V, warp, g, t);
#pragma unroll
        for (int j = 0; j < L * VS / 256; ++j) {
            const int i = threadIdx.x + j * 256;
            sDy[(i % VS) * (L + PADE) + i / VS] = __float2bfloat16(dy_next[j]);
        }
        if (c > 0) fetch_dy(c - 1);
        __syncthreads();
        // dU = QK^T dy + K_e dh
        float accDU[NTL][4];
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt) accDU[nt][0] = accDU[nt][1] = accDU[nt][2] = accDU[nt][3] = 0.f;
        warp_mma<NTL>(accDU, sQkt, L + PADE, mi * 16, sDy, L + PADE, nh * (VS / 2), L, g, t);
        warp_mma<NTL>(accDU, sKe, K + PADE, mi * 16, sDh, K + PADE, nh * (VS / 2), K, g, t);
        __nv_bfloat16* dug = p.du_all + chunk * L * V + v0;
#pragma unroll
        for (int nt = 0; nt < NTL; ++nt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = mi * 16 + g + 8 * half, col = nh * (VS / 2) + nt * 8 + 2 * t;
                const float x0 = accDU[nt][2 * half], x1 = accDU[nt][2 * half + 1];
                sDu[col * (L + PADE) + row] = __float2bfloat16(x0);
                sDu[(col + 1) * (L + PADE) + row] = __float2bfloat16(x1);
                *reinterpret_cast<uint32_t*>(dug + static_cast<long long>(row) * V + col) = pack2(x0, x1);
            }
        __syncthreads();
        if (c > 0) stage_first(c - 1); else cp_commit();
        cp_wait<1>();
        __syncthreads();
        // dh = a dh + Q_e^T dy - W_k^T dU
        const float a = p.a[chunk];
#pragma unroll
        for (int mt = 0; mt < K / 128; ++mt) {
#pragma unroll
            for (int nt = 0; nt < VS / 8; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) dh[mt][nt][i] *= a;
            warp_mma<VS / 8>(dh[mt], sQet, L + PADE, warp * (K / 8) + mt * 16, sDy, L + PADE, 0, L, g, t);
            if (p.wkt)
                warp_mma<VS / 8, true>(dh[mt], sWkt, L + PADE, warp * (K / 8) + mt * 16, sDu, L + PADE, 0, L, g, t);
        }
        __syncthreads();
        if (c > 0) stage_second(c - 1); else cp_commit();
    }
    cp_wait<0>();
#pragma unroll
    for (int mt = 0; mt < K / 128; ++mt)
#pragma unroll
        for (int nt = 0; nt < VS / 8; ++nt)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int row = warp * (K / 8) + mt * 16 + g + 8 * half, col = nt * 8 + 2 * t;
                *reinterpret_cast<float2*>(p.dh0 + (bn * K + row) * V + v0 + col) =
                    make_float2(dh[mt][nt][2 * half], dh[mt][nt][2 * half + 1]);
            }
}

template <int K, int VS>
constexpr int fwd_smem_bytes() {
    return 2 * (2 * L * (K + PADE) + K * (L + PADE) + L * (L + PADE) + VS * (K + PADE) + VS * (L + PADE));
}
template <int K, int VS>
constexpr int bwd_smem_bytes() {
    return 2 * (L * (L + PADE) + L * (K + PADE) + 2 * K * (L + PADE) + 2 * VS * (L + PADE) + VS * (K + PADE));
}

template <int K, int VS>
static int launch_fwd(const FwdArgs& p, int BN, cudaStream_t st) {
    if (cudaFuncSetAttribute(delta_chain_fwd_kernel<K, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             fwd_smem_bytes<K, VS>()) != cudaSuccess)
        return LME_ERR_LAUNCH;
    delta_chain_fwd_kernel<K, VS><<<dim3(p.V / VS, BN), 256, fwd_smem_bytes<K, VS>(), st>>>(p);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
template <int K, int VS>
static int launch_bwd(const BwdArgs& p, int BN, cudaStream_t st) {
    if (cudaFuncSetAttribute(delta_chain_bwd_kernel<K, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             bwd_smem_bytes<K, VS>()) != cudaSuccess)
        return LME_ERR_LAUNCH;
    delta_chain_bwd_kernel<K, VS><<<dim3(p.V / VS, BN), 256, bwd_smem_bytes<K, VS>(), st>>>(p);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

}  // namespace dr
}  // namespace lme

static int delta_chain_check(int BN, int nc, int K, int V) {
    if (BN <= 0 || BN > 65535 || nc <= 0 || (K != 128 && K != 256) || V <= 0 || V % 64) return LME_ERR_SHAPE;
    return LME_OK;
}

extern "C" int lme_delta_chain_fwd(const void* wk, const void* qe, const void* ket, const void* qk, const float* wv,
                                   const float* a, const float* h0, float* y, void* u_all, void* h_all, float* h_final,
                                   int BN, int nc, int K, int V, void* stream) {
    if (int rc = delta_chain_check(BN, nc, K, V)) return rc;
    using bf = __nv_bfloat16;
    lme::dr::FwdArgs p{static_cast<const bf*>(wk), static_cast<const bf*>(qe), static_cast<const bf*>(ket),
                       static_cast<const bf*>(qk), wv, a, h0, y, static_cast<bf*>(u_all), static_cast<bf*>(h_all),
                       h_final, nc, V};
    auto st = static_cast<cudaStream_t>(stream);
    // 64-column slices unless they leave most SMs without a CTA
    const bool narrow = static_cast<long long>(BN) * (V / 64) < 100;
    if (K == 256) return narrow ? lme::dr::launch_fwd<256, 32>(p, BN, st) : lme::dr::launch_fwd<256, 64>(p, BN, st);
    return narrow ? lme::dr::launch_fwd<128, 32>(p, BN, st) : lme::dr::launch_fwd<128, 64>(p, BN, st);
}

extern "C" int lme_delta_chain_bwd(const void* qkt, const void* ke, const void* qet, const void* wkt,
                                   const float* dy, const float* a, const float* dh_final, void* du_all, void* dh_all,
                                   float* dh0, int BN, int nc, int K, int V, void* stream) {
    if (int rc = delta_chain_check(BN, nc, K, V)) return rc;
    using bf = __nv_bfloat16;
    lme::dr::BwdArgs p{static_cast<const bf*>(qkt), static_cast<const bf*>(ke), static_cast<const bf*>(qet),
                       static_cast<const bf*>(wkt), dy, a, dh_final, static_cast<bf*>(du_all),
                       static_cast<bf*>(dh_all), dh0, nc, V};
    auto st = static_cast<cudaStream_t>(stream);
    const bool narrow = static_cast<long long>(BN) * (V / 64) < 100;
    if (K == 256) return narrow ? lme::dr::launch_bwd<256, 32>(p, BN, st) : lme::dr::launch_bwd<256, 64>(p, BN, st);
    return narrow ? lme::dr::launch_bwd<128, 32>(p, BN, st) : lme::dr::launch_bwd<128, 64>(p, BN, st);
}
