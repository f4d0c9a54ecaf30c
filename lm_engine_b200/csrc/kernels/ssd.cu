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


// ------------------------------------------------------------------------------------------------ scan glue
// The element-wise passes around the products of the chunked scan, one kernel per direction instead of a chain of
// PyTorch ops over [tokens, heads, P] fp32 tensors (BC = batch x chunks, rows l of a chunk, heads n, P values):
//   prep     xh [BC,N,L,P]  = x[BC,L,N,P] * dt[BC,L,N]                         (operand of the intra-chunk product)
//            xwT[BC,N,P,L]  = x * dt * tail[BC,L,N], transposed                 (operand of the chunk-state product)
//   prep^T   dx = dt (dxh + tail dxwT^T),  ddt = sum_p x (dxh + tail dxwT^T),  dtail = dt sum_p x dxwT^T
//   combine  y[BC,L,N,P] = yin[BC,N,L,P] + off[BC,G,L,rep*P] * ecum[BC,L,N] + D[n] * x
//   combine^T dyin = dy, doff = dy * ecum, decum = sum_p dy off, dDp[BC,L,N] = sum_p dy x, dx = D dy
// One block handles 32 rows of one (BC, n); a warp owns a row at a time (coalesced along P); the transposed operand
// goes through a padded shared-memory tile so that both its reads and writes are coalesced.
constexpr int GLUE_ROWS = 32;

template <int P>
__global__ void __launch_bounds__(256)
ssd_prep_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ dt, const float* __restrict__ tail,
                __nv_bfloat16* __restrict__ xh, __nv_bfloat16* __restrict__ xwT, int N, int L) {
    __shared__ float tile[GLUE_ROWS][P + 1];
    const int l0 = blockIdx.x * GLUE_ROWS, n = blockIdx.y;
    const long long bc = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < GLUE_ROWS; r += 8) {
        const int l = l0 + r;
        const long long tok = (bc * L + l) * N + n;
        const float d = dt[tok], tl = tail[tok];
        const __nv_bfloat16* xr = x + tok * P;
        __nv_bfloat16* hr = xh + ((bc * N + n) * L + l) * P;
#pragma unroll
        for (int p = lane; p < P; p += 32) {
            const float v = __bfloat162float(xr[p]) * d;
            hr[p] = __float2bfloat16(v);
            tile[r][p] = v * tl;
        }
    }
    __syncthreads();
    __nv_bfloat16* wt = xwT + (bc * N + n) * static_cast<long long>(P) * L + l0;
    for (int p = warp; p < P; p += 8) wt[static_cast<long long>(p) * L + lane] = __float2bfloat16(tile[lane][p]);
}

template <int P>
__global__ void __launch_bounds__(256)
ssd_prep_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ dt, const float* __restrict__ tail,
                    const float* __restrict__ dxh, const __nv_bfloat16* __restrict__ dxwT,
                    __nv_bfloat16* __restrict__ dx, float* __restrict__ ddt, float* __restrict__ dtail, int N, int L) {
    __shared__ float tile[GLUE_ROWS][P + 1];
    const int l0 = blockIdx.x * GLUE_ROWS, n = blockIdx.y;
    const long long bc = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16* wt = dxwT + (bc * N + n) * static_cast<long long>(P) * L + l0;
    for (int p = warp; p < P; p += 8) tile[lane][p] = __bfloat162float(wt[static_cast<long long>(p) * L + lane]);
    __syncthreads();
    for (int r = warp; r < GLUE_ROWS; r += 8) {
        const int l = l0 + r;
        const long long tok = (bc * L + l) * N + n;
        const float d = dt[tok], tl = tail[tok];
        const __nv_bfloat16* xr = x + tok * P;
        const float* gh = dxh + ((bc * N + n) * L + l) * P;
        __nv_bfloat16* dxr = dx + tok * P;
        float s_dt = 0.f, s_tail = 0.f;
#pragma unroll
        for (int p = lane; p < P; p += 32) {
            const float w = tile[r][p], xv = __bfloat162float(xr[p]);
            const float g = gh[p] + tl * w;
            dxr[p] = __float2bfloat16(d * g);
            s_dt += xv * g;
            s_tail += xv * w;
        }
        s_dt = warp_sum(s_dt);
        s_tail = warp_sum(s_tail);
        if (lane == 0) {
            ddt[tok] = s_dt;
            dtail[tok] = d * s_tail;
        }
    }
}

// one warp per (bc, l, n) row
template <int P>
__global__ void __launch_bounds__(256)
ssd_combine_kernel(const float* __restrict__ yin, const float* __restrict__ off, const float* __restrict__ ecum,
                   const float* __restrict__ D, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                   long long rows, int N, int L, int G) {
    const long long row = blockIdx.x * 8ll + (threadIdx.x >> 5);       // (bc * L + l) * N + n
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const int n = static_cast<int>(row % N), l = static_cast<int>((row / N) % L);
    const long long bc = row / N / L;
    const int rep = N / G, g = n / rep, r = n % rep;
    const float e = ecum[row], dn = D[n];
    const float* yi = yin + ((bc * N + n) * L + l) * P;
    const float* of = off + ((bc * G + g) * L + l) * static_cast<long long>(rep) * P + r * P;
#pragma unroll
    for (int p = lane; p < P; p += 32)
        y[row * P + p] = __float2bfloat16(yi[p] + of[p] * e + dn * __bfloat162float(x[row * P + p]));
}

template <int P>
__global__ void __launch_bounds__(256)
ssd_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ off,
                       const float* __restrict__ ecum, const float* __restrict__ D,
                       const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ dyin,
                       __nv_bfloat16* __restrict__ doff, float* __restrict__ decum, float* __restrict__ dDp,
                       __nv_bfloat16* __restrict__ dx, long long rows, int N, int L, int G) {
    const long long row = blockIdx.x * 8ll + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const int n = static_cast<int>(row % N), l = static_cast<int>((row / N) % L);
    const long long bc = row / N / L;
    const int rep = N / G, g = n / rep, r = n % rep;
    const float e = ecum[row], dn = D[n];
    const long long o_in = ((bc * N + n) * L + l) * P;
    const long long o_off = ((bc * G + g) * L + l) * static_cast<long long>(rep) * P + r * P;
    float s_e = 0.f, s_d = 0.f;
#pragma unroll
    for (int p = lane; p < P; p += 32) {
        const float gy = __bfloat162float(dy[row * P + p]);
        dyin[o_in + p] = dy[row * P + p];
        doff[o_off + p] = __float2bfloat16(gy * e);
        dx[row * P + p] = __float2bfloat16(dn * gy);
        s_e += gy * off[o_off + p];
        s_d += gy * __bfloat162float(x[row * P + p]);
    }
    s_e = warp_sum(s_e);
    s_d = warp_sum(s_d);
    if (lane == 0) {
        decum[row] = s_e;
        dDp[row] = s_d;
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

// Scan glue (see the kernels): BC = batch x chunks, L % 32 == 0, P in {32, 64, 128}, N % G == 0.  mode 0 = forward,
// 1 = backward; unused pointers of a mode may be null.
extern "C" int lme_ssd_prep(const void* x, const float* dt, const float* tail, void* xh, void* xwT,
                            const float* dxh, const void* dxwT, void* dx, float* ddt, float* dtail, long long BC,
                            int N, int L, int P, int mode, void* stream) {
    if (BC <= 0) return LME_OK;
    if (L % lme::GLUE_ROWS || BC > 65535 || N > 65535) return LME_ERR_SHAPE;
    dim3 grid(L / lme::GLUE_ROWS, N, static_cast<unsigned>(BC));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto X = static_cast<const __nv_bfloat16*>(x);
#define LME_PREP(PP)                                                                                                  \
    if (mode == 0)                                                                                                    \
        ssd_prep_kernel<PP><<<grid, 256, 0, st>>>(X, dt, tail, static_cast<__nv_bfloat16*>(xh),                       \
                                                  static_cast<__nv_bfloat16*>(xwT), N, L);                           \
    else                                                                                                              \
        ssd_prep_bwd_kernel<PP><<<grid, 256, 0, st>>>(X, dt, tail, dxh, static_cast<const __nv_bfloat16*>(dxwT),      \
                                                      static_cast<__nv_bfloat16*>(dx), ddt, dtail, N, L);
    if (P == 32) { LME_PREP(32) } else if (P == 64) { LME_PREP(64) } else if (P == 128) { LME_PREP(128) } else return LME_ERR_SHAPE;
#undef LME_PREP
    return LME_LAUNCH_OK();
}

extern "C" int lme_ssd_combine(const float* yin, const float* off, const float* ecum, const float* D, const void* x,
                               void* y, const void* dy, void* dyin, void* doff, float* decum, float* dDp, void* dx,
                               long long BC, int N, int L, int G, int P, int mode, void* stream) {
    if (BC <= 0) return LME_OK;
    if (N % G) return LME_ERR_SHAPE;
    const long long rows = BC * L * N;
    const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto X = static_cast<const __nv_bfloat16*>(x);
#define LME_COMB(PP)                                                                                                  \
    if (mode == 0)                                                                                                    \
        ssd_combine_kernel<PP><<<grid, 256, 0, st>>>(yin, off, ecum, D, X, static_cast<__nv_bfloat16*>(y), rows, N,  \
                                                     L, G);                                                           \
    else                                                                                                              \
        ssd_combine_bwd_kernel<PP><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(dy), off, ecum, D, X,      \
                                                         static_cast<__nv_bfloat16*>(dyin),                           \
                                                         static_cast<__nv_bfloat16*>(doff), decum, dDp,               \
                                                         static_cast<__nv_bfloat16*>(dx), rows, N, L, G);
    if (P == 32) { LME_COMB(32) } else if (P == 64) { LME_COMB(64) } else if (P == 128) { LME_COMB(128) } else return LME_ERR_SHAPE;
#undef LME_COMB
    return LME_LAUNCH_OK();
}

// ----------------------------------------------------------------------------------------------------------------
// Chunk-boundary recurrence of the SSD scan:  h_0 = h_init,  h_{c+1} = decay[c] * h_c + S_c  per (batch, head), where
// S_c [P * Sd] is the summary of chunk c and decay[c] = exp(sum of dt A over the chunk).  The forward kernel walks the
// chunks once and writes the state at every chunk start (bf16: the operand of the carried-state product; optionally
// fp32 for the backward pass) and the final state; the backward kernel walks them in reverse:
//   dS_c = g,   d decay[c] = <g, h_c>,   g <- decay[c] * g + dh_c        (g starts as d h_final, ends as d h_init)
// One CTA per (batch, head); the P * Sd state elements are spread over its threads, 4 per thread and pass.
namespace lme {

// E = P * Sd (multiple of 4).  states / h0_f32 / dh0 / dstates: [B, NC, N, E];  decay / ddecay: [B, NC, N].
__global__ void __launch_bounds__(256)
ssd_boundary_fwd_kernel(const float* __restrict__ states, const float* __restrict__ decay,
                        const float* __restrict__ h_init, __nv_bfloat16* __restrict__ h0_bf16,
                        float* __restrict__ h0_f32, float* __restrict__ h_final, int NC, int N, int E) {
    const int b = blockIdx.x / N, n = blockIdx.x % N;
    for (int e = threadIdx.x * 4; e < E; e += blockDim.x * 4) {
        float4 h = make_float4(0.f, 0.f, 0.f, 0.f);
        if (h_init != nullptr) h = *reinterpret_cast<const float4*>(h_init + (static_cast<long long>(b) * N + n) * E + e);
        for (int c = 0; c < NC; ++c) {
            const long long row = (static_cast<long long>(b) * NC + c) * N + n;
            const long long off = row * E + e;
            uint2 o;
            o.x = pack_bf16x2(h.x, h.y);
            o.y = pack_bf16x2(h.z, h.w);
            *reinterpret_cast<uint2*>(h0_bf16 + off) = o;
            if (h0_f32 != nullptr) *reinterpret_cast<float4*>(h0_f32 + off) = h;
            const float d = __ldg(decay + row);
            const float4 s = *reinterpret_cast<const float4*>(states + off);
            h.x = h.x * d + s.x; h.y = h.y * d + s.y; h.z = h.z * d + s.z; h.w = h.w * d + s.w;
        }
        *reinterpret_cast<float4*>(h_final + (static_cast<long long>(b) * N + n) * E + e) = h;
    }
}

// blockDim.x * 4 >= E is not required: every thread keeps its running gradient per owned 4-vector in registers for
// up to MAXV vectors (E <= 256 threads * 4 * MAXV).
template <int MAXV>
__global__ void __launch_bounds__(256)
ssd_boundary_bwd_kernel(const float* __restrict__ dh0, const float* __restrict__ dh_final,
                        const float* __restrict__ h0_f32, const float* __restrict__ decay,
                        float* __restrict__ dstates, float* __restrict__ ddecay, float* __restrict__ dh_init, int NC,
                        int N, int E) {
    __shared__ float red[32];
    const int b = blockIdx.x / N, n = blockIdx.x % N;
    float4 g[MAXV];
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
        const int e = (v * blockDim.x + threadIdx.x) * 4;
        g[v] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (e < E && dh_final != nullptr)
            g[v] = *reinterpret_cast<const float4*>(dh_final + (static_cast<long long>(b) * N + n) * E + e);
    }
    for (int c = NC - 1; c >= 0; --c) {
        const long long row = (static_cast<long long>(b) * NC + c) * N + n;
        const float d = __ldg(decay + row);
        float dot = 0.f;
#pragma unroll
        for (int v = 0; v < MAXV; ++v) {
            const int e = (v * blockDim.x + threadIdx.x) * 4;
            if (e < E) {
                const long long off = row * E + e;
                *reinterpret_cast<float4*>(dstates + off) = g[v];
                const float4 h = *reinterpret_cast<const float4*>(h0_f32 + off);
                dot += g[v].x * h.x + g[v].y * h.y + g[v].z * h.z + g[v].w * h.w;
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
                if (dh0 != nullptr) a = *reinterpret_cast<const float4*>(dh0 + off);
                g[v].x = g[v].x * d + a.x; g[v].y = g[v].y * d + a.y;
                g[v].z = g[v].z * d + a.z; g[v].w = g[v].w * d + a.w;
            }
        }
        dot = block_sum(dot, red);
        if (threadIdx.x == 0) ddecay[row] = dot;
    }
    if (dh_init != nullptr) {
#pragma unroll
        for (int v = 0; v < MAXV; ++v) {
            const int e = (v * blockDim.x + threadIdx.x) * 4;
            if (e < E) *reinterpret_cast<float4*>(dh_init + (static_cast<long long>(b) * N + n) * E + e) = g[v];
        }
    }
}

}  // namespace lme

extern "C" int lme_ssd_boundary_fwd(const float* states, const float* decay, const float* h_init, void* h0_bf16,
                                    float* h0_f32, float* h_final, int B, int NC, int N, int E, void* stream) {
    if (B <= 0 || NC <= 0 || N <= 0 || E <= 0 || (E % 4)) return LME_ERR_SHAPE;
    lme::ssd_boundary_fwd_kernel<<<B * N, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        states, decay, h_init, static_cast<__nv_bfloat16*>(h0_bf16), h0_f32, h_final, NC, N, E);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}

extern "C" int lme_ssd_boundary_bwd(const float* dh0, const float* dh_final, const float* h0_f32, const float* decay,
                                    float* dstates, float* ddecay, float* dh_init, int B, int NC, int N, int E,
                                    void* stream) {
    if (B <= 0 || NC <= 0 || N <= 0 || E <= 0 || (E % 4) || E > 256 * 4 * 16) return LME_ERR_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int vecs = (E / 4 + 255) / 256;
    if (vecs <= 2)
        lme::ssd_boundary_bwd_kernel<2><<<B * N, 256, 0, st>>>(dh0, dh_final, h0_f32, decay, dstates, ddecay, dh_init,
                                                              NC, N, E);
    else if (vecs <= 8)
        lme::ssd_boundary_bwd_kernel<8><<<B * N, 256, 0, st>>>(dh0, dh_final, h0_f32, decay, dstates, ddecay, dh_init,
                                                              NC, N, E);
    else
        lme::ssd_boundary_bwd_kernel<16><<<B * N, 256, 0, st>>>(dh0, dh_final, h0_f32, decay, dstates, ddecay,
                                                               dh_init, NC, N, E);
    return cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH;
}
