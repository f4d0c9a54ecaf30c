// Bandwidth-bound kernels of the dense transformer block: RMSNorm (+ fused residual add) fwd/bwd, SwiGLU on
// interleaved (gate, up) columns fwd/bwd, fused QKV split + rotary embedding fwd/bwd, cross-entropy statistics and
// in-place gradient (vocab-parallel capable), fused AdamW on flat shards, squared-norm reduction and the clip
// coefficient.  All activations are bf16, all math is fp32, all global accesses are 16-byte vectors.
#include "common.cuh"
#include "../lme_api.h"

namespace lme {

struct alignas(16) bf16x8 {
    uint32_t w[4];
};
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
    bf16x8 v = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = unpack_bf16x2(v.w[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
    bf16x8 v;
#pragma unroll
    for (int i = 0; i < 4; ++i) v.w[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<bf16x8*>(p) = v;
}

// ---------------------------------------------------------------------------------------------- RMSNorm
// h = x (+ residual);  y = h * rsqrt(mean(h^2) + eps) * w.   One CTA per row, row cached in registers.
template <int VPT>  // 8-element vectors per thread (H <= VPT * 8 * blockDim)
__global__ void __launch_bounds__(512) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd, int H, float eps) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const __nv_bfloat16* xr = x + row * H;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        int c = (i * blockDim.x + threadIdx.x) * 8;
        if (c < H) {
            load8(xr + c, v[i]);
            if (residual != nullptr) {
                float r[8];
                load8(residual + row * H + c, r);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i][j] = __bfloat162float(__float2bfloat16_rn(v[i][j] + r[j]));
                if (h_out != nullptr) store8(h_out + row * H + c, v[i]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
        }
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / H + eps);
    if (threadIdx.x == 0 && rstd != nullptr) rstd[row] = rs;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        int c = (i * blockDim.x + threadIdx.x) * 8;
        if (c < H) {
            float o[8];
            if (w != nullptr) {
                float wv[8];
                load8(w + c, wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rs * wv[j];
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rs;
            }
            store8(y + row * H + c, o);
        }
    }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) (+ dres);  dw partial sums per CTA (rows strided by gridDim).
template <int VPT>
__global__ void __launch_bounds__(512, 3) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int T, int H) {
    __shared__ float red[32];
    float dwacc[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    float wv[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        int c = (i * blockDim.x + threadIdx.x) * 8;
        if (c < H && w != nullptr) {
            load8(w + c, wv[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[i][j] = 1.f;
        }
    }
    for (long long row = blockIdx.x; row < T; row += gridDim.x) {
        const float rs = rstd[row];
        float g[VPT][8], xh[VPT][8];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int c = (i * blockDim.x + threadIdx.x) * 8;
            if (c < H) {
                load8(dy + row * H + c, g[i]);
                load8(h + row * H + c, xh[i]);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    xh[i][j] *= rs;
                    dwacc[i][j] += g[i][j] * xh[i][j];
                    g[i][j] *= wv[i][j];
                    dot += g[i][j] * xh[i][j];
                }
            }
        }
        dot = block_sum(dot, red) / H;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int c = (i * blockDim.x + threadIdx.x) * 8;
            if (c < H) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = rs * (g[i][j] - xh[i][j] * dot);
                if (dres != nullptr) {
                    float r[8];
                    load8(dres + row * H + c, r);
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] += r[j];
                }
                store8(dx + row * H + c, o);
            }
        }
    }
    if (dw_partial != nullptr) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int c = (i * blockDim.x + threadIdx.x) * 8;
            if (c < H) {
                float* o = dw_partial + static_cast<long long>(blockIdx.x) * H + c;
                *reinterpret_cast<float4*>(o) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
            }
        }
    }
}

// out[c] (+)= sum_r partial[r, c]   (fp32 out).  Block = 32 columns x 32 row lanes: every row lane sums a strided
// subset of the rows with coalesced 128-byte loads, the lanes are combined through shared memory.
__global__ void __launch_bounds__(1024) colsum_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                      int R, int H, int accumulate) {
    __shared__ float tile[32][33];
    const int c = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (c < H)
        for (int r = threadIdx.y; r < R; r += 32) s += partial[static_cast<long long>(r) * H + c];
    tile[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < H) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) t += tile[i][threadIdx.x];
        out[c] = accumulate ? out[c] + t : t;
    }
}

// ---------------------------------------------------------------------------------------------- SwiGLU
// x [T, 2I] interleaved (gate at even, up at odd columns) -> y [T, I] = up * silu(gate)
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                  long long n_out8) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_out8;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float a[8], b[8], o[8];
        load8(x + i * 16, a);
        load8(x + i * 16 + 8, b);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            o[j] = a[2 * j + 1] * silu_f(a[2 * j]);
            o[4 + j] = b[2 * j + 1] * silu_f(b[2 * j]);
        }
        store8(y + i * 8, o);
    }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dx, long long n_out8) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_out8;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float a[16], g[8], o[16];
        {
            float t0[8], t1[8];
            load8(x + i * 16, t0);
            load8(x + i * 16 + 8, t1);
#pragma unroll
            for (int j = 0; j < 8; ++j) { a[j] = t0[j]; a[8 + j] = t1[j]; }
        }
        load8(dy + i * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float gate = a[2 * j], up = a[2 * j + 1];
            float s = 1.f / (1.f + __expf(-gate));
            o[2 * j] = g[j] * up * s * (1.f + gate * (1.f - s));
            o[2 * j + 1] = g[j] * gate * s;
        }
        float o0[8], o1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { o0[j] = o[j]; o1[j] = o[8 + j]; }
        store8(dx + i * 16, o0);
        store8(dx + i * 16 + 8, o1);
    }
}

// The same on rows grouped in 128-row tiles of which only those with tile_group[tile] >= 0 hold data (the padded
// per-expert layout of the grouped GEMMs): one CTA per tile, tiles without an expert are not touched.
__global__ void __launch_bounds__(256)
swiglu_bwd_tiles_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                        __nv_bfloat16* __restrict__ dx, int I8, const int* __restrict__ tile_group) {
    if (tile_group[blockIdx.x] < 0) return;
    const long long first = static_cast<long long>(blockIdx.x) * 128 * I8;
    for (int u = threadIdx.x; u < 128 * I8; u += blockDim.x) {
        const long long i = first + u;
        float t0[8], t1[8], g[8], o0[8], o1[8];
        load8(x + i * 16, t0);
        load8(x + i * 16 + 8, t1);
        load8(dy + i * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gate = j < 4 ? t0[2 * j] : t1[2 * j - 8], up = j < 4 ? t0[2 * j + 1] : t1[2 * j - 7];
            const float s = 1.f / (1.f + __expf(-gate));
            const float dg = g[j] * up * s * (1.f + gate * (1.f - s)), du = g[j] * gate * s;
            if (j < 4) { o0[2 * j] = dg; o0[2 * j + 1] = du; } else { o1[2 * j - 8] = dg; o1[2 * j - 7] = du; }
        }
        store8(dx + i * 16, o0);
        store8(dx + i * 16 + 8, o1);
    }
}

// ---------------------------------------------------------------------------------------------- QKV split + RoPE
// qkv [T, Hkv, (G+2)*D] (per KV head: G query heads, then K, then V)  <->  q [T, Hkv*G, D], k [T, Hkv, D], v [T, Hkv, D]
// Rotation (NeoX half-rotation) on the last `rd` channels of each q / k head with angle table cos/sin [P, rd] (fp32,
// both halves identical), position pos[t] (or t % S when pos == nullptr).  inverse = 1 applies the transposed
// rotation and packs (dq, dk, dv) back into dqkv.
__global__ void qkv_rope_kernel(__nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q,
                                __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v,
                                const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                const int* __restrict__ pos, int T, int S, int Hkv, int G, int D, int rd,
                                int max_pos, int inverse) {
    const int heads_per_group = G + 2;
    const int vec_per_head = D / 8;
    const int half = rd / 2;
    const int r0 = D - rd;
    const long long total = static_cast<long long>(T) * Hkv * heads_per_group * vec_per_head;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        int vec = i % vec_per_head;
        long long rest = i / vec_per_head;
        int hg = rest % heads_per_group;
        rest /= heads_per_group;
        int kvh = rest % Hkv;
        long long t = rest / Hkv;
        int c = vec * 8;
        __nv_bfloat16* packed = qkv + ((t * Hkv + kvh) * heads_per_group + hg) * D;
        __nv_bfloat16* split;
        bool rotate = rd > 0;
        if (hg < G) split = q + ((t * Hkv + kvh) * G + hg) * D;
        else if (hg == G) split = k + (t * Hkv + kvh) * D;
        else { split = v + (t * Hkv + kvh) * D; rotate = false; }
        const __nv_bfloat16* src = inverse ? split : packed;
        __nv_bfloat16* dst = inverse ? packed : split;
        float a[8];
        if (rotate && c >= r0) {
            // The vector in the first half of the rotary span and its partner in the second half use the same
            // angles: the thread that owns the first-half vector rotates both (one load of each vector and of the
            // cos / sin row), the owner of the partner has nothing left to do.
            const int rc = c - r0;
            if (rc >= half) continue;
            float b[8];
            load8(src + c, a);
            load8(src + c + half, b);
            int p = pos != nullptr ? pos[t] : static_cast<int>(t % S);
            if (p < 0 || p >= max_pos) {  // position outside the angle table: record it and leave the head unrotated
                report_error(STATUS_BOUNDS, static_cast<unsigned int>(p));
                store8(dst + c, a);
                store8(dst + c + half, b);
                continue;
            }
            const float4* cs = reinterpret_cast<const float4*>(cos_t + static_cast<long long>(p) * rd + rc);
            const float4* sn = reinterpret_cast<const float4*>(sin_t + static_cast<long long>(p) * rd + rc);
            const float4 c0 = __ldg(cs), c1 = __ldg(cs + 1), s0 = __ldg(sn), s1 = __ldg(sn + 1);
            const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const float sgn = inverse ? -1.f : 1.f;
            float oa[8], ob[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                oa[j] = a[j] * cv[j] - sgn * b[j] * sv[j];
                ob[j] = b[j] * cv[j] + sgn * a[j] * sv[j];
            }
            store8(dst + c, oa);
            store8(dst + c + half, ob);
            continue;
        }
        load8(src + c, a);
        store8(dst + c, a);
    }
}

// ---------------------------------------------------------------------------------------------- cross entropy
// Per-row statistics over a (local) vocabulary slice: running max, sum exp(x - max), and the target logit if the
// label falls inside [v0, v0 + V).  logits bf16 [T, ld].
__global__ void ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                                const long long* __restrict__ labels, float* __restrict__ row_max,
                                float* __restrict__ row_sum, float* __restrict__ tgt_logit, int V, int v0) {
    __shared__ float red[32];
    const long long row = blockIdx.x;
    const __nv_bfloat16* lr = logits + row * ld;
    float m = -INFINITY, s = 0.f;
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
        float a[8];
        load8(lr + c, a);
        float lm = a[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) lm = fmaxf(lm, a[j]);
        float nm = fmaxf(m, lm);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += __expf(a[j] - nm);
        s = s * __expf(m - nm) + acc;
        m = nm;
    }
    float gm = block_max(m, red);
    float gs = block_sum(m == -INFINITY ? 0.f : s * __expf(m - gm), red);
    if (threadIdx.x == 0) {
        row_max[row] = gm;
        row_sum[row] = gs;
        long long lab = labels[row] - v0;
        tgt_logit[row] = (lab >= 0 && lab < V) ? __bfloat162float(lr[lab]) : 0.f;
    }
}
// In place: logits <- (exp(x - lse) - [col == label]) * scale   (zero rows whose label == ignore_index)
__global__ void ce_grad_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                               const long long* __restrict__ labels, const float* __restrict__ lse, int V, int v0,
                               float scale, const float* __restrict__ scale_dev, long long ignore_index) {
    if (scale_dev != nullptr) scale *= *scale_dev;
    const long long row = blockIdx.x;
    __nv_bfloat16* lr = logits + row * ld;
    const long long lab_g = labels[row];
    const bool ignored = lab_g == ignore_index;
    const long long lab = lab_g - v0;
    const float l = lse[row];
    for (int c = threadIdx.x * 8; c < V; c += blockDim.x * 8) {
        float a[8];
        if (ignored) {
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = 0.f;
        } else {
            load8(lr + c, a);
#pragma unroll
            for (int j = 0; j < 8; ++j) a[j] = (__expf(a[j] - l) - ((c + j) == lab ? 1.f : 0.f)) * scale;
        }
        store8(lr + c, a);
    }
}

// ---------------------------------------------------------------------------------------------- optimizer
// torch.optim.AdamW semantics on a flat shard.  g may be bf16 or fp32; the bf16 compute copy is refreshed in the
// same pass.  *gscale (optional, device) multiplies the gradient (clip coefficient x unscale).
template <typename GT>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, float* __restrict__ m,
                                                    float* __restrict__ v, const GT* __restrict__ g,
                                                    __nv_bfloat16* __restrict__ p_lp, long long n, float lr,
                                                    float b1, float b2, float eps, float wd, float bc1,
                                                    float bc2_sqrt, const float* __restrict__ gscale) {
    const float gs = gscale != nullptr ? *gscale : 1.f;
    const float step = lr / bc1;
    const float decay = 1.f - lr * wd;
    const float rbc2 = 1.f / bc2_sqrt;
    // 8 elements per thread and iteration: 2 x 16-byte accesses on every fp32 stream, one on the bf16 streams
    for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 8; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
        if (i + 8 <= n) {
            float pp[8], mm[8], v2[8], gg[8];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float4 a = *reinterpret_cast<const float4*>(p + i + 4 * h);
                float4 b = *reinterpret_cast<const float4*>(m + i + 4 * h);
                float4 c = *reinterpret_cast<const float4*>(v + i + 4 * h);
                pp[4 * h] = a.x; pp[4 * h + 1] = a.y; pp[4 * h + 2] = a.z; pp[4 * h + 3] = a.w;
                mm[4 * h] = b.x; mm[4 * h + 1] = b.y; mm[4 * h + 2] = b.z; mm[4 * h + 3] = b.w;
                v2[4 * h] = c.x; v2[4 * h + 1] = c.y; v2[4 * h + 2] = c.z; v2[4 * h + 3] = c.w;
            }
            if constexpr (sizeof(GT) == 2) {
                load8(reinterpret_cast<const __nv_bfloat16*>(g) + i, gg);
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float4 a = *reinterpret_cast<const float4*>(g + i + 4 * h);
                    gg[4 * h] = a.x; gg[4 * h + 1] = a.y; gg[4 * h + 2] = a.z; gg[4 * h + 3] = a.w;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float gr = gg[j] * gs;
                pp[j] *= decay;
                mm[j] = b1 * mm[j] + (1.f - b1) * gr;
                v2[j] = b2 * v2[j] + (1.f - b2) * gr * gr;
                float denom = sqrtf(v2[j]) * rbc2 + eps;
                pp[j] -= step * mm[j] / denom;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                *reinterpret_cast<float4*>(p + i + 4 * h) = make_float4(pp[4 * h], pp[4 * h + 1], pp[4 * h + 2], pp[4 * h + 3]);
                *reinterpret_cast<float4*>(m + i + 4 * h) = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
                *reinterpret_cast<float4*>(v + i + 4 * h) = make_float4(v2[4 * h], v2[4 * h + 1], v2[4 * h + 2], v2[4 * h + 3]);
            }
            if (p_lp != nullptr) store8(p_lp + i, pp);
        } else {
            for (long long k = i; k < n; ++k) {
                float gr = static_cast<float>(g[k]) * gs;
                float pq = p[k] * decay;
                float mq = b1 * m[k] + (1.f - b1) * gr;
                float vq = b2 * v[k] + (1.f - b2) * gr * gr;
                pq -= step * mq / (sqrtf(vq) * rbc2 + eps);
                p[k] = pq; m[k] = mq; v[k] = vq;
                if (p_lp != nullptr) p_lp[k] = __float2bfloat16_rn(pq);
            }
        }
    }
}

// partial[b] = sum over this CTA's grid-stride slice of x^2 (16-byte loads, scalar tail)
template <typename T>
__global__ void sumsq_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ partial) {
    __shared__ float red[32];
    constexpr int VEC = 16 / sizeof(T);
    float s = 0.f;
    const long long nvec = n / VEC;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        if constexpr (sizeof(T) == 2) {
            float f[8];
            load8(reinterpret_cast<const __nv_bfloat16*>(x) + i * 8, f);
#pragma unroll
            for (int j = 0; j < 8; ++j) s += f[j] * f[j];
        } else {
            float4 f = *reinterpret_cast<const float4*>(x + i * 4);
            s += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
        }
    }
    if (blockIdx.x == 0) {
        for (long long i = nvec * VEC + threadIdx.x; i < n; i += blockDim.x) {
            float f = static_cast<float>(x[i]);
            s += f * f;
        }
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// out[0] (+)= sum(partial[0..n))  - single CTA, deterministic order
__global__ void sum_partials_kernel(const float* __restrict__ partial, int n, float* __restrict__ out,
                                    int accumulate) {
    __shared__ float red[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
    s = block_sum(s, red);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}
// norm = sqrt(sumsq); coef = min(1, max_norm / (norm + 1e-6))   (max_norm <= 0: coef = 1)
__global__ void clip_coef_kernel(const float* __restrict__ sumsq, float max_norm, float* __restrict__ norm_out,
                                 float* __restrict__ coef_out) {
    float n = sqrtf(sumsq[0]);
    norm_out[0] = n;
    float c = max_norm > 0.f ? max_norm / (n + 1e-6f) : 1.f;
    coef_out[0] = fminf(c, 1.f);
}

static inline int grid_for(long long work, int block, int cap) {
    long long g = (work + block - 1) / block;
    if (g < 1) g = 1;
    return static_cast<int>(g < cap ? g : cap);
}

}  // namespace lme

using namespace lme;

#define LME_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? LME_OK : LME_ERR_LAUNCH)

extern "C" int lme_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out,
                               float* rstd, int T, int H, float eps, void* stream) {
    if (H % 8 || H > 16384) return LME_ERR_SHAPE;
    if (T == 0) return LME_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto X = static_cast<const __nv_bfloat16*>(x);
    auto R = static_cast<const __nv_bfloat16*>(residual);
    auto W = static_cast<const __nv_bfloat16*>(w);
    auto Y = static_cast<__nv_bfloat16*>(y);
    auto HO = static_cast<__nv_bfloat16*>(h_out);
    int vecs = H / 8;
    if (vecs <= 128) rmsnorm_fwd_kernel<1><<<T, 128, 0, st>>>(X, R, W, Y, HO, rstd, H, eps);
    else if (vecs <= 256) rmsnorm_fwd_kernel<1><<<T, 256, 0, st>>>(X, R, W, Y, HO, rstd, H, eps);
    else if (vecs <= 512) rmsnorm_fwd_kernel<1><<<T, 512, 0, st>>>(X, R, W, Y, HO, rstd, H, eps);
    else if (vecs <= 1024) rmsnorm_fwd_kernel<2><<<T, 512, 0, st>>>(X, R, W, Y, HO, rstd, H, eps);
    else rmsnorm_fwd_kernel<4><<<T, 512, 0, st>>>(X, R, W, Y, HO, rstd, H, eps);
    return LME_LAUNCH_OK();
}

// Rows of dw_partial the backward kernel writes for a [T, H] problem (the caller sizes the scratch with it).
// 3 CTAs of 512 threads are resident per SM (40 registers per thread): one wave of 148 x 3 CTAs
extern "C" int lme_rmsnorm_bwd_partial_rows(int T) {
    return T < LME_RMSNORM_BWD_MAX_PARTIAL_ROWS ? (T < 1 ? 1 : T) : LME_RMSNORM_BWD_MAX_PARTIAL_ROWS;
}

// dw_partial: fp32 scratch [lme_rmsnorm_bwd_partial_rows(T), H] (may be null when w is null / dw not needed).
extern "C" int lme_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                               void* dx, float* dw_partial, float* dw, int dw_accumulate, int T, int H,
                               void* stream) {
    if (H % 8 || H > 16384) return LME_ERR_SHAPE;
    if (T == 0) return LME_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto DY = static_cast<const __nv_bfloat16*>(dy);
    auto HH = static_cast<const __nv_bfloat16*>(h);
    auto W = static_cast<const __nv_bfloat16*>(w);
    auto DR = static_cast<const __nv_bfloat16*>(dres);
    auto DX = static_cast<__nv_bfloat16*>(dx);
    int G = lme_rmsnorm_bwd_partial_rows(T);
    int vecs = H / 8;
    if (vecs <= 128) rmsnorm_bwd_kernel<1><<<G, 128, 0, st>>>(DY, HH, W, rstd, DR, DX, dw_partial, T, H);
    else if (vecs <= 256) rmsnorm_bwd_kernel<1><<<G, 256, 0, st>>>(DY, HH, W, rstd, DR, DX, dw_partial, T, H);
    else if (vecs <= 512) rmsnorm_bwd_kernel<1><<<G, 512, 0, st>>>(DY, HH, W, rstd, DR, DX, dw_partial, T, H);
    else if (vecs <= 1024) rmsnorm_bwd_kernel<2><<<G, 512, 0, st>>>(DY, HH, W, rstd, DR, DX, dw_partial, T, H);
    else rmsnorm_bwd_kernel<4><<<G, 512, 0, st>>>(DY, HH, W, rstd, DR, DX, dw_partial, T, H);
    if (dw_partial != nullptr && dw != nullptr)
        colsum_kernel<<<(H + 31) / 32, dim3(32, 32), 0, st>>>(dw_partial, dw, G, H, dw_accumulate);
    return LME_LAUNCH_OK();
}

extern "C" int lme_swiglu_fwd(const void* x, void* y, long long T, long long I, void* stream) {
    if (I % 8) return LME_ERR_SHAPE;
    long long n8 = T * I / 8;
    if (n8 == 0) return LME_OK;
    swiglu_fwd_kernel<<<grid_for(n8, 256, 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n8);
    return LME_LAUNCH_OK();
}
extern "C" int lme_swiglu_bwd(const void* x, const void* dy, void* dx, long long T, long long I, void* stream) {
    if (I % 8) return LME_ERR_SHAPE;
    long long n8 = T * I / 8;
    if (n8 == 0) return LME_OK;
    swiglu_bwd_kernel<<<grid_for(n8, 256, 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
        static_cast<__nv_bfloat16*>(dx), n8);
    return LME_LAUNCH_OK();
}

extern "C" int lme_swiglu_bwd_tiles(const void* x, const void* dy, void* dx, long long T, long long I,
                                    const int* tile_group, void* stream) {
    if (I % 8 || T % 128 || T / 128 > 0x7fffffffll) return LME_ERR_SHAPE;
    if (T == 0 || I == 0) return LME_OK;
    swiglu_bwd_tiles_kernel<<<static_cast<unsigned>(T / 128), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx),
        static_cast<int>(I / 8), tile_group);
    return LME_LAUNCH_OK();
}

extern "C" int lme_qkv_rope(void* qkv, void* q, void* k, void* v, const float* cos_t, const float* sin_t,
                            const int* pos, int T, int S, int Hkv, int G, int D, int rope_dim, int max_pos,
                            int inverse, void* stream) {
    if (D % 8 || rope_dim % 16 || rope_dim > D) return LME_ERR_SHAPE;
    long long total = static_cast<long long>(T) * Hkv * (G + 2) * (D / 8);
    if (total == 0) return LME_OK;
    qkv_rope_kernel<<<grid_for(total, 256, 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k),
        static_cast<__nv_bfloat16*>(v), cos_t, sin_t, pos, T, S, Hkv, G, D, rope_dim, max_pos, inverse);
    return LME_LAUNCH_OK();
}

extern "C" int lme_ce_stats(const void* logits, long long ld, const long long* labels, float* row_max,
                            float* row_sum, float* tgt_logit, int T, int V, int v0, void* stream) {
    if (V % 8 || ld % 8) return LME_ERR_SHAPE;
    if (T == 0) return LME_OK;
    ce_stats_kernel<<<T, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), ld, labels, row_max, row_sum, tgt_logit, V, v0);
    return LME_LAUNCH_OK();
}
extern "C" int lme_ce_grad(void* logits, long long ld, const long long* labels, const float* lse, int T, int V,
                           int v0, float scale, const float* scale_dev, long long ignore_index, void* stream) {
    if (V % 8 || ld % 8) return LME_ERR_SHAPE;
    if (T == 0) return LME_OK;
    ce_grad_kernel<<<T, 1024, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(logits), ld,
                                                                      labels, lse, V, v0, scale, scale_dev, ignore_index);
    return LME_LAUNCH_OK();
}

extern "C" int lme_adamw(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p_lp, long long n,
                         float lr, float b1, float b2, float eps, float wd, int step, const float* gscale,
                         void* stream) {
    if (n == 0) return LME_OK;
    if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(g)) & 15)
        return LME_ERR_ALIGN;
    if (p_lp != nullptr && (reinterpret_cast<uintptr_t>(p_lp) & 15)) return LME_ERR_ALIGN;
    float bc1 = 1.f - powf(b1, static_cast<float>(step));
    float bc2 = 1.f - powf(b2, static_cast<float>(step));
    float bc2_sqrt = sqrtf(bc2);
    int grid = grid_for((n + 7) / 8, 256, 148 * 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g_is_bf16)
        adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, m, v, static_cast<const __nv_bfloat16*>(g),
                                                           static_cast<__nv_bfloat16*>(p_lp), n, lr, b1, b2, eps,
                                                           wd, bc1, bc2_sqrt, gscale);
    else
        adamw_kernel<float><<<grid, 256, 0, st>>>(p, m, v, static_cast<const float*>(g),
                                                   static_cast<__nv_bfloat16*>(p_lp), n, lr, b1, b2, eps, wd, bc1,
                                                   bc2_sqrt, gscale);
    return LME_LAUNCH_OK();
}

// out[0] (+)= sum(x^2).  `partials` is fp32 scratch of at least LME_SUMSQ_MAX_PARTIALS floats.
extern "C" int lme_sumsq(const void* x, int is_bf16, long long n, float* partials, float* out, int accumulate,
                         void* stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (reinterpret_cast<uintptr_t>(x) & 15) return LME_ERR_ALIGN;
    int grid = grid_for(n / 8 + 1, 256, LME_SUMSQ_MAX_PARTIALS);
    if (is_bf16) sumsq_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, partials);
    else sumsq_partial_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), n, partials);
    sum_partials_kernel<<<1, 256, 0, st>>>(partials, grid, out, accumulate);
    return LME_LAUNCH_OK();
}
// out (=|+=) scale * sum_r src[r]: the local half of a reduce-scatter whose slices were pulled into local memory by
// copy engines.  bf16 (or fp32) slices, fp32 accumulation.
struct SlicePtrs { const void* p[8]; };
template <typename T>
__global__ void reduce_slices_kernel(SlicePtrs src, int nsrc, T* __restrict__ out, long long n, float scale,
                                     int accumulate) {
    constexpr int VEC = 16 / sizeof(T);
    const long long nvec = n / VEC;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < nsrc; ++r) {
            if constexpr (sizeof(T) == 2) {
                float f[8];
                load8(static_cast<const __nv_bfloat16*>(src.p[r]) + i * 8, f);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += f[j];
            } else {
                const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(src.p[r]) + i * 4);
                acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
            }
        }
        if constexpr (sizeof(T) == 2) {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + i * 8;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = acc[j] * scale;
            if (accumulate) {
                float old[8];
                load8(o, old);
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] += old[j];
            }
            store8(o, f);
        } else {
            float* o = reinterpret_cast<float*>(out) + i * 4;
            float4 v = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
            if (accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(o);
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            *reinterpret_cast<float4*>(o) = v;
        }
    }
}

// n must be a multiple of 8 (bf16) / 4 (fp32) elements and every pointer 16-byte aligned.
extern "C" int lme_reduce_slices(const void* const* src, int nsrc, void* out, long long n, int is_bf16, float scale,
                                 int accumulate, void* stream) {
    if (nsrc < 1 || nsrc > 8 || n < 0 || (n % (is_bf16 ? 8 : 4))) return LME_ERR_SHAPE;
    if (n == 0) return LME_OK;
    SlicePtrs sp;
    for (int r = 0; r < 8; ++r) {
        sp.p[r] = r < nsrc ? src[r] : nullptr;
        if (r < nsrc && (reinterpret_cast<uintptr_t>(src[r]) & 15)) return LME_ERR_ALIGN;
    }
    if (reinterpret_cast<uintptr_t>(out) & 15) return LME_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int grid = grid_for(n / 8 + 1, 256, 148 * 8);
    if (is_bf16)
        reduce_slices_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(sp, nsrc, static_cast<__nv_bfloat16*>(out), n,
                                                                  scale, accumulate);
    else
        reduce_slices_kernel<float><<<grid, 256, 0, st>>>(sp, nsrc, static_cast<float*>(out), n, scale, accumulate);
    return LME_LAUNCH_OK();
}

extern "C" int lme_clip_coef(const float* sumsq, float max_norm, float* norm_out, float* coef_out, void* stream) {
    clip_coef_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, norm_out, coef_out);
    return LME_LAUNCH_OK();
}
