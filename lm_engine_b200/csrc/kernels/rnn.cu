// Vector-state multi-head RNN and GRU scans.
//
//   RNN: h_t = tanh(h_{t-1} W + x_t)
//   GRU: f = sigmoid(h_{t-1} Wf + xf_t), r = sigmoid(h_{t-1} Wr + xr_t), z = tanh((h_{t-1} * r) W + x_t),
//        h_t = f h_{t-1} + (1 - f) z
//
// The state of one (batch, head) is a vector of H values and W belongs to the head, so the batch elements of a head
// form the rows of a small matrix product.  One warp owns one head and up to 16 batch rows and walks the sequence
// alone, like the matrix-state kernel in m2rnn.cu whose helpers it shares: the state lives in mma.sync accumulator
// layout and re-enters the next product as the A operand without leaving registers; W (and W^T for the reverse
// pass) sit in registers as B fragments; the inputs of TC steps are staged by cp.async one chunk ahead.
//
// Every state is an output (y_t = h_t), so the backward pass needs no replay: it reads y, recomputes the gates of
// the GRU from h_{t-1} = y_{t-1}, and runs
//   RNN: d = clip(dh + dy_t); da = d (1 - h_t^2); dx_t = da; dh = da W^T
//   GRU: d = clip(dh + dy_t); daz = d (1 - f)(1 - z^2); dhr = daz W^T; daf = d (h_{t-1} - z) f (1 - f);
//        dar = dhr h_{t-1} r (1 - r); dh = d f + dhr r + daf Wf^T + dar Wr^T
// writing dx (, dxf, dxr and hr = h_{t-1} r); the weight gradients sum_t h_{t-1}^T da_t are batched GEMMs.
//
// Role of `xma.layers.rnn / gru` used by the reference (lm_engine/modeling_utils/sequence_mixer_blocks/
// rnn/module.py:189-197, gru/module.py:218-230; oracles rnn/op.py:13-46, gru/module.py:261-357).
namespace lme {
namespace rnn {

using m2::cp16;
using m2::cp_commit;
using m2::cp_wait;
using m2::mma16816;
using m2::pack2;
using m2::tanh_fast;
using m2::TC;
using m2::unpack2;

__device__ __forceinline__ float sigmoid_fast(float x) { return 0.5f * tanh_fast(0.5f * x) + 0.5f; }

template <int H>
struct Tile {                                   // TC steps x 16 batch rows, rows padded against bank conflicts
    __nv_bfloat16 d[2][TC][16][H + 8];
};

// Stages rows [0, rows) of steps tc0 .. tc0+TC-1 (those inside [t_lo, t_hi)) of a [B, S, heads, H] operand;
// `shift` reads step t - shift instead, and a step that falls before 0 reads `first` ([B, N, H], row stride fs).
template <int H>
__device__ __forceinline__ void stage(Tile<H>& dst, int stg, const __nv_bfloat16* base, long long row_stride,
                                      long long t_stride, int tc0, int t_lo, int t_hi, int rows, int lane,
                                      int shift = 0, const __nv_bfloat16* first = nullptr, long long fs = 0) {
    for (int i = lane; i < TC * 16 * (H / 8); i += 32) {
        const int part = i % (H / 8), row = (i / (H / 8)) % 16, st = i / (16 * (H / 8)), t = tc0 + st;
        if (t < t_lo || t >= t_hi || row >= rows) continue;
        const __nv_bfloat16* src = (t - shift >= 0) ? base + row * row_stride + (t - shift) * t_stride + 8 * part
                                                    : first + row * fs + 8 * part;
        cp16(&dst.d[stg][st][row][8 * part], src);
    }
}

template <int H>
__device__ __forceinline__ void read_tile(const Tile<H>& t, int stg, int st, int g, int qd, float (&out)[H / 8][4]) {
#pragma unroll
    for (int nt = 0; nt < H / 8; ++nt) {
        const float2 lo = unpack2(*reinterpret_cast<const uint32_t*>(&t.d[stg][st][g][8 * nt + 2 * qd]));
        const float2 hi = unpack2(*reinterpret_cast<const uint32_t*>(&t.d[stg][st][g + 8][8 * nt + 2 * qd]));
        out[nt][0] = lo.x, out[nt][1] = lo.y, out[nt][2] = hi.x, out[nt][3] = hi.y;
    }
}

// rows g / g+8 of an accumulator-layout block to a [B, S, N, H] bf16 tensor at (b0 + row, t, n)
template <int H>
__device__ __forceinline__ void write_rows(void* base, long long row0_off, long long b_stride, int g, int qd,
                                           bool ok_lo, bool ok_hi, const float (&v)[H / 8][4]) {
    __nv_bfloat16* p = static_cast<__nv_bfloat16*>(base) + row0_off + 2 * qd;
#pragma unroll
    for (int nt = 0; nt < H / 8; ++nt) {
        if (ok_lo) *reinterpret_cast<uint32_t*>(p + g * b_stride + 8 * nt) = pack2(v[nt][0], v[nt][1]);
        if (ok_hi) *reinterpret_cast<uint32_t*>(p + (g + 8) * b_stride + 8 * nt) = pack2(v[nt][2], v[nt][3]);
    }
}

template <int H>
__device__ __forceinline__ void pack_a(const float (&h)[H / 8][4], uint32_t (&a)[H / 16][4]) {
#pragma unroll
    for (int s = 0; s < H / 16; ++s) {
        a[s][0] = pack2(h[2 * s][0], h[2 * s][1]);
        a[s][1] = pack2(h[2 * s][2], h[2 * s][3]);
        a[s][2] = pack2(h[2 * s + 1][0], h[2 * s + 1][1]);
        a[s][3] = pack2(h[2 * s + 1][2], h[2 * s + 1][3]);
    }
}

// B fragments of a head's [H, H] matrix M (TRANSPOSED = false) or of M^T (true)
template <int H, bool TRANSPOSED>
__device__ __forceinline__ void load_b(const void* base, int head, int g, int qd, uint32_t (&f)[H / 16][H / 8][2]) {
    const __nv_bfloat16* M = static_cast<const __nv_bfloat16*>(base) + static_cast<long long>(head) * H * H;
#pragma unroll
    for (int s = 0; s < H / 16; ++s)
#pragma unroll
        for (int nt = 0; nt < H / 8; ++nt) {
            if (TRANSPOSED) {
                const __nv_bfloat16* row = M + (8 * nt + g) * H + 16 * s + 2 * qd;
                f[s][nt][0] = *reinterpret_cast<const uint32_t*>(row);
                f[s][nt][1] = *reinterpret_cast<const uint32_t*>(row + 8);
            } else {
                const int r = 16 * s + 2 * qd, c = 8 * nt + g;
                f[s][nt][0] = pack2(__bfloat162float(M[r * H + c]), __bfloat162float(M[(r + 1) * H + c]));
                f[s][nt][1] = pack2(__bfloat162float(M[(r + 8) * H + c]), __bfloat162float(M[(r + 9) * H + c]));
            }
        }
}

template <int H>
__device__ __forceinline__ void matmul(float (&acc)[H / 8][4], const uint32_t (&a)[H / 16][4],
                                       const uint32_t (&b)[H / 16][H / 8][2]) {
#pragma unroll
    for (int s = 0; s < H / 16; ++s)
#pragma unroll
        for (int nt = 0; nt < H / 8; ++nt) mma16816(acc[nt], a[s], b[s][nt][0], b[s][nt][1]);
}


struct Lane {
    int n, b0, rows, lane, g, qd;
    bool ok_lo, ok_hi;
};
__device__ __forceinline__ Lane locate(const LmeRnnArgs& p) {
    Lane w;
    w.n = blockIdx.x % p.N;
    w.b0 = (blockIdx.x / p.N) * 16;
    w.rows = min(16, p.B - w.b0);
    w.lane = threadIdx.x;
    w.g = w.lane >> 2;
    w.qd = w.lane & 3;
    w.ok_lo = w.g < w.rows;
    w.ok_hi = w.g + 8 < w.rows;
    return w;
}

template <int H, bool GRU>
__global__ void __launch_bounds__(32) rnn_fwd_kernel(const LmeRnnArgs p) {
    constexpr int NT = H / 8, KS = H / 16;
    extern __shared__ __align__(16) unsigned char rnn_smem[];
    Tile<H>* tiles = reinterpret_cast<Tile<H>*>(rnn_smem);   // x (, xf, xr)
    const Lane w = locate(p);
    const int g = w.g, qd = w.qd;
    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(p.x) + w.b0 * p.x_b + (w.n / (p.N / p.Nx)) * H;
    const __nv_bfloat16* xfb = nullptr;
    const __nv_bfloat16* xrb = nullptr;
    uint32_t Wz[KS][NT][2], Wff[GRU ? KS : 1][GRU ? NT : 1][2], Wrf[GRU ? KS : 1][GRU ? NT : 1][2];
    load_b<H, false>(p.W, w.n / (p.N / p.Nw), g, qd, Wz);
    if constexpr (GRU) {
        xfb = static_cast<const __nv_bfloat16*>(p.xf) + w.b0 * p.xf_b + (w.n / (p.N / p.Nxf)) * H;
        xrb = static_cast<const __nv_bfloat16*>(p.xr) + w.b0 * p.xr_b + (w.n / (p.N / p.Nxr)) * H;
        load_b<H, false>(p.Wf, w.n / (p.N / p.Nwf), g, qd, Wff);
        load_b<H, false>(p.Wr, w.n / (p.N / p.Nwr), g, qd, Wrf);
    }
    float h[NT][4];
    {
        const __nv_bfloat16* h0 = static_cast<const __nv_bfloat16*>(p.h0) + (static_cast<long long>(w.b0) * p.N + w.n) * H + 2 * qd;
        const long long rs = static_cast<long long>(p.N) * H;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float2 lo = w.ok_lo ? unpack2(*reinterpret_cast<const uint32_t*>(h0 + g * rs + 8 * nt)) : make_float2(0.f, 0.f);
            const float2 hi = w.ok_hi ? unpack2(*reinterpret_cast<const uint32_t*>(h0 + (g + 8) * rs + 8 * nt)) : make_float2(0.f, 0.f);
            h[nt][0] = lo.x, h[nt][1] = lo.y, h[nt][2] = hi.x, h[nt][3] = hi.y;
        }
    }
    auto issue = [&](int c) {
        const int stg = c & 1, tc0 = c * TC;
        stage<H>(tiles[0], stg, xb, p.x_b, p.x_t, tc0, 0, p.S, w.rows, w.lane);
        if constexpr (GRU) {
            stage<H>(tiles[1], stg, xfb, p.xf_b, p.xf_t, tc0, 0, p.S, w.rows, w.lane);
            stage<H>(tiles[2], stg, xrb, p.xr_b, p.xr_t, tc0, 0, p.S, w.rows, w.lane);
        }
        cp_commit();
    };
    const long long y_bs = static_cast<long long>(p.S) * p.N * H;
    const int nchunks = (p.S + TC - 1) / TC;
    issue(0);
    for (int c = 0; c < nchunks; ++c) {
        if (c + 1 < nchunks) {
            issue(c + 1);
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncwarp();
        const int stg = c & 1;
        for (int st = 0; st < TC; ++st) {
            const int t = c * TC + st;
            if (t >= p.S) break;
            float acc[NT][4];
            uint32_t a[KS][4];
            read_tile<H>(tiles[0], stg, st, g, qd, acc);
            pack_a<H>(h, a);
            if constexpr (GRU) {
                float fa[NT][4], ra[NT][4];
                read_tile<H>(tiles[1], stg, st, g, qd, fa);
                read_tile<H>(tiles[2], stg, st, g, qd, ra);
                matmul<H>(fa, a, Wff);
                matmul<H>(ra, a, Wrf);
                float hr[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        fa[nt][e] = sigmoid_fast(fa[nt][e]);
                        hr[nt][e] = h[nt][e] * sigmoid_fast(ra[nt][e]);
                    }
                uint32_t a2[KS][4];
                pack_a<H>(hr, a2);
                matmul<H>(acc, a2, Wz);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) h[nt][e] = fa[nt][e] * h[nt][e] + (1.f - fa[nt][e]) * tanh_fast(acc[nt][e]);
            } else {
                matmul<H>(acc, a, Wz);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) h[nt][e] = tanh_fast(acc[nt][e]);
            }
            write_rows<H>(p.y, ((static_cast<long long>(w.b0) * p.S + t) * p.N + w.n) * H, y_bs, g, qd, w.ok_lo, w.ok_hi, h);
        }
        __syncwarp();
    }
}

template <int H, bool GRU>
__global__ void __launch_bounds__(32) rnn_bwd_kernel(const LmeRnnArgs p) {
    constexpr int NT = H / 8, KS = H / 16;
    extern __shared__ __align__(16) unsigned char rnn_smem[];
    // RNN: [0] h_t (= y_t), [1] dy_t.   GRU: [0] h_{t-1} (y shifted by one step, h0 first), [1] dy_t, [2] x, [3] xf, [4] xr
    Tile<H>* tiles = reinterpret_cast<Tile<H>*>(rnn_smem);
    const Lane w = locate(p);
    const int g = w.g, qd = w.qd;
    const long long bs = static_cast<long long>(p.S) * p.N * H, ts = static_cast<long long>(p.N) * H;
    const long long out0 = (static_cast<long long>(w.b0) * p.S * p.N + w.n) * H;      // (b0, t = 0, n, 0) of [B, S, N, H]
    const __nv_bfloat16* yb = static_cast<const __nv_bfloat16*>(p.y) + out0;
    const __nv_bfloat16* dyb = static_cast<const __nv_bfloat16*>(p.dy) + out0;
    const __nv_bfloat16* h0b = static_cast<const __nv_bfloat16*>(p.h0) + (static_cast<long long>(w.b0) * p.N + w.n) * H;
    const __nv_bfloat16 *xb = nullptr, *xfb = nullptr, *xrb = nullptr;
    uint32_t WzT[KS][NT][2];
    uint32_t Wz[GRU ? KS : 1][GRU ? NT : 1][2], Wff[GRU ? KS : 1][GRU ? NT : 1][2], Wrf[GRU ? KS : 1][GRU ? NT : 1][2];
    uint32_t WfT[GRU ? KS : 1][GRU ? NT : 1][2], WrT[GRU ? KS : 1][GRU ? NT : 1][2];
    load_b<H, true>(p.W, w.n / (p.N / p.Nw), g, qd, WzT);
    if constexpr (GRU) {
        xb = static_cast<const __nv_bfloat16*>(p.x) + w.b0 * p.x_b + (w.n / (p.N / p.Nx)) * H;
        xfb = static_cast<const __nv_bfloat16*>(p.xf) + w.b0 * p.xf_b + (w.n / (p.N / p.Nxf)) * H;
        xrb = static_cast<const __nv_bfloat16*>(p.xr) + w.b0 * p.xr_b + (w.n / (p.N / p.Nxr)) * H;
        load_b<H, false>(p.W, w.n / (p.N / p.Nw), g, qd, Wz);
        load_b<H, false>(p.Wf, w.n / (p.N / p.Nwf), g, qd, Wff);
        load_b<H, false>(p.Wr, w.n / (p.N / p.Nwr), g, qd, Wrf);
        load_b<H, true>(p.Wf, w.n / (p.N / p.Nwf), g, qd, WfT);
        load_b<H, true>(p.Wr, w.n / (p.N / p.Nwr), g, qd, WrT);
    }
    float dh[NT][4];
    float* dhp = p.dh + (static_cast<long long>(w.b0) * p.N + w.n) * H + 2 * qd;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float2 lo = w.ok_lo ? *reinterpret_cast<const float2*>(dhp + g * ts + 8 * nt) : make_float2(0.f, 0.f);
        const float2 hi = w.ok_hi ? *reinterpret_cast<const float2*>(dhp + (g + 8) * ts + 8 * nt) : make_float2(0.f, 0.f);
        dh[nt][0] = lo.x, dh[nt][1] = lo.y, dh[nt][2] = hi.x, dh[nt][3] = hi.y;
    }
    auto issue = [&](int c) {
        const int stg = c & 1, tc0 = c * TC;
        if constexpr (GRU) {
            stage<H>(tiles[0], stg, yb, bs, ts, tc0, 0, p.S, w.rows, w.lane, 1, h0b, ts);
            stage<H>(tiles[2], stg, xb, p.x_b, p.x_t, tc0, 0, p.S, w.rows, w.lane);
            stage<H>(tiles[3], stg, xfb, p.xf_b, p.xf_t, tc0, 0, p.S, w.rows, w.lane);
            stage<H>(tiles[4], stg, xrb, p.xr_b, p.xr_t, tc0, 0, p.S, w.rows, w.lane);
        } else {
            stage<H>(tiles[0], stg, yb, bs, ts, tc0, 0, p.S, w.rows, w.lane);
        }
        stage<H>(tiles[1], stg, dyb, bs, ts, tc0, 0, p.S, w.rows, w.lane);
        cp_commit();
    };
    const int nchunks = (p.S + TC - 1) / TC;
    issue(nchunks - 1);
    for (int c = nchunks - 1; c >= 0; --c) {
        if (c > 0) {
            issue(c - 1);
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncwarp();
        const int stg = c & 1;
        for (int st = TC - 1; st >= 0; --st) {
            const int t = c * TC + st;
            if (t >= p.S) continue;
            const long long o = out0 + t * ts;
            float d[NT][4], hv[NT][4];
            read_tile<H>(tiles[1], stg, st, g, qd, d);
            read_tile<H>(tiles[0], stg, st, g, qd, hv);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    d[nt][e] += dh[nt][e];
                    if (p.clip > 0.f) d[nt][e] = fminf(fmaxf(d[nt][e], -p.clip), p.clip);
                }
            uint32_t a[KS][4];
            if constexpr (!GRU) {
                float da[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        da[nt][e] = d[nt][e] * (1.f - hv[nt][e] * hv[nt][e]);
                        dh[nt][e] = 0.f;
                    }
                write_rows<H>(p.dx, o, bs, g, qd, w.ok_lo, w.ok_hi, da);
                pack_a<H>(da, a);
                matmul<H>(dh, a, WzT);
            } else {
                float fa[NT][4], ra[NT][4], za[NT][4], hr[NT][4];
                read_tile<H>(tiles[3], stg, st, g, qd, fa);
                read_tile<H>(tiles[4], stg, st, g, qd, ra);
                read_tile<H>(tiles[2], stg, st, g, qd, za);
                pack_a<H>(hv, a);
                matmul<H>(fa, a, Wff);
                matmul<H>(ra, a, Wrf);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        fa[nt][e] = sigmoid_fast(fa[nt][e]);
                        ra[nt][e] = sigmoid_fast(ra[nt][e]);
                        hr[nt][e] = hv[nt][e] * ra[nt][e];
                    }
                write_rows<H>(p.hr, o, bs, g, qd, w.ok_lo, w.ok_hi, hr);
                pack_a<H>(hr, a);
                matmul<H>(za, a, Wz);
                float daz[NT][4], dhr[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        za[nt][e] = tanh_fast(za[nt][e]);
                        daz[nt][e] = d[nt][e] * (1.f - fa[nt][e]) * (1.f - za[nt][e] * za[nt][e]);
                        dhr[nt][e] = 0.f;
                    }
                write_rows<H>(p.dx, o, bs, g, qd, w.ok_lo, w.ok_hi, daz);
                pack_a<H>(daz, a);
                matmul<H>(dhr, a, WzT);
                float daf[NT][4], dar[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float f = fa[nt][e], r = ra[nt][e];
                        daf[nt][e] = d[nt][e] * (hv[nt][e] - za[nt][e]) * f * (1.f - f);
                        dar[nt][e] = dhr[nt][e] * hv[nt][e] * r * (1.f - r);
                        dh[nt][e] = d[nt][e] * f + dhr[nt][e] * r;
                    }
                write_rows<H>(p.dxf, o, bs, g, qd, w.ok_lo, w.ok_hi, daf);
                write_rows<H>(p.dxr, o, bs, g, qd, w.ok_lo, w.ok_hi, dar);
                pack_a<H>(daf, a);
                matmul<H>(dh, a, WfT);
                pack_a<H>(dar, a);
                matmul<H>(dh, a, WrT);
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        if (w.ok_lo) *reinterpret_cast<float2*>(dhp + g * ts + 8 * nt) = make_float2(dh[nt][0], dh[nt][1]);
        if (w.ok_hi) *reinterpret_cast<float2*>(dhp + (g + 8) * ts + 8 * nt) = make_float2(dh[nt][2], dh[nt][3]);
    }
}

template <int H, bool GRU>
int launch(const LmeRnnArgs& p, int mode, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(p.N) * ((p.B + 15) / 16);
    const int ntiles = mode == 0 ? (GRU ? 3 : 1) : (GRU ? 5 : 2);
    const int bytes = ntiles * static_cast<int>(sizeof(Tile<H>));
    static int configured[2] = {0, 0};
    if (configured[mode] < bytes) {
        const cudaError_t e = mode == 0
            ? cudaFuncSetAttribute(rnn_fwd_kernel<H, GRU>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)
            : cudaFuncSetAttribute(rnn_bwd_kernel<H, GRU>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return -4;
        configured[mode] = bytes;
    }
    if (mode == 0) rnn_fwd_kernel<H, GRU><<<grid, 32, bytes, stream>>>(p);
    else rnn_bwd_kernel<H, GRU><<<grid, 32, bytes, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace rnn
}  // namespace lme

extern "C" int lme_rnn(const LmeRnnArgs* args, int mode, void* stream) {
    const LmeRnnArgs& p = *args;
    if (mode < 0 || mode > 1 || p.B <= 0 || p.S <= 0 || p.N <= 0) return -1;
    if (p.N % p.Nx || p.N % p.Nw) return -1;
    if (p.gru && (p.N % p.Nxf || p.N % p.Nxr || p.N % p.Nwf || p.N % p.Nwr)) return -1;
    if (static_cast<long long>(p.N) * ((p.B + 15) / 16) > 2147483647ll) return -6;
    auto mis = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
    if (mis(p.x) || mis(p.W) || mis(p.h0) || mis(p.y) || (p.x_b | p.x_t) % 8) return -2;
    if (p.gru && (mis(p.xf) || mis(p.xr) || mis(p.Wf) || mis(p.Wr) || (p.xf_b | p.xf_t | p.xr_b | p.xr_t) % 8)) return -2;
    if (mode == 1 && (mis(p.dy) || mis(p.dx) || !p.dh)) return -2;
    if (mode == 1 && p.gru && (mis(p.dxf) || mis(p.dxr) || mis(p.hr))) return -2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p.gru) {
        switch (p.H) {
            case 16: return lme::rnn::launch<16, true>(p, mode, st);
            case 32: return lme::rnn::launch<32, true>(p, mode, st);
            default: return -1;
        }
    }
    switch (p.H) {
        case 16: return lme::rnn::launch<16, false>(p, mode, st);
        case 32: return lme::rnn::launch<32, false>(p, mode, st);
        case 64: return lme::rnn::launch<64, false>(p, mode, st);
        default: return -1;
    }
}
