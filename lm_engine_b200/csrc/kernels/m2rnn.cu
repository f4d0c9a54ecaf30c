// Matrix-state RNN (M2RNN) scan:   z_t = tanh(h_{t-1} W + k_t (x) v_t),   h_t = f_t h_{t-1} + (1 - f_t) z_t,
// y_t = q_t . h_t      with h [K, V] per (batch, head), W [V, V], f_t a scalar in (0, 1).
//
// The recurrence is sequential in t and non-linear, so the only parallelism is over (batch, head) and over the ROWS
// of h: row i of h_t depends on row i of h_{t-1} only.  One warp owns 16 rows of one (batch, head) state and walks
// the sequence alone - no block-level synchronisation anywhere.  Per step the warp issues V/16 * V/8 tensor-core
// instructions (mma.sync m16n8k16, bf16 operands, fp32 accumulate); the state stays in fp32 accumulator-layout
// registers, and because the accumulator layout of two adjacent 8-column tiles IS the A-operand layout of one
// 16-deep k-step, the state re-enters the next step's product without leaving the register file.  tcgen05 is the
// wrong tool here: its minimum tile is 64 x N x 16 issued asynchronously through shared memory / TMEM, and the chain
// h_t -> h_{t+1} would pay that round trip 4096 times; the per-step latency of mma.sync is ~30 cycles.
//
// Inputs of TC consecutive steps are staged in shared memory by cp.async one chunk ahead of their use.
//
// Training keeps memory bounded by segments: the forward pass stores an fp32 snapshot of the state at the start of
// every segment; the backward pass walks the segments right to left and, per segment, (1) re-runs the forward
// recurrence from the snapshot writing h_{t-1} and z_t in bf16 (SAVE mode), (2) runs the reverse recurrence
//      dh_t   = clip(dh_t + q_t (x) dy_t)                      dq_t = h_t dy_t
//      df_t   = sum(dh_t * (h_{t-1} - z_t))                    da_t = (1 - f_t) dh_t (1 - z_t^2)
//      dk_t   = da_t v_t            dv_t = da_t^T k_t          dh_{t-1} = f_t dh_t + da_t W^T
//     overwriting z_t with da_t, and (3) leaves dW = sum_t h_{t-1}^T da_t to one batched GEMM over the segment.
// Column sums (y, dv) are partial per 16-row block and written as such; the caller adds the K/16 partials.
//
// Role of the `m2rnn` kernel of the XMA package used by the reference
// (lm_engine/modeling_utils/sequence_mixer_blocks/m2rnn/module.py:56-67; oracle m2rnn/op.py:11-66).
namespace lme {
namespace m2 {

constexpr int TC = 8;   // time steps per staged chunk

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ float2 unpack2(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void cp16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
                 "l"(src));
}
__device__ __forceinline__ void cp4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(
                     static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
                 "l"(src));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// Sum over the 8 lane groups (lane bits 2..4) of N_ x 2 per-thread values.  While more than one tile is left each
// exchange halves the tiles a lane keeps (reduce-scatter), afterwards it is a plain butterfly.  On return `out` is
// the finished pair of tile `nt` on the lanes with `writer` still true.
template <int N_, int BIT>
struct ColReduce {
    static __device__ __forceinline__ void run(float (&x)[N_][2], int lane, float2& out, int& nt, bool& writer) {
        const bool hi = (lane & BIT) != 0;
        if constexpr (N_ > 1) {
            float y[N_ / 2][2];
#pragma unroll
            for (int i = 0; i < N_ / 2; ++i)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float keep = hi ? x[i + N_ / 2][e] : x[i][e];
                    const float send = hi ? x[i][e] : x[i + N_ / 2][e];
                    y[i][e] = keep + __shfl_xor_sync(0xffffffffu, send, BIT);
                }
            nt = nt * 2 + (hi ? 1 : 0);
            if constexpr (BIT > 4) {
                ColReduce<N_ / 2, BIT / 2>::run(y, lane, out, nt, writer);
            } else {
                static_assert(N_ == 2 || BIT > 4, "at most 8 column tiles");
                out = make_float2(y[0][0], y[0][1]);
            }
        } else {
            x[0][0] += __shfl_xor_sync(0xffffffffu, x[0][0], BIT);
            x[0][1] += __shfl_xor_sync(0xffffffffu, x[0][1], BIT);
            if (hi) writer = false;
            if constexpr (BIT > 4) {
                ColReduce<1, BIT / 2>::run(x, lane, out, nt, writer);
            } else {
                out = make_float2(x[0][0], x[0][1]);
            }
        }
    }
};

// transposes an 8 x 8 block of 16-bit values held as a fragment (lane (g, qd) holds row g, columns 2qd, 2qd+1)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

__device__ __forceinline__ float quad_sum(float x) {
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}


struct Where {
    int b, n, rb, lane, g, qd;
    long long state_off;   // first element of this warp's 16 rows in a [B, N, K, V] tensor
};

template <int V>
__device__ __forceinline__ Where locate(const LmeM2rnnArgs& p) {
    Where w;
    const int RB = p.K / 16;
    w.rb = blockIdx.x % RB;
    w.n = (blockIdx.x / RB) % p.N;
    w.b = blockIdx.x / (RB * p.N);
    w.lane = threadIdx.x;
    w.g = w.lane >> 2;
    w.qd = w.lane & 3;
    w.state_off = ((static_cast<long long>(w.b) * p.N + w.n) * p.K + 16 * w.rb) * V;
    return w;
}

// accumulator-layout load / store of a 16 x V fp32 block whose first row starts at `base`
template <int V>
__device__ __forceinline__ void load_state(const float* base, const Where& w, float (&h)[V / 8][4]) {
#pragma unroll
    for (int nt = 0; nt < V / 8; ++nt) {
        const float2 lo = *reinterpret_cast<const float2*>(base + w.g * V + 8 * nt + 2 * w.qd);
        const float2 hi = *reinterpret_cast<const float2*>(base + (w.g + 8) * V + 8 * nt + 2 * w.qd);
        h[nt][0] = lo.x, h[nt][1] = lo.y, h[nt][2] = hi.x, h[nt][3] = hi.y;
    }
}
template <int V>
__device__ __forceinline__ void store_state(float* base, const Where& w, const float (&h)[V / 8][4]) {
#pragma unroll
    for (int nt = 0; nt < V / 8; ++nt) {
        *reinterpret_cast<float2*>(base + w.g * V + 8 * nt + 2 * w.qd) = make_float2(h[nt][0], h[nt][1]);
        *reinterpret_cast<float2*>(base + (w.g + 8) * V + 8 * nt + 2 * w.qd) = make_float2(h[nt][2], h[nt][3]);
    }
}

// SAVE = false: forward pass (y partials, snapshots, final state).  SAVE = true: replay of one segment from its
// snapshot that records the bf16 operand h_{t-1} and z_t of every step.
template <int V, bool SAVE>
__global__ void __launch_bounds__(32) m2rnn_fwd_kernel(const LmeM2rnnArgs p) {
    constexpr int NT = V / 8, KS = V / 16;
    __shared__ __align__(16) __nv_bfloat16 qs[2][TC][16];
    __shared__ __align__(16) __nv_bfloat16 ks[2][TC][16];
    __shared__ __align__(16) __nv_bfloat16 vs[2][TC][V];
    __shared__ __align__(16) float fs[2][TC];
    const Where w = locate<V>(p);
    const int lane = w.lane, g = w.g, qd = w.qd;
    const __nv_bfloat16* qbase =
        static_cast<const __nv_bfloat16*>(p.q) + w.b * p.q_b + (w.n / (p.N / p.Nq)) * p.K + 16 * w.rb;
    const __nv_bfloat16* kbase =
        static_cast<const __nv_bfloat16*>(p.k) + w.b * p.k_b + (w.n / (p.N / p.Nk)) * p.K + 16 * w.rb;
    const __nv_bfloat16* vbase = static_cast<const __nv_bfloat16*>(p.v) + w.b * p.v_b + (w.n / (p.N / p.Nv)) * V;
    const float* fbase = p.f + static_cast<long long>(w.b) * p.S * p.Nf + w.n / (p.N / p.Nf);

    // B-operand fragments of W: b0 = W[16s+2qd .. +1][8nt+g], b1 = W[16s+2qd+8 .. +9][8nt+g]
    uint32_t Wf[KS][NT][2];
    {
        const __nv_bfloat16* Wn = static_cast<const __nv_bfloat16*>(p.W) + static_cast<long long>(w.n / (p.N / p.Nw)) * V * V;
#pragma unroll
        for (int s = 0; s < KS; ++s)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int r = 16 * s + 2 * qd, c = 8 * nt + g;
                Wf[s][nt][0] = pack2(__bfloat162float(Wn[r * V + c]), __bfloat162float(Wn[(r + 1) * V + c]));
                Wf[s][nt][1] = pack2(__bfloat162float(Wn[(r + 8) * V + c]), __bfloat162float(Wn[(r + 9) * V + c]));
            }
    }

    const int t_begin = SAVE ? p.t0 : 0;
    const int t_end = SAVE ? p.t0 + p.T : p.S;
    const int nseg = (p.S + p.seg_len - 1) / p.seg_len;
    const long long KV = static_cast<long long>(p.K) * V;
    float h[NT][4];
    {
        const float* src = nullptr;
        if (SAVE) src = p.ckpt + ((static_cast<long long>(w.b) * p.N + w.n) * nseg + p.t0 / p.seg_len) * KV + 16 * w.rb * V;
        else if (p.h0) src = p.h0 + w.state_off;
        if (src) load_state<V>(src, w, h);
        else
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) h[nt][0] = h[nt][1] = h[nt][2] = h[nt][3] = 0.f;
    }

    auto issue = [&](int c) {
        const int stage = c & 1, tc0 = t_begin + c * TC;
        for (int i = lane; i < TC * 2; i += 32) {
            const int st = i >> 1, part = i & 1, t = tc0 + st;
            if (t < t_end) {
                cp16(&ks[stage][st][8 * part], kbase + t * p.k_t + 8 * part);
                if (!SAVE) cp16(&qs[stage][st][8 * part], qbase + t * p.q_t + 8 * part);
            }
        }
        for (int i = lane; i < TC * (V / 8); i += 32) {
            const int st = i / (V / 8), part = i % (V / 8), t = tc0 + st;
            if (t < t_end) cp16(&vs[stage][st][8 * part], vbase + t * p.v_t + 8 * part);
        }
        if (lane < TC && tc0 + lane < t_end) cp4(&fs[stage][lane], fbase + static_cast<long long>(tc0 + lane) * p.Nf);
        cp_commit();
    };

    const long long rec0 = SAVE ? ((static_cast<long long>(w.b) * p.N + w.n) * p.Tcap * p.K + 16 * w.rb + g) * V + 2 * qd : 0;
    int next_ckpt = (!SAVE && p.ckpt) ? 0 : -1;
    float* ckpt_ptr = p.ckpt ? p.ckpt + (static_cast<long long>(w.b) * p.N + w.n) * nseg * KV + 16 * w.rb * V : nullptr;
    // (rb, b, t_begin, n, 0) of y_part [RB, B, S, N, V]; advanced by one token per step
    float* y_ptr = SAVE ? nullptr : p.y_part + (((static_cast<long long>(w.rb) * p.B + w.b) * p.S + t_begin) * p.N + w.n) * V;
    const long long y_step = static_cast<long long>(p.N) * V;
    const int nchunks = (t_end - t_begin + TC - 1) / TC;
    if (nchunks > 0) issue(0);
    for (int c = 0; c < nchunks; ++c) {
        if (c + 1 < nchunks) {
            issue(c + 1);
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncwarp();
        const int stage = c & 1;
        // two steps per trip (small states): the output reduction and stores of one step overlap the dependent
        // product -> tanh chain of the next
#pragma unroll(V <= 32 ? 2 : 1)
        for (int st = 0; st < TC; ++st) {
            const int t = t_begin + c * TC + st;
            if (t >= t_end) break;
            if (!SAVE && t == next_ckpt) {    // t_begin = 0: snapshots at 0, seg_len, 2 seg_len, ...
                store_state<V>(ckpt_ptr, w, h);
                ckpt_ptr += KV;
                next_ckpt += p.seg_len;
            }
            const float k0 = __bfloat162float(ks[stage][st][g]), k1 = __bfloat162float(ks[stage][st][g + 8]);
            const float gt = fs[stage][st];
            uint32_t a[KS][4];
#pragma unroll
            for (int s = 0; s < KS; ++s) {
                a[s][0] = pack2(h[2 * s][0], h[2 * s][1]);
                a[s][1] = pack2(h[2 * s][2], h[2 * s][3]);
                a[s][2] = pack2(h[2 * s + 1][0], h[2 * s + 1][1]);
                a[s][3] = pack2(h[2 * s + 1][2], h[2 * s + 1][3]);
            }
            // element offset of (row g, column 2 qd) of this step's 16 x V tile in the [B, N, Tcap, K, V] records
            const long long rec = rec0 + static_cast<long long>(t - t_begin) * KV;
            if (SAVE) {
                __nv_bfloat16* hp = static_cast<__nv_bfloat16*>(p.hprev) + rec;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    *reinterpret_cast<uint32_t*>(hp + 8 * nt) = a[nt >> 1][(nt & 1) * 2];
                    *reinterpret_cast<uint32_t*>(hp + 8 * V + 8 * nt) = a[nt >> 1][(nt & 1) * 2 + 1];
                }
            }
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float2 vv = unpack2(*reinterpret_cast<const uint32_t*>(&vs[stage][st][8 * nt + 2 * qd]));
                acc[nt][0] = k0 * vv.x, acc[nt][1] = k0 * vv.y, acc[nt][2] = k1 * vv.x, acc[nt][3] = k1 * vv.y;
            }
#pragma unroll
            for (int s = 0; s < KS; ++s)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma16816(acc[nt], a[s], Wf[s][nt][0], Wf[s][nt][1]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float z[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    z[e] = tanh_fast(acc[nt][e]);
                    h[nt][e] = gt * h[nt][e] + (1.f - gt) * z[e];
                }
                if (SAVE) {
                    __nv_bfloat16* zp = static_cast<__nv_bfloat16*>(p.z) + rec + 8 * nt;
                    *reinterpret_cast<uint32_t*>(zp) = pack2(z[0], z[1]);
                    *reinterpret_cast<uint32_t*>(zp + 8 * V) = pack2(z[2], z[3]);
                }
            }
            if (!SAVE) {
                const float q0 = __bfloat162float(qs[stage][st][g]), q1 = __bfloat162float(qs[stage][st][g + 8]);
                float part[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    part[nt][0] = q0 * h[nt][0] + q1 * h[nt][2];
                    part[nt][1] = q0 * h[nt][1] + q1 * h[nt][3];
                }
                float2 out;
                int nt_out = 0;
                bool writer = true;
                ColReduce<NT, 16>::run(part, lane, out, nt_out, writer);
                if (writer) *reinterpret_cast<float2*>(y_ptr + 8 * nt_out + 2 * qd) = out;
                y_ptr += y_step;
            }
        }
        __syncwarp();
    }
    if (!SAVE && p.h_out) store_state<V>(p.h_out + w.state_off, w, h);
}

template <int V>
struct BwdSmem {
    static constexpr int LD = V + 8;   // padded row: the 8 row groups of a fragment read hit 32 different banks
    __nv_bfloat16 hp[2][TC][16][LD];
    __nv_bfloat16 z[2][TC][16][LD];
    __nv_bfloat16 q[2][TC][16];
    __nv_bfloat16 k[2][TC][16];
    __nv_bfloat16 v[2][TC][V];
    __nv_bfloat16 dy[2][TC][V];
    float f[2][TC];
};

template <int V>
__global__ void __launch_bounds__(32) m2rnn_bwd_kernel(const LmeM2rnnArgs p) {
    constexpr int NT = V / 8, KS = V / 16;
    extern __shared__ __align__(16) unsigned char m2_smem[];
    BwdSmem<V>& sm = *reinterpret_cast<BwdSmem<V>*>(m2_smem);
    const Where w = locate<V>(p);
    const int lane = w.lane, g = w.g, qd = w.qd;
    const __nv_bfloat16* qbase =
        static_cast<const __nv_bfloat16*>(p.q) + w.b * p.q_b + (w.n / (p.N / p.Nq)) * p.K + 16 * w.rb;
    const __nv_bfloat16* kbase =
        static_cast<const __nv_bfloat16*>(p.k) + w.b * p.k_b + (w.n / (p.N / p.Nk)) * p.K + 16 * w.rb;
    const __nv_bfloat16* vbase = static_cast<const __nv_bfloat16*>(p.v) + w.b * p.v_b + (w.n / (p.N / p.Nv)) * V;
    const __nv_bfloat16* dybase =
        static_cast<const __nv_bfloat16*>(p.dy) + (static_cast<long long>(w.b) * p.S * p.N + w.n) * V;
    const float* fbase = p.f + static_cast<long long>(w.b) * p.S * p.Nf + w.n / (p.N / p.Nf);
    // first element of this warp's rows in step (t - t0) of the [B, N, Tcap, K, V] records
    const long long rec0 = ((static_cast<long long>(w.b) * p.N + w.n) * p.Tcap * p.K + 16 * w.rb) * V;
    const long long rec_step = static_cast<long long>(p.K) * V;
    const __nv_bfloat16* hprec = static_cast<const __nv_bfloat16*>(p.hprev) + rec0;
    __nv_bfloat16* zrec = static_cast<__nv_bfloat16*>(p.z) + rec0;

    // B-operand fragments of W^T: b0 = W[8nt+g][16s+2qd .. +1], b1 = W[8nt+g][16s+2qd+8 .. +9]
    uint32_t WTf[KS][NT][2];
    {
        const __nv_bfloat16* Wn = static_cast<const __nv_bfloat16*>(p.W) + static_cast<long long>(w.n / (p.N / p.Nw)) * V * V;
#pragma unroll
        for (int s = 0; s < KS; ++s)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const __nv_bfloat16* row = Wn + (8 * nt + g) * V + 16 * s + 2 * qd;
                WTf[s][nt][0] = *reinterpret_cast<const uint32_t*>(row);
                WTf[s][nt][1] = *reinterpret_cast<const uint32_t*>(row + 8);
            }
    }
    float dh[NT][4];
    load_state<V>(p.dh + w.state_off, w, dh);
    // dW of this warp's rows over this launch's steps, accumulator layout: [m-tile of i][n-tile of j]
    constexpr bool DW_IN_KERNEL = V <= 32;
    float dWacc[DW_IN_KERNEL ? KS : 1][DW_IN_KERNEL ? NT : 1][4];
#pragma unroll
    for (int mt = 0; mt < (DW_IN_KERNEL ? KS : 1); ++mt)
#pragma unroll
        for (int nt = 0; nt < (DW_IN_KERNEL ? NT : 1); ++nt) dWacc[mt][nt][0] = dWacc[mt][nt][1] = dWacc[mt][nt][2] = dWacc[mt][nt][3] = 0.f;

    const int t_begin = p.t0, t_end = p.t0 + p.T;
    auto issue = [&](int c) {
        const int stage = c & 1, tc0 = t_begin + c * TC;
        for (int i = lane; i < TC * 2; i += 32) {
            const int st = i >> 1, part = i & 1, t = tc0 + st;
            if (t < t_end) {
                cp16(&sm.k[stage][st][8 * part], kbase + t * p.k_t + 8 * part);
                cp16(&sm.q[stage][st][8 * part], qbase + t * p.q_t + 8 * part);
            }
        }
        for (int i = lane; i < TC * (V / 8); i += 32) {
            const int st = i / (V / 8), part = i % (V / 8), t = tc0 + st;
            if (t < t_end) {
                cp16(&sm.v[stage][st][8 * part], vbase + t * p.v_t + 8 * part);
                cp16(&sm.dy[stage][st][8 * part], dybase + static_cast<long long>(t) * p.N * V + 8 * part);
            }
        }
        for (int i = lane; i < TC * 16 * (V / 8); i += 32) {
            const int part = i % (V / 8), row = (i / (V / 8)) % 16, st = i / (16 * (V / 8)), t = tc0 + st;
            if (t < t_end) {
                const long long off = (t - p.t0) * rec_step + row * V + 8 * part;
                cp16(&sm.hp[stage][st][row][8 * part], hprec + off);
                cp16(&sm.z[stage][st][row][8 * part], zrec + off);
            }
        }
        if (lane < TC && tc0 + lane < t_end) cp4(&sm.f[stage][lane], fbase + static_cast<long long>(tc0 + lane) * p.Nf);
        cp_commit();
    };

    // output pointers of the last step of this launch; they walk backwards with the scan
    const long long qk_step = static_cast<long long>(p.N) * p.K;
    float* dq_ptr = p.dq + ((static_cast<long long>(w.b) * p.S + (t_end - 1)) * p.N + w.n) * p.K + 16 * w.rb + g;
    float* dk_ptr = p.dk + (dq_ptr - p.dq);
    float* df_ptr = p.df_part + ((static_cast<long long>(w.rb) * p.B + w.b) * p.S + (t_end - 1)) * p.N + w.n;
    float* dv_ptr = p.dv_part + (df_ptr - p.df_part) * V;
    const int nchunks = (t_end - t_begin + TC - 1) / TC;
    if (nchunks > 0) issue(nchunks - 1);
    for (int c = nchunks - 1; c >= 0; --c) {
        if (c > 0) {
            issue(c - 1);
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncwarp();
        const int stage = c & 1;
#pragma unroll(V <= 32 ? 2 : 1)
        for (int st = TC - 1; st >= 0; --st) {
            const int t = t_begin + c * TC + st;
            if (t >= t_end) continue;
            const float gt = sm.f[stage][st];
            const float q0 = __bfloat162float(sm.q[stage][st][g]), q1 = __bfloat162float(sm.q[stage][st][g + 8]);
            const float k0 = __bfloat162float(sm.k[stage][st][g]), k1 = __bfloat162float(sm.k[stage][st][g + 8]);
            float dq0 = 0.f, dq1 = 0.f, dk0 = 0.f, dk1 = 0.f, dfp = 0.f;
            float dvp[NT][2], acc[NT][4];
            uint32_t a[KS][4];
            uint32_t hraw[NT][2];
            __nv_bfloat16* zout = zrec + (t - p.t0) * rec_step + g * V + 2 * qd;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float2 dyv = unpack2(*reinterpret_cast<const uint32_t*>(&sm.dy[stage][st][8 * nt + 2 * qd]));
                const float2 vv = unpack2(*reinterpret_cast<const uint32_t*>(&sm.v[stage][st][8 * nt + 2 * qd]));
                hraw[nt][0] = *reinterpret_cast<const uint32_t*>(&sm.hp[stage][st][g][8 * nt + 2 * qd]);
                hraw[nt][1] = *reinterpret_cast<const uint32_t*>(&sm.hp[stage][st][g + 8][8 * nt + 2 * qd]);
                const float2 hp01 = unpack2(hraw[nt][0]);
                const float2 hp23 = unpack2(hraw[nt][1]);
                const float2 z01 = unpack2(*reinterpret_cast<const uint32_t*>(&sm.z[stage][st][g][8 * nt + 2 * qd]));
                const float2 z23 = unpack2(*reinterpret_cast<const uint32_t*>(&sm.z[stage][st][g + 8][8 * nt + 2 * qd]));
                const float hpv[4] = {hp01.x, hp01.y, hp23.x, hp23.y};
                const float zv[4] = {z01.x, z01.y, z23.x, z23.y};
                const float dyc[4] = {dyv.x, dyv.y, dyv.x, dyv.y};
                const float vc[4] = {vv.x, vv.y, vv.x, vv.y};
                float da[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float d = dh[nt][e] + (e < 2 ? q0 : q1) * dyc[e];
                    if (p.clip > 0.f) d = fminf(fmaxf(d, -p.clip), p.clip);
                    const float ht = gt * hpv[e] + (1.f - gt) * zv[e];
                    if (e < 2) dq0 += ht * dyc[e];
                    else dq1 += ht * dyc[e];
                    dfp += d * (hpv[e] - zv[e]);
                    da[e] = (1.f - gt) * d * (1.f - zv[e] * zv[e]);
                    if (e < 2) dk0 += da[e] * vc[e];
                    else dk1 += da[e] * vc[e];
                    acc[nt][e] = gt * d;
                }
                dvp[nt][0] = k0 * da[0] + k1 * da[2];
                dvp[nt][1] = k0 * da[1] + k1 * da[3];
                const uint32_t p01 = pack2(da[0], da[1]), p23 = pack2(da[2], da[3]);
                if (!DW_IN_KERNEL) {      // the caller forms dW = sum h_{t-1}^T da_t from the records
                    *reinterpret_cast<uint32_t*>(zout + 8 * nt) = p01;
                    *reinterpret_cast<uint32_t*>(zout + 8 * V + 8 * nt) = p23;
                }
                a[nt >> 1][(nt & 1) * 2] = p01;
                a[nt >> 1][(nt & 1) * 2 + 1] = p23;
            }
            if (DW_IN_KERNEL) {
                // dW[i][j] += sum_rows h_{t-1}[row][i] da[row][j]: both operands are the register pairs above with
                // their 8 x 8 blocks transposed (rows become the contraction index)
                uint32_t bt[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    bt[nt][0] = movmatrix_trans(a[nt >> 1][(nt & 1) * 2]);
                    bt[nt][1] = movmatrix_trans(a[nt >> 1][(nt & 1) * 2 + 1]);
                }
#pragma unroll
                for (int mt = 0; mt < KS; ++mt) {
                    uint32_t at[4];
                    at[0] = movmatrix_trans(hraw[2 * mt][0]);
                    at[1] = movmatrix_trans(hraw[2 * mt + 1][0]);
                    at[2] = movmatrix_trans(hraw[2 * mt][1]);
                    at[3] = movmatrix_trans(hraw[2 * mt + 1][1]);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) mma16816(dWacc[DW_IN_KERNEL ? mt : 0][DW_IN_KERNEL ? nt : 0], at, bt[nt][0], bt[nt][1]);
                }
            }
            dq0 = quad_sum(dq0), dq1 = quad_sum(dq1), dk0 = quad_sum(dk0), dk1 = quad_sum(dk1);
            if (qd == 0) dq_ptr[0] = dq0, dq_ptr[8] = dq1, dk_ptr[0] = dk0, dk_ptr[8] = dk1;
            dq_ptr -= qk_step, dk_ptr -= qk_step;
            dfp = quad_sum(dfp);
            dfp += __shfl_xor_sync(0xffffffffu, dfp, 4);
            dfp += __shfl_xor_sync(0xffffffffu, dfp, 8);
            dfp += __shfl_xor_sync(0xffffffffu, dfp, 16);
            if (lane == 0) *df_ptr = dfp;
            {
                float2 out;
                int nt_out = 0;
                bool writer = true;
                ColReduce<NT, 16>::run(dvp, lane, out, nt_out, writer);
                if (writer) *reinterpret_cast<float2*>(dv_ptr + 8 * nt_out + 2 * qd) = out;
            }
            df_ptr -= p.N, dv_ptr -= static_cast<long long>(p.N) * V;
#pragma unroll
            for (int s = 0; s < KS; ++s)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma16816(acc[nt], a[s], WTf[s][nt][0], WTf[s][nt][1]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) dh[nt][e] = acc[nt][e];
        }
        __syncwarp();
    }
    store_state<V>(p.dh + w.state_off, w, dh);
    if (DW_IN_KERNEL) {
        // dW_part [B, N, RB, V, V] accumulates over the launches of one backward pass (the caller zeroes it)
        float* out = p.dW_part + ((static_cast<long long>(w.b) * p.N + w.n) * (p.K / 16) + w.rb) * V * V;
#pragma unroll
        for (int mt = 0; mt < KS; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float2* lo = reinterpret_cast<float2*>(out + (16 * mt + g) * V + 8 * nt + 2 * qd);
                float2* hi = reinterpret_cast<float2*>(out + (16 * mt + g + 8) * V + 8 * nt + 2 * qd);
                float2 a0 = *lo, a1 = *hi;
                a0.x += dWacc[mt][nt][0], a0.y += dWacc[mt][nt][1], a1.x += dWacc[mt][nt][2], a1.y += dWacc[mt][nt][3];
                *lo = a0, *hi = a1;
            }
    }
}

template <int V>
int launch(const LmeM2rnnArgs& p, int mode, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(p.B) * p.N * (p.K / 16);
    if (mode == 0) {
        m2rnn_fwd_kernel<V, false><<<grid, 32, 0, stream>>>(p);
    } else if (mode == 1) {
        m2rnn_fwd_kernel<V, true><<<grid, 32, 0, stream>>>(p);
    } else {
        const int bytes = static_cast<int>(sizeof(BwdSmem<V>));
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(m2rnn_bwd_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
                return -4;
            configured = true;
        }
        m2rnn_bwd_kernel<V><<<grid, 32, bytes, stream>>>(p);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace m2
}  // namespace lme

extern "C" int lme_m2rnn(const LmeM2rnnArgs* args, int mode, void* stream) {
    const LmeM2rnnArgs& p = *args;
    if (mode < 0 || mode > 2 || p.B <= 0 || p.S <= 0 || p.N <= 0 || p.K % 16 || p.K <= 0) return -1;
    if (p.N % p.Nq || p.N % p.Nk || p.N % p.Nv || p.N % p.Nf || p.N % p.Nw) return -1;
    if (static_cast<long long>(p.B) * p.N * (p.K / 16) > 2147483647ll) return -6;
    auto mis = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) != 0; };
    if (mis(p.q) || mis(p.k) || mis(p.v) || mis(p.W) || (p.q_b | p.q_t | p.k_b | p.k_t | p.v_b | p.v_t) % 8) return -2;
    if (mode >= 1 && (mis(p.hprev) || mis(p.z) || p.T <= 0 || p.T > p.Tcap || p.t0 % p.seg_len)) return -2;
    if (mode == 2 && mis(p.dy)) return -2;
    if (mode == 0 && p.ckpt && p.seg_len <= 0) return -1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (p.V) {
        case 16: return lme::m2::launch<16>(p, mode, st);
        case 32: return lme::m2::launch<32>(p, mode, st);
        case 64: return lme::m2::launch<64>(p, mode, st);
        default: return -1;
    }
}
