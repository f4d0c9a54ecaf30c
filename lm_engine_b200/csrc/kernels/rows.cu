// Row movers: embedding lookup and its gradient, and packing / unpacking of left-padded batches.
//
//   embedding_fwd : out[t, :] = (lo <= ids[t] < hi) ? W[ids[t] - lo, :] : 0        (vocab-parallel masked lookup)
//   embedding_bwd : dW[v, :] = sum over the tokens with id v of dy[t, :]; the caller passes the token order sorted by
//                   id, one block per run of equal ids adds the run in fp32 and writes the row once - no atomics, the
//                   result does not depend on scheduling
//   pack_rows     : packed[cu[b] + j, :] = x[b, S - len_b + j, :]                   (len_b = cu[b+1] - cu[b])
//   unpack_rows   : x[b, s, :] = s >= S - len_b ? packed[cu[b] + s - (S - len_b), :] : 0
// Rows are moved as 16-byte vectors (row_bytes % 16 == 0, bases 16-byte aligned).
// Role of DTensor F.embedding (lm_engine/modeling_utils/embedding.py:37-92) and of xma pack_sequence /
// unpack_sequence (lm_engine/modeling_utils/sequence_packing.py:32-33,65-68) in the reference.
namespace lme {
namespace rows {

__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const uint4* __restrict__ W, uint4* __restrict__ out,
                     long long T, int vec_per_row, long long lo, long long hi) {
    const long long total = T * vec_per_row;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
        const long long t = i / vec_per_row;
        const int v = static_cast<int>(i % vec_per_row);
        const long long id = ids[t];
        out[i] = (id >= lo && id < hi) ? W[(id - lo) * vec_per_row + v] : make_uint4(0u, 0u, 0u, 0u);
    }
}

// sorted_ids[j] ascending, order[j] = the token that holds it.  Block j works only when it starts a run.
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ sorted_ids, const long long* __restrict__ order,
                     const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dW, long long T, int H,
                     long long lo, long long hi) {
    const long long j0 = blockIdx.x;
    const long long id = sorted_ids[j0];
    if (id < lo || id >= hi || (j0 > 0 && sorted_ids[j0 - 1] == id)) return;
    long long j1 = j0 + 1;
    while (j1 < T && sorted_ids[j1] == id) ++j1;
    for (int c = threadIdx.x * 8; c < H; c += 256 * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (long long j = j0; j < j1; ++j) {
            float v[8];
            load8(dy + order[j] * H + c, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] += v[e];
        }
        store8(dW + (id - lo) * H + c, acc);
    }
}

__device__ __forceinline__ int find_row(const int* __restrict__ cu, int B, long long t) {
    int lo = 0, hi = B;                        // largest b with cu[b] <= t
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cu[mid] <= t) lo = mid;
        else hi = mid;
    }
    return lo;
}

__global__ void __launch_bounds__(256)
pack_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ cu, uint4* __restrict__ out, int B, int S,
                 long long T, int vec_per_row) {
    const long long total = T * vec_per_row;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
        const long long t = i / vec_per_row;
        const int v = static_cast<int>(i % vec_per_row);
        const int b = find_row(cu, B, t);
        const int len = cu[b + 1] - cu[b];
        const long long s = S - len + (t - cu[b]);
        out[i] = x[(static_cast<long long>(b) * S + s) * vec_per_row + v];
    }
}

__global__ void __launch_bounds__(256)
unpack_rows_kernel(const uint4* __restrict__ packed, const int* __restrict__ cu, uint4* __restrict__ x, int B, int S,
                   int vec_per_row) {
    const long long total = static_cast<long long>(B) * S * vec_per_row;
    for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
        const int v = static_cast<int>(i % vec_per_row);
        const long long bs = i / vec_per_row;
        const int b = static_cast<int>(bs / S), s = static_cast<int>(bs % S);
        const int len = cu[b + 1] - cu[b];
        x[i] = s >= S - len ? packed[(static_cast<long long>(cu[b]) + s - (S - len)) * vec_per_row + v]
                            : make_uint4(0u, 0u, 0u, 0u);
    }
}

inline unsigned grid_for(long long total) {
    const long long blocks = (total + 255) / 256;
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks > 148 * 16 ? 148 * 16 : blocks));
}

}  // namespace rows
}  // namespace lme

extern "C" int lme_embedding_fwd(const long long* ids, const void* W, void* out, long long T, int H, long long lo,
                                 long long hi, void* stream) {
    if (T <= 0 || H <= 0 || H % 8) return -1;
    if ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
    lme::rows::embedding_fwd_kernel<<<lme::rows::grid_for(T * (H / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        ids, static_cast<const uint4*>(W), static_cast<uint4*>(out), T, H / 8, lo, hi);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int lme_embedding_bwd(const long long* sorted_ids, const long long* order, const void* dy, void* dW,
                                 long long T, int H, long long lo, long long hi, void* stream) {
    if (T <= 0 || H <= 0 || H % 8 || T > 2147483647ll) return -1;
    if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dW)) & 15) return -2;
    lme::rows::embedding_bwd_kernel<<<static_cast<unsigned>(T), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sorted_ids, order, static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dW), T, H, lo, hi);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int lme_pack_rows(const void* x, const int* cu_seqlens, void* out, int B, int S, long long T,
                             long long row_bytes, void* stream) {
    if (B <= 0 || S <= 0 || T <= 0 || row_bytes <= 0 || row_bytes % 16) return -1;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
    const int vec = static_cast<int>(row_bytes / 16);
    lme::rows::pack_rows_kernel<<<lme::rows::grid_for(T * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x), cu_seqlens, static_cast<uint4*>(out), B, S, T, vec);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int lme_unpack_rows(const void* packed, const int* cu_seqlens, void* x, int B, int S, long long row_bytes,
                               void* stream) {
    if (B <= 0 || S <= 0 || row_bytes <= 0 || row_bytes % 16) return -1;
    if ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(x)) & 15) return -2;
    const int vec = static_cast<int>(row_bytes / 16);
    lme::rows::unpack_rows_kernel<<<lme::rows::grid_for(static_cast<long long>(B) * S * vec), 256, 0,
                                    static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(packed), cu_seqlens, static_cast<uint4*>(x), B, S, vec);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
