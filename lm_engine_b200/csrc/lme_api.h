// C ABI of liblme_cuda.so.  Every entry point takes raw device pointers and a cudaStream_t (as void*), returns
// LME_OK or a negative error code, never allocates device memory unless stated, and never synchronises.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define LME_OK 0
#define LME_ERR_SHAPE (-1)
#define LME_ERR_ALIGN (-2)
#define LME_ERR_TMAP (-3)
#define LME_ERR_LAUNCH (-4)
#define LME_ERR_DRIVER (-5)
#define LME_ERR_TOO_LARGE (-6)

// lme_gemm_bf16 flags
#define LME_GEMM_OUT_F32 1
#define LME_GEMM_ACCUMULATE 2
#define LME_GEMM_SWIGLU 4
// timing probes for the micro-benchmarks (results are meaningless): the TMA producer declares every stage full
// without loading it / the MMA issuer releases every stage without multiplying it
#define LME_GEMM_PROBE_NO_LOAD 64
#define LME_GEMM_PROBE_NO_MMA 128

// C[M,N] (+)= A x B^T (+ bias) (+ residual); operands K-major ([rows, K]) or MN-major ([K, rows]).
// ld* are row pitches in elements.  With LME_GEMM_SWIGLU, C is [M, N/2] and `preact` (optional) gets [M, N].
int lme_gemm_bf16(const void* A, int a_mn_major, long long lda, const void* B, int b_mn_major, long long ldb,
                  void* C, long long ldc, int M, int N, int K, int flags, const void* bias, const void* residual,
                  long long ldr, void* preact, long long ldp, int max_ctas, void* stream);


// Batched form: C[b] (+)= A[b] x B[b]^T for b < batch; operand / output b starts *_batch_ld elements after b - 1.
// Flags: LME_GEMM_OUT_F32, LME_GEMM_ACCUMULATE.  Rows past M / N of a batch read as zeros (3-D tensor maps).
int lme_gemm_bf16_batched(const void* A, int a_mn_major, long long lda, long long a_batch_ld, const void* B,
                          int b_mn_major, long long ldb, long long b_batch_ld, void* C, long long ldc,
                          long long c_batch_ld, int batch, int M, int N, int K, int flags, int max_ctas, void* stream);

// Grouped GEMM (mixture of experts).  A / C rows are in a padded per-group layout in which every 128-row tile belongs
// to one group: tile_group[m-tile] = group (< 0: unused tile).  B holds all groups: K-major [G * N, K] (forward,
// C = A B_e^T) or MN-major [G * K, N] (input gradient, C = A B_e).  Flags / SwiGLU epilogue as lme_gemm_bf16.
int lme_gemm_bf16_grouped(const void* A, long long lda, const void* B, int b_mn_major, long long ldb, void* C,
                          long long ldc, int M, int N, int K, int num_groups, int flags, void* preact, long long ldp,
                          const int* tile_group, int max_ctas, void* stream);

// dW[e] [M, N] (+)= dY[rows of e]^T X[rows of e]; group e owns rows [group_k0[e], group_k0[e] + 64 * group_kb[e]).
int lme_gemm_bf16_grouped_wgrad(const void* dY, long long lddy, const void* X, long long ldx, void* dW, long long ldw,
                                int M, int N, int rows, int num_groups, const int* group_k0, const int* group_kb,
                                int flags, int max_ctas, void* stream);

// C[M, N] = (A[M, K] * B[N, K]^T) * scale_a[0] * scale_b[0]: 1-byte e4m3 (fmt 0) / e5m2 (fmt 1) operands, both
// K-major, fp32 accumulation in TMEM; same flags and fused epilogue as lme_gemm_bf16.  K, lda, ldb % 16 == 0.
int lme_gemm_fp8(const void* A, int a_fmt, long long lda, const void* B, int b_fmt, long long ldb,
                 const float* scale_a, const float* scale_b, void* C, long long ldc, int M, int N, int K, int flags,
                 const void* bias, const void* residual, long long ldr, void* preact, long long ldp, int max_ctas,
                 void* stream);

// All-gather fused into the GEMM: C = A_gathered * B^T where A_gathered [M, K] (local, written by this call) is the
// concatenation in rank order of `world` contributions of shard_bytes each.  Copy CTAs of the GEMM's own grid move
// this rank's contribution (local_src) and the peers' (through the symmetric staging buffers stage[r]) with bulk
// asynchronous copies over NVLink while the other CTAs multiply the rows that have arrived.  pads[r]: 16-word int32
// signal pad of rank r in symmetric memory; ready / counters: local scratch words (see kernels/gather.cuh);
// seq = 1, 2, ... per call on one set of buffers, the same on every rank.  All waits are bounded.
int lme_gemm_bf16_allgather_a(void* A_gathered, long long lda, const void* B, int b_mn_major, long long ldb, void* C,
                              long long ldc,
                              int M, int N, int K, int flags, const void* bias, const void* residual, long long ldr,
                              void* preact, long long ldp, const void* local_src, void* const* stage,
                              int* const* pads, int* ready, unsigned int* counters, long long shard_bytes, int rank,
                              int world, int seq, int n_copy, int seg_shift, int max_ctas, void* stream);

// With n_copy == 0 the peers' rows are delivered by copy engines instead (device-to-device copies on a side stream,
// each followed by lme_stream_write_words on the `ready` word of that chunk of 1 << seg_shift bytes); the GEMM only
// waits for the words.  lme_gather_signal announces this rank's staging slot; lme_gather_wait_peer holds a stream
// (bounded) until a peer's announcement for `seq` is in this rank's pad.
int lme_gather_signal(int* const* pads, int rank, int world, int seq, void* stream);
int lme_gather_wait_peer(const int* pad, int src, int seq, void* stream);
int lme_stream_write_words(int* words, int count, int value, void* stream);
// holds the stream until *word >= value (stream memory operation, takes no SM; not bounded by itself)
int lme_stream_wait_word(const int* word, int value, void* stream);

// Reduce-scatter fused into the GEMM epilogue: out[M / world, N] = sum over ranks of (A * B^T)[rows of this rank]
// (+ bias) (+ residual).  Tiles of a peer's rows are stored into that peer's receive slab over NVLink with an
// arrival flag; own rows are multiplied last and their epilogue adds what the peers delivered.  slabs[r] / flags[r]:
// slab (slot of this call) and flag words of rank r in symmetric memory; M / world % 128 == 0; seq = 1, 2, ...
int lme_gemm_bf16_reduce_scatter(const void* A, long long lda, const void* B, int b_mn_major, long long ldb, void* out,
                                 long long ldo,
                                 int M, int N, int K, const void* bias, const void* residual, long long ldr,
                                 void* const* slabs, int* const* flags, int rank, int world, int seq, int max_ctas,
                                 void* stream);

// Mixture-of-experts token movement on bf16 rows of H elements (H % 8 == 0); slot[t * K + k] = row of the padded
// per-expert layout holding the k-th assignment of token t (< 0: none); w (optional) = bf16 [T, K] weights.
//   scatter_rows : dst[slot[t,k]] = w[t,k] * src[t]      gather_reduce : dst[t] = sum_k w[t,k] * src[slot[t,k]]
//   row_dots     : out[t,k] = <a[slot[t,k]], b[t]>
int lme_moe_scatter_rows(const void* src, const int* slot, const void* w, void* dst, int T, int H, int K, void* stream);
int lme_moe_gather_reduce(const void* src, const int* slot, const void* w, void* dst, int T, int H, int K,
                          void* stream);
int lme_moe_row_dots(const void* a, const int* slot, const void* b, void* out, int T, int H, int K, void* stream);

// Router: top-k selection fused with the softmax on bf16 logits [T, E] (E <= 512, K <= 32), one warp per token.
// normalized != 0: weights = softmax over the K selected logits; else softmax over all experts read at the selected
// ones (lse [T] fp32 receives the row log-sum-exp the backward call needs).  selected is int64 [T, K], descending,
// the lower index first among equal logits.  The backward call writes every element of dlogits [T, E].
int lme_moe_topk_softmax_fwd(const void* logits, int T, int E, int K, int normalized, void* weights,
                             long long* selected, float* lse, void* stream);
int lme_moe_topk_softmax_bwd(const void* logits, const long long* selected, const void* dw, const float* lse, int T,
                             int E, int K, int normalized, void* dlogits, void* stream);

// Expert-parallel token exchange over peer memory (kernels/ep_exchange.cu has the protocol).  Pointer arrays have one
// entry per rank of the expert-parallel group ([rank] = this rank's own memory): counts[r] = rank r's [world][E] int32
// table, pads[r] = rank r's flag block of this direction (lme_ep_flag_words() int32 words, zero at start), tables[r] =
// rank r's row table (int32 [cap][2], zero at start), stages[r] = its staged rows, slabs[r] = its output slab.  `seq` is the round number (grows by
// one per round of a direction, the same on every rank).  dest is int32 [A][2] = (owner, row or -1).
int lme_ep_flag_words(void);
int lme_ep_publish_counts(const long long* freq, void* const* counts, void* const* pads, int rank, int world, int E,
                          int seq, void* stream);
int lme_ep_bases(const int* counts, const int* pad, int rank, int world, int E, int seq, int cap, int* base,
                 int* k0_own, int* kb_own, int* rows_own, int* tile_group, void* stream);
int lme_ep_dest(const long long* sel, const int* slot, const int* k0_local, const int* base, int A, int E, int world,
                int cap, void* dest, void* stream);
int lme_ep_offer_rows(const void* dest, void* const* tables, void* const* pads, int A, unsigned int* counter,
                      int rank, int world, int seq, void* stream);
int lme_ep_land_rows(void* const* stages, const void* table, const int* tile_group, void* out, int cap, int H, int rep,
                     int seq, int world, void* stream);
int lme_ep_wait(const int* pad, int which, int world, int seq, void* stream);   // which: 0 rows arrived, 1 output ready
int lme_ep_signal_done(void* const* pads, int rank, int world, int seq, void* stream);
int lme_ep_pull_rows(void* const* slabs, const void* dest, void* out, int T, int K, int H, int reduce, int world,
                     void* stream);

// Padded per-expert row layout from the unsorted selection (total = T * K entries, E <= 1024): freq[e] = count,
// k0[e] = first row (multiple of 128), kb[e] = padded rows / 64, tile_group[tile] = expert of a 128-row tile or -1,
// slot[i] = row of assignment i (assignments of an expert keep their index order; < 0 for an id outside [0, E)).
// ntiles * 128 >= total + 127 * E.  scratch holds lme_moe_route_chunks(total) * E ints.
int lme_moe_route_chunks(int total);
int lme_moe_route_layout(const long long* selected, int total, int E, int* scratch, long long* freq, int* k0, int* kb,
                         int* tile_group, int ntiles, int* slot, void* stream);

// Inter-chunk chain of the gated delta rule (kernels/delta_rule.cu has the recurrences).  BN = batch * heads, nc chunks
// of 64 rows, K in {128, 256}, V % 64 == 0.  Forward operands (bf16): wk = W_k [BN][nc][64][K], qe [BN][nc][64][K],
// ket = K_e^T [BN][nc][K][64], qk [BN][nc][64][64]; fp32: wv [BN][nc][64][V], a [BN][nc], h0 [BN][K][V] or null.
// Outputs: y fp32 [BN][nc][64][V], u_all bf16 [BN][nc][64][V], h_all bf16 [BN][nc][K][V] (state entering each chunk),
// h_final fp32 [BN][K][V].  Backward operands (bf16): qkt = QK^T, ke [BN][nc][64][K], qet = Q_e^T [BN][nc][K][64],
// wkt = W_k^T [BN][nc][K][64] (wk / wkt may be null: no correction term, the chain of linear attention); dy fp32; outputs du_all bf16, dh_all bf16 (gradient leaving each chunk), dh0 fp32.
int lme_delta_chain_fwd(const void* wk, const void* qe, const void* ket, const void* qk, const float* wv,
                        const float* a, const float* h0, float* y, void* u_all, void* h_all, float* h_final, int BN,
                        int nc, int K, int V, void* stream);
int lme_delta_chain_bwd(const void* qkt, const void* ke, const void* qet, const void* wkt, const float* dy,
                        const float* a, const float* dh_final, void* du_all, void* dh_all, float* dh0, int BN, int nc,
                        int K, int V, void* stream);

// Depthwise causal convolution on channel-last bf16 activations x [B, S, C], weight [C, K] (K <= 8), optional bias [C]
// and initial state init [B, C, K-1] (the inputs before t = 0); silu != 0 fuses the activation.  Backward recomputes
// the pre-activation; dw [C, K] / dbias [C] are fp32 accumulators the caller zeroes, dinit [B, C, K-1] is written.
int lme_causal_conv1d_fwd(const void* x, const void* w, const void* bias, const void* init, void* y, int B, int S,
                          int C, int K, int silu, void* stream);
int lme_causal_conv1d_bwd(const void* x, const void* w, const void* bias, const void* init, const void* dy, void* dx,
                          float* dw, float* dbias, float* dinit, int B, int S, int C, int K, int silu, void* stream);

// out (=|+=) scale * sum of nsrc <= 8 local slices of n elements (bf16 or fp32, fp32 accumulation): the reduction
// half of a reduce-scatter whose peer slices were pulled by copy engines.
int lme_reduce_slices(const void* const* src, int nsrc, void* out, long long n, int is_bf16, float scale,
                      int accumulate, void* stream);

// Gradient reduce-scatter in one kernel: out[n] (=|+=) scale * sum over ranks of this rank's slice of every rank's
// buffer (symmetric memory; src[r] = the slice inside rank r's buffer as mapped here, [rank] local), fp32 sums in
// rank order, plus one partial sum of squares of the written values per CTA (partials[ctas], may be null).
// mc_src != null: the slice's multicast mapping, read with multimem.ld_reduce (the switch adds) instead of
// `world` peer loads.  pads[r]: 16-word int32 signal pad of rank r; seq = 1, 2, ... per call, the same on every
// rank.  The kernel announces this rank's buffer, waits (bounded) for every peer's announcement, then reads.
int lme_reduce_scatter_peers(const void* const* src, int* const* pads, const void* mc_src, int rank, int world,
                             int seq, void* out, long long n, int is_bf16, float scale, int accumulate,
                             float* partials, int ctas, void* stream);
// out[0] (+)= sum of n floats in a fixed order
int lme_sum_partials(const float* partials, int n, float* out, int accumulate, void* stream);
// limit of the device-side waits on words written by another GPU (default 2000 ms)
int lme_set_peer_wait_limit_ms(long long ms);

// Mamba-2 SSD intra-chunk helpers (L % 8 == 0, L <= 1024; BC = batch x chunks):
//   decay_matrix: m[BC,N,L,L] = cb[BC,G,L,L] * exp(cum[BC,N,l] - cum[BC,N,s]) for s <= l else 0 (bf16; cum fp32)
//   dcb         : dcb[BC,G,L,L] = sum over the heads of a group of dm[BC,N,L,L] * exp(cum[l] - cum[s]), s <= l
int lme_ssd_decay_matrix(const void* cb, const float* cum, void* m, long long BC, int N, int G, int L, void* stream);
int lme_ssd_dcb(const void* dm, const float* cum, void* dcb, long long BC, int N, int G, int L, void* stream);

// Matrix-state RNN scan (kernels/m2rnn.cu).  q/k [B,S,Nq|Nk,K] and v [B,S,Nv,V] are bf16 with element strides
// *_b (batch) and *_t (token), the K (V) values of a head contiguous; f fp32 [B,S,Nf]; W bf16 [Nw,V,V]; every head
// count divides N and operand heads are shared by consecutive groups of N / count heads.  K % 16 == 0, V in
// {16, 32, 64}, all bases and strides 16-byte aligned.  RB = K / 16.
//   mode 0 forward : y_part fp32 [RB,B,S,N,V] (sum over RB = y), h_out fp32 [B,N,K,V], optional h0 (same shape),
//                    optional ckpt fp32 [B,N,ceil(S/seg_len),K,V] = state before each segment
//   mode 1 replay  : steps t0 .. t0+T-1 from ckpt[t0 / seg_len]; writes hprev, z bf16 [B,N,Tcap,K,V]
//   mode 2 backward: steps t0+T-1 .. t0; reads hprev, z (overwritten with da), dy bf16 [B,S,N,V], dh fp32 [B,N,K,V]
//                    (in: gradient of the state after step t0+T-1, out: before step t0); writes dq, dk fp32
//                    [B,S,N,K], dv_part fp32 [RB,B,S,N,V], df_part fp32 [RB,B,S,N]; clip > 0 clamps dh every step.
//                    V = 64: z is overwritten with da for the caller's dW GEMM; V <= 32: dW_part is accumulated
typedef struct LmeM2rnnArgs {
    const void *q, *k, *v;
    const float* f;
    const void* W;
    long long q_b, q_t, k_b, k_t, v_b, v_t;
    int B, S, N, K, V, Nq, Nk, Nv, Nf, Nw;
    const float* h0;
    float* h_out;
    float* y_part;
    float* ckpt;
    int seg_len, t0, T, Tcap;
    void *hprev, *z;
    const void* dy;
    float *dh, *dq, *dk, *dv_part, *df_part;
    float clip;
    float* dW_part;   // V <= 32: fp32 [B,N,RB,V,V], += sum_t h_{t-1}^T da_t of each launch (hprev / z stay inputs only)
} LmeM2rnnArgs;
int lme_m2rnn(const LmeM2rnnArgs* args, int mode, void* stream);

// Vector-state RNN / GRU scans (kernels/rnn.cu), state h [B,N,H] per (batch, head), H in {16, 32} (RNN also 64):
//   RNN: h_t = tanh(h_{t-1} W + x_t)
//   GRU: f = sigmoid(h_{t-1} Wf + xf_t), r = sigmoid(h_{t-1} Wr + xr_t), z = tanh((h_{t-1} * r) W + x_t),
//        h_t = f h_{t-1} + (1 - f) z
// x* bf16 [B,S,Nx*,H] with element strides *_b / *_t (16-byte aligned), W* bf16 [Nw*,H,H], h0 bf16 [B,N,H] (never
// null: zeros for a fresh state), y bf16 [B,S,N,H] (= every state, so the last step is the final state).
//   mode 0 forward ; mode 1 backward: reads y, dy bf16 [B,S,N,H] and dh fp32 [B,N,H] (in: gradient of the final
//   state, out: of h0); writes dx (, dxf, dxr, hr = h_{t-1} * r) bf16 [B,S,N,H]; the weight gradients are
//   sum_t h_{t-1}^T dx_t etc., left to batched GEMMs.  clip > 0 clamps the state gradient at every step.
typedef struct LmeRnnArgs {
    const void *x, *xf, *xr;
    const void *W, *Wf, *Wr;
    long long x_b, x_t, xf_b, xf_t, xr_b, xr_t;
    int B, S, N, H, Nx, Nxf, Nxr, Nw, Nwf, Nwr, gru, pad_;
    const void* h0;
    void* y;
    const void* dy;
    float* dh;
    void *dx, *dxf, *dxr, *hr;
    float clip;
} LmeRnnArgs;
int lme_rnn(const LmeRnnArgs* args, int mode, void* stream);

// Row movers (kernels/rows.cu); H % 8 == 0 / row_bytes % 16 == 0, 16-byte aligned bases.
//   embedding_fwd: out[t,:] = lo <= ids[t] < hi ? W[ids[t]-lo,:] : 0 (bf16 rows of H values)
//   embedding_bwd: dW[v-lo,:] = sum of dy[t,:] over tokens with id v; sorted_ids ascending with order[j] the token of
//                  sorted position j; dW must be zero on entry (rows without tokens are not touched)
//   pack_rows / unpack_rows: left-padded [B,S,row] <-> packed [T,row] by cu_seqlens (int32 [B+1]); unpack zero-fills
int lme_embedding_fwd(const long long* ids, const void* W, void* out, long long T, int H, long long lo, long long hi,
                      void* stream);
int lme_embedding_bwd(const long long* sorted_ids, const long long* order, const void* dy, void* dW, long long T,
                      int H, long long lo, long long hi, void* stream);
int lme_pack_rows(const void* x, const int* cu_seqlens, void* out, int B, int S, long long T, long long row_bytes,
                  void* stream);
int lme_unpack_rows(const void* packed, const int* cu_seqlens, void* x, int B, int S, long long row_bytes,
                    void* stream);

// Flash-attention forward (kernels/attention.cu): head dim 128, bf16, S_q and S_kv multiples of 128, Hq % Hkv == 0.
// q [B,S_q,Hq,128], k / v [B,S_kv,Hkv,128] with token pitch ld* elements (heads contiguous inside a token, batches
// back to back); o [B,S_q,Hq,128] with token pitch ldo; lse fp32 [B,Hq,S_q] or null.  causal aligns the last query
// with the last key; window > 0 (causal only) is a sliding window: query i sees its last `window` visible keys.
// scale multiplies q.k before the softmax.  Packed sequences: cu_seqlens (int32 [B+1], device) with q / k / v / o
// as [total_tokens, H, 128], S_q = S_kv = the longest sequence (any lengths), lse [B,Hq,S_pad], S_pad = S_q rounded
// up to 128; cu_seqlens null = batches.
// kv_ready != null (batches only): chunks of kv_chunk_rows key / value rows (a multiple of 64) become valid while the
// kernel runs - word [b * chunks + c] of kv_ready holds kv_seq once chunk c of batch entry b is complete (written by
// the stream that copied it in); the kernel's loader waits, bounded, for the word of a tile's chunk.
int lme_attention_fwd(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                      void* o, long long ldo, float* lse, int B, int S_q, int S_kv, int Hq, int Hkv, int causal,
                      int window, float scale, const int* cu_seqlens, long long total_tokens, const int* kv_ready,
                      int kv_chunk_rows, int kv_seq, void* stream);

// Gradients of lme_attention_fwd (kernels/attention_bwd.cu; two kernels, no atomics, deterministic).  dout and out
// laid out like q; lse fp32 [B,Hq,S_q]; delta fp32 scratch of that shape (receives rowsum(dout * out));
// dq [B,S_q,Hq,128], dk / dv [B,S_kv,Hkv,128] bf16 with token pitches ldd*, written whole.  S_q and S_kv multiples
// of 128.
int lme_attention_bwd(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                      const void* dout, long long lddo, const void* out, long long ldo, const float* lse,
                      float* delta, void* dq,
                      long long lddq, void* dk, long long lddk, void* dv, long long lddv, int B, int S_q, int S_kv,
                      int Hq, int Hkv, int causal, int window, float scale, const int* cu_seqlens,
                      long long total_tokens, void* stream);

// Element-wise glue of the chunked SSD scan (kernels/ssd.cu), BC = batch x chunks, L % 32 == 0, P in {32, 64, 128}:
//   prep    (mode 0) xh[BC,N,L,P] = x[BC,L,N,P] dt[BC,L,N];  xwT[BC,N,P,L] = x dt tail, transposed          (bf16)
//           (mode 1) dx, ddt, dtail from dxh (fp32 [BC,N,L,P]) and dxwT (bf16 [BC,N,P,L])
//   combine (mode 0) y[BC,L,N,P] = yin[BC,N,L,P] + off[BC,G,L,(N/G)P] ecum[BC,L,N] + D[n] x                 (bf16 out)
//           (mode 1) dyin, doff (bf16), decum, dDp[BC,L,N] (fp32 row sums of dy x), dx = D dy
int lme_ssd_prep(const void* x, const float* dt, const float* tail, void* xh, void* xwT, const float* dxh,
                 const void* dxwT, void* dx, float* ddt, float* dtail, long long BC, int N, int L, int P, int mode,
                 void* stream);
int lme_ssd_combine(const float* yin, const float* off, const float* ecum, const float* D, const void* x, void* y,
                    const void* dy, void* dyin, void* doff, float* decum, float* dDp, void* dx, long long BC, int N,
                    int L, int G, int P, int mode, void* stream);
// Chunk-boundary recurrence h_{c+1} = decay[c] h_c + states[c] per (batch, head), E = P * Sd elements (E % 4 == 0):
// forward writes the state at every chunk start (bf16, and fp32 when h0_f32 != null) and the final state; backward
// (E <= 16384) returns dstates, ddecay and (optionally) dh_init from dh0 / dh_final (either may be null).
int lme_ssd_boundary_fwd(const float* states, const float* decay, const float* h_init, void* h0_bf16, float* h0_f32,
                         float* h_final, int B, int NC, int N, int E, void* stream);
int lme_ssd_boundary_bwd(const float* dh0, const float* dh_final, const float* h0_f32, const float* decay,
                         float* dstates, float* ddecay, float* dh_init, int B, int NC, int N, int E, void* stream);


// max |x| of n bf16 values, max-combined into *amax (which must hold 0 or an earlier running maximum).
int lme_fp8_amax(const void* x, long long n, float* amax, void* stream);

// Tensor-wise scaled cast of a bf16 [rows, cols] matrix to 8 bits with scale fmax / amax[0]; writes q [rows, cols]
// and / or its transpose qt [cols, rows] (either may be null) and scale_inv[0] = amax / fmax.
int lme_fp8_quantize(const void* x, int rows, int cols, long long ldx, const float* amax, int fmt, void* q,
                     long long ldq, void* qt, long long ldqt, float* scale_inv, void* stream);

// Copies the 8-word device status block to the host (synchronising copy); optionally clears it.
int lme_read_status(unsigned int* out8, int clear);

// ---- bandwidth-bound block kernels (bf16 activations, fp32 math) ----
// y = rmsnorm(x (+ residual)) * w; h_out (optional) receives x + residual; rstd (optional) the per-row 1/rms.
int lme_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out, float* rstd, int T,
                    int H, float eps, void* stream);
// rows of the weight-gradient scratch that lme_rmsnorm_bwd writes for T rows: min(max(T, 1), 444), one per CTA of
// a single wave (148 SMs x 3 resident CTAs)
#define LME_RMSNORM_BWD_MAX_PARTIAL_ROWS 444
int lme_rmsnorm_bwd_partial_rows(int T);
// dx = d rmsnorm / d h  (+ dres); dw (fp32, optional accumulate) via the fp32 scratch dw_partial
// [lme_rmsnorm_bwd_partial_rows(T), H].
int lme_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres, void* dx,
                    float* dw_partial, float* dw, int dw_accumulate, int T, int H, void* stream);
// x [T, 2I] with (gate, up) interleaved -> y [T, I] = up * silu(gate)
int lme_swiglu_fwd(const void* x, void* y, long long T, long long I, void* stream);
int lme_swiglu_bwd(const void* x, const void* dy, void* dx, long long T, long long I, void* stream);
// the same on 128-row tiles of which only those with tile_group[tile] >= 0 are read and written (T % 128 == 0)
int lme_swiglu_bwd_tiles(const void* x, const void* dy, void* dx, long long T, long long I, const int* tile_group,
                         void* stream);
// fused QKV split + NeoX rotary embedding (inverse = 1: backward, packs dq/dk/dv into dqkv).  cos_t / sin_t are
// [max_pos, rope_dim]; pos (optional) has T entries, else position = t % S.  A position outside the table sets the
// status word (STATUS_BOUNDS) instead of reading out of bounds.
int lme_qkv_rope(void* qkv, void* q, void* k, void* v, const float* cos_t, const float* sin_t, const int* pos,
                 int T, int S, int Hkv, int G, int D, int rope_dim, int max_pos, int inverse, void* stream);
// cross entropy over a vocabulary slice [v0, v0+V): row statistics, then in-place gradient
int lme_ce_stats(const void* logits, long long ld, const long long* labels, float* row_max, float* row_sum,
                 float* tgt_logit, int T, int V, int v0, void* stream);
// gradient scale = scale * (*scale_dev if scale_dev != NULL)
int lme_ce_grad(void* logits, long long ld, const long long* labels, const float* lse, int T, int V, int v0,
                float scale, const float* scale_dev, long long ignore_index, void* stream);
// torch.optim.AdamW step on a flat fp32 shard (+ refresh of the bf16 compute copy); step counts from 1
int lme_adamw(float* p, float* m, float* v, const void* g, int g_is_bf16, void* p_lp, long long n, float lr,
              float b1, float b2, float eps, float wd, int step, const float* gscale, void* stream);
#define LME_SUMSQ_MAX_PARTIALS 1184
int lme_sumsq(const void* x, int is_bf16, long long n, float* partials, float* out, int accumulate, void* stream);
int lme_clip_coef(const float* sumsq, float max_norm, float* norm_out, float* coef_out, void* stream);

#ifdef __cplusplus
}
#endif
