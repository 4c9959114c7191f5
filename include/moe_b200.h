/*
 * moe_b200 -- C ABI of the B200 (sm_100a) MoE-layer hot path.
 *
 * The reference project exposes this path as Python functions only (package
 * `kernels`); it has no FFI of its own.  Each entry point below names the
 * reference function (file:line inside the reference project) whose device work
 * it replaces.  A Python binding calls these through ctypes on the caller's
 * thread (tilelang_moe_b200/_lib.py is such a binding).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer, borrowed for the duration of the call,
 *     unless the parameter comment says "host";
 *   - the library never allocates or frees memory on behalf of these calls:
 *     scratch is passed in as (ws, ws_bytes), sized by the matching *_workspace
 *     query;
 *   - every call only enqueues work on `stream` (a cudaStream_t passed as void*)
 *     and returns without synchronising;
 *   - return value: 0 ok; negative = argument / shape error found on the host
 *     before any launch; positive = CUDA runtime error code.  A message for the
 *     last non-zero return on the calling thread is at moe_last_error();
 *   - kernels that wait on barriers do so with a time limit; if a limit is hit
 *     the kernel stores a non-zero code in the caller's `status` word (device
 *     int32[MOE_STATUS_WORDS], may be NULL) and returns normally.
 */
#ifndef MOE_B200_H_
#define MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_OK 0
#define MOE_ERR_ARG (-1)          /* bad pointer / size / alignment            */
#define MOE_ERR_UNSUPPORTED (-2)  /* shape outside what the kernels cover      */
#define MOE_ERR_WORKSPACE (-3)    /* ws_bytes smaller than the query's answer  */
#define MOE_ERR_DEVICE (-4)       /* not an sm_100 device                      */

#define MOE_STATUS_WORDS 4        /* int32 words in a status buffer            */

/* softmax / selection convention of the router */
#define MOE_TOPK_MODE_B 0         /* top-k of logits, softmax over the k        */
#define MOE_TOPK_MODE_A 1         /* softmax over N, pick k, no renormalisation */
#define MOE_TOPK_MODE_A_RENORM 2  /* as A, then scores / sum(scores)            */

/* epilogue of the expert GEMM */
#define MOE_GEMM_PLAIN 0          /* Y[dst(r)] = A[r] . B[e]^T              (bf16) */
#define MOE_GEMM_SILU_GATE 1      /* Y[r] = silu(A[r].Bg[e]^T) * (A[r].Bu[e]^T)    */
#define MOE_GEMM_SCALE_SCATTER 2  /* Y[dst(r)] = w[r] * (A[r] . B[e]^T)            */
#define MOE_GEMM_PLAIN_F32 3      /* as PLAIN, fp32 output                         */
#define MOE_GEMM_SCALE_SCATTER_DSTW 4 /* Y[dst(r)] = w[dst(r)] * (A[r] . B[e]^T): the weight is
                                         read at the destination row, e.g. straight from the
                                         [T,k] score matrix when dst = perm               */

/* 16-bit element type of activations, weights and outputs (accumulation is always fp32).
 * The reference's wrappers default to fp16 (kernels/fusedmoe_tilelang.py:257), the
 * benchmark contract is quoted in bf16; both run on the same kernels. */
#define MOE_DTYPE_BF16 0
#define MOE_DTYPE_F16 1

const char* moe_last_error(void);
int moe_abi_version(void);

/* Device properties the host side needs (SM count, sm_100 check). host out. */
int moe_device_info(int device, int* sm_count, int* cc_major, int* cc_minor);

/* ---- router: fused top-k + softmax -------------------------------------------
 * Replaces kernels/topk_softmax_baseline.py:39-66 (mode B), :15-36 (mode A),
 * :223-236 (mode A_RENORM) and the GPU op kernels/topk_softmax_tilelang.py:1103-1135.
 * logits fp32 [M,N] with row stride ld (elements).  scores fp32 [M,k]; indices
 * int64 [M,k] and/or indices32 int32 [M,k] (either may be NULL, not both).
 * Output is sorted by value descending; equal values come lowest index first;
 * -0.0 == +0.0; NaN ranks above every number.  No workspace.
 * N <= 1024 and k <= 64: one warp per row.  Otherwise (N <= 131072, k <= 4096):
 * radix select by a cluster of CTAs per row.
 */
int moe_topk_softmax(const float* logits, int64_t M, int64_t N, int64_t ld, int k, int mode,
                     float* scores, int64_t* indices, int32_t* indices32, int32_t* status,
                     void* stream);

/* ---- permutation / histogram ---------------------------------------------------
 * Replaces the argsort / bincount / cumsum of kernels/fusedmoe_baseline.py:123-134
 * and the host loops of kernels/fusedmoe_tilelang.py:338-372 (no D2H sync).
 * topk_idx: n = T*k expert ids, int64 (idx_is_int64 != 0) or int32, flattened
 * row-major.  counts int32 [E]; offsets int32 [E+1] exclusive prefix (offsets[E]=n);
 * perm int32 [n]: perm[p] = flat entry at expert-sorted position p (stable);
 * inv int32 [n]: inverse of perm.  perm / inv may be NULL.  Ids outside [0,E)
 * set status[0] and are skipped.  id_map (int32 [E], may be NULL) renumbers the
 * ids before counting (expert parallelism sorts by destination rank first).
 */
size_t moe_route_histogram_workspace(int64_t n, int E);
int moe_route_histogram(const void* topk_idx, int idx_is_int64, int64_t n, int E, const int32_t* id_map,
                        int32_t* counts, int32_t* offsets, int32_t* perm, int32_t* inv, void* ws,
                        size_t ws_bytes, int32_t* status, void* stream);

/* Same result as moe_route_histogram, for callers that cannot hand over a workspace.
 * This entry point has no counterpart in the reference.  Some hosts give a plug-in only
 * its input and output buffers and forbid it to create device memory of its own: a
 * serving loop that may not stall on the device-wide synchronisation an allocation can
 * cause, or an embedding runtime that owns the whole memory pool.  For them the count
 * table lives in a 1 MiB array built into the library's device image (present on every
 * GPU that loads the library until the process exits).
 *   - limit: ceil(n / 1024) * E <= 262144, otherwise MOE_ERR_UNSUPPORTED (use the
 *     workspace variant); with E = 256 that is n <= 1 048 576 routed entries;
 *   - the first call on each GPU looks up the array's device address; make that call
 *     outside any stream capture;
 *   - all calls on a GPU share the one array: two calls whose kernels may overlap on the
 *     device (different streams, no ordering between them) race and give wrong results.
 *     Calls ordered on one stream are safe, and nothing needs clearing between them;
 *   - the call itself allocates and frees nothing.
 */
int moe_route_histogram_static(const void* topk_idx, int idx_is_int64, int64_t n, int E,
                               const int32_t* id_map, int32_t* counts, int32_t* offsets,
                               int32_t* perm, int32_t* inv, int32_t* status, void* stream);

/* ---- row gather -----------------------------------------------------------------
 * dst[p, :] = src[perm[p] / div, :] for p < n_rows (rows of `cols` bf16, 16-byte
 * aligned, cols % 8 == 0).  Replaces the expert-stacking copy loops of
 * kernels/fusedmoe_tilelang.py:346-355 and X[sorted] in grouped_gemm_tilelang.py:700.
 * If w_src != NULL also w_dst[p] = w_src[perm[p]] (fp32 routing weights).
 */
int moe_gather_rows(const void* src, const int32_t* perm, int div, int64_t n_rows, int64_t cols,
                    void* dst, const float* w_src, float* w_dst, void* stream);

/* ---- expert grouped GEMM (tcgen05 / TMEM / TMA) -----------------------------------
 * Replaces kernels/grouped_gemm_baseline.py:14-57, kernels/grouped_gemm_tilelang.py:119-214
 * and the expert matmuls of kernels/fusedmoe_baseline.py:93-103,148-158 /
 * kernels/fusedmoe_tilelang.py:123-238.
 *   A        bf16 [rows, K] row-major, rows sorted by expert (expert e owns rows
 *            offsets[e] .. offsets[e+1]-1)
 *   B, B2    bf16 [E, N, K] (the reference's (E,I,H) layout: K contiguous);
 *            B2 is the "up" weight for MOE_GEMM_SILU_GATE, else NULL
 *   offsets  int32 [E+1] on the device (output of moe_route_histogram)
 *   dst_rows int32 [rows] or NULL: output row of sorted row r (PLAIN, SCALE_SCATTER)
 *   row_w    fp32 [rows]: routing weight of sorted row r (SCALE_SCATTER)
 *   Y        bf16 [*, N] row stride ldy (fp32 for MOE_GEMM_PLAIN_F32)
 *   max_rows rows of A that may be read (its allocation; >= offsets[E]); rows beyond
 *            offsets[E] are never written
 *   expected_rows  how many rows the caller expects to be live (0 = max_rows): only
 *            steers the choice of tile shape when max_rows is a buffer capacity
 * K % 8 == 0, N % 8 == 0.  Workspace: none.
 */
int moe_grouped_gemm(int epilogue, const void* A, const void* B, const void* B2,
                     const int32_t* offsets, const int32_t* dst_rows, const float* row_w, void* Y,
                     int64_t ldy, int64_t max_rows, int64_t expected_rows, int K, int N, int E,
                     int dtype, int32_t* status, void* stream);

/* moe_grouped_gemm with the row gather fused into the operand pipeline: sorted row r of A is
 * row gather_idx[r] / gather_div of X [x_rows, K] (gather_idx = `perm` of moe_route_histogram,
 * gather_div = k), fetched by the kernel itself, so that neither moe_gather_rows nor the sorted
 * copy of the activations is needed.  Same role as X[sorted_indices] feeding the kernel in
 * kernels/grouped_gemm_tilelang.py:700 and the stacking loops of kernels/fusedmoe_tilelang.py:346-355.
 * gather_idx int32 [max_rows]; indices are clamped to x_rows - 1.  K % 64 == 0.  Other arguments as
 * moe_grouped_gemm.
 */
int moe_grouped_gemm_gathered(int epilogue, const void* X, int64_t x_rows, const int32_t* gather_idx,
                              int gather_div, const void* B, const void* B2, const int32_t* offsets,
                              const int32_t* dst_rows, const float* row_w, void* Y, int64_t ldy,
                              int64_t max_rows, int64_t expected_rows, int K, int N, int E, int dtype,
                              int32_t* status, void* stream);

/* ---- combine ----------------------------------------------------------------------
 * out[t,:] = (shared ? shared[t,:] : 0) + sum_{s<k} c(t,s) * Yk[r(t,s),:], fp32 sum in
 * slot order, rounded once to bf16, with f = t*k+s, r = row_of ? row_of[f] : f and
 * c = scale ? scale[f] : 1.  Replaces scatter_reduce_ + add of
 * kernels/fusedmoe_baseline.py:90,161-166 (and, with scale, the weighting of :156-158
 * when expert outputs come back unscaled from other ranks).  H % 8 == 0.
 */
int moe_combine(const void* Yk, const void* shared, const int32_t* row_of, const float* scale,
                int64_t T, int k, int64_t H, int dtype, void* out, void* stream);

/* ---- router logits ------------------------------------------------------------------
 * logits[t,e] = sum_h x[t,h] * Wr[e,h], 16-bit inputs, fp32 accumulate and output.
 * Replaces kernels/fusedmoe_baseline.py:72.  H % 8 == 0.
 */
int moe_router_logits(const void* x, const void* Wr, int64_t T, int H, int E, int dtype, float* logits,
                      int32_t* status, void* stream);

/* Router GEMM + top-k + softmax in ONE kernel: the [T,E] logits never travel through memory (they are
 * written only if logits_out != NULL).  Same result as moe_router_logits / moe_grouped_gemm(PLAIN_F32)
 * followed by moe_topk_softmax on those logits: indices sorted by value, ties lowest index first.
 * Replaces the fused family of kernels/router_gemm_topk_softmax.py:148-1141.
 *   x [T,H], Wr [E,H] 16-bit (dtype), fp32 accumulation; scores fp32 [T,k]; indices int64 and / or
 *   indices32 int32 [T,k]; mode as moe_topk_softmax.
 * Two kernels behind it: E <= 32 with E*H*2 <= 200 KB - CUDA cores, one warp per token, any k <= E;
 * otherwise E % 8 == 0, E <= 256, k <= 8 - tcgen05 GEMM whose epilogue selects from the TMEM accumulator row.
 * Other shapes: MOE_ERR_UNSUPPORTED (use the two separate calls).
 */
int moe_router_topk(const void* x, const void* Wr, int64_t T, int H, int E, int k, int mode, int dtype,
                    float* scores, int64_t* indices, int32_t* indices32, float* logits_out,
                    int32_t* status, void* stream);

/* ---- expert-parallel regroup table -----------------------------------------------------
 * No counterpart in the reference (it has no multi-GPU code).  recv_counts int32
 * [G][E_local]: rows received from source rank s for local expert j, laid out
 * source-major in the receive buffer.  Writes offsets int32 [E_local+1] (expert-major
 * exclusive prefix, the `offsets` of moe_grouped_gemm) and src_row int32 [n_recv]:
 * the receive-buffer row held at expert-major position p (gather list before the up
 * GEMM, dst_rows of the down GEMM).  G * E_local <= 20000.
 */
int moe_ep_regroup(const int32_t* recv_counts, int G, int E_local, int32_t* offsets,
                   int32_t* src_row, void* stream);

/* Router for few tokens (decode-sized batches): with only ceil(T/128) row tiles the router GEMM would keep a handful
 * of SMs busy, so it is split along K into S slices (1..16, chosen from T and H) that give every SM a tile; a second
 * kernel adds a token's slices in fixed order and does the top-k + softmax.  Same outputs as moe_router_topk; the
 * logits (logits_out, optional) are the slice sums, i.e. equal to an unsplit fp32 accumulation up to summation order.
 * E % 8 == 0, E <= 256, k <= 32.  ws: moe_router_topk_splitk_workspace(T, H, E) bytes.
 */
size_t moe_router_topk_splitk_workspace(int64_t T, int H, int E);
int moe_router_topk_splitk(const void* x, const void* Wr, int64_t T, int H, int E, int k, int mode, int dtype,
                           float* scores, int64_t* indices, int32_t* indices32, float* logits_out, void* ws,
                           size_t ws_bytes, int32_t* status, void* stream);

/* ---- the whole layer in one call -----------------------------------------------------
 * FusedMoEPyTorch.forward / FusedMoETileLang.forward (kernels/fusedmoe_baseline.py:46-91,
 * kernels/fusedmoe_tilelang.py:309-417) as one C call that sequences the entry points above on
 * `stream`: router (logits fp32 [T,E] if given, else x . router_weight^T) -> softmax over all experts,
 * top-k without renormalisation -> histogram / offsets / permutation -> up GEMM (gathering its rows,
 * SiLU gate fused) -> down GEMM (routing weight + scatter fused) -> combine with the shared expert.
 *   x [T,H]; router_weight [E,H] or NULL; shared_gate, shared_up [SI,H], shared_down [H,SI] (SI = 0: no
 *   shared expert, pointers ignored); routed_gate, routed_up [E,I,H], routed_down [E,H,I]; out [T,H]; all
 *   16-bit of `dtype`.  ws: moe_layer_workspace(T,k,H,I,E,SI) bytes of device scratch, 256-byte aligned.
 *   side_stream: optional second stream for the shared expert (fork / join by events; NULL = same stream).
 * Results are bit-identical to issuing the calls one by one.  No host synchronisation.  With a side stream the
 * fork / join uses two events that the library keeps per device: host threads that call this function for the
 * same device at the same time must pass side_stream = NULL.  Every return after the fork, errors included, first
 * makes `stream` wait for the side stream again, so a stream capture around the call is never left unjoined.
 * Shared expert as one more group: when SI == I, H % 64 == 0 and the shared weights lie directly behind the routed
 * ones in memory (shared_gate == routed_gate + E*I*H elements, likewise up and down: one [E+1, ...] tensor per
 * projection), the shared expert runs as expert E of the routed grouped GEMMs - every token gets k + 1 entries, the
 * last with weight 1 - and the whole layer is five launches on `stream` (the reference overlaps its shared and
 * routed kernels on two streams instead, kernels/fusedmoe_tilelang.py:428-553).  Same bits as the other form.
 * The router kernel (one kernel, split along K, or GEMM then top-k) is chosen from T, H and E: fp32 logits of one
 * token can differ in summation order between batch sizes, so a near-tie may route differently in another batch size.
 */
size_t moe_layer_workspace(int64_t T, int k, int H, int I, int E, int SI);
int moe_layer_forward(const void* x, const void* router_weight, const float* logits, const void* shared_gate,
                      const void* shared_up, const void* shared_down, const void* routed_gate,
                      const void* routed_up, const void* routed_down, int64_t T, int H, int I, int E, int k,
                      int SI, int dtype, void* ws, size_t ws_bytes, void* out, int32_t* status, void* stream,
                      void* side_stream);

/* ---- mHC pre / post blocks ---------------------------------------------------------------
 * The operators on either side of the MoE layer in the model the reference targets
 * (kernels/mhc_baseline.py:48-163; recommended entry points kernels/mhc_tilelang.py:494-582).
 *   R = 2*hc_mult + hc_mult^2, K = hc_mult*hidden.  hc_mult 2 or 4, hidden % 8 == 0, K*2 <= 200 KB.
 * moe_mhc_split_weights: fn fp32 [R, K] -> fn3 bf16 [3*R, K] = hi, mid, lo with hi+mid+lo = fn to 24 bits;
 *   done once per weight, lets the skinny GEMM run on the tensor cores in bf16 at fp32 accuracy.
 * moe_mhc_pre: residual bf16 [T, hc_mult, hidden] ->
 *   post_mix fp32 [T, hc_mult], comb_mix fp32 [T, hc_mult, hc_mult], layer_input bf16 [T, hidden].
 *   mixes = (residual_flat . fn^T) * rsqrt(mean(residual_flat^2) + rms_eps) * scale + base;
 *   pre = sigmoid(mixes[:hc]) + hc_pre_eps; post_mix = sigmoid(mixes[hc:2hc]) * hc_post_mult_value;
 *   comb_mix = Sinkhorn(mixes[2hc:], sinkhorn_repeat, hc_sinkhorn_eps); layer_input = sum_m pre[m]*residual[m].
 *   ws: moe_mhc_pre_workspace(T, hc_mult, hidden) bytes of device scratch (the split-K slices of the GEMM).
 * moe_mhc_post: out bf16 [T, hc_mult, hidden] = x[T,hidden] * post_layer_mix[T,hc] + comb_res_mix[T,hc,hc]^T @ residual.
 */
size_t moe_mhc_pre_workspace(int64_t T, int hc_mult, int64_t hidden);
int moe_mhc_split_weights(const float* fn, int rows, int64_t K, void* fn3, void* stream);
int moe_mhc_pre(const void* residual, const void* fn3, const float* hc_scale, const float* hc_base, int64_t T,
                int hc_mult, int64_t hidden, float rms_eps, float hc_pre_eps, float hc_sinkhorn_eps,
                float hc_post_mult_value, int sinkhorn_repeat, void* ws, size_t ws_bytes, float* post_mix,
                float* comb_mix, void* layer_input, int32_t* status, void* stream);
int moe_mhc_post(const void* x, const void* residual, const float* post_layer_mix, const float* comb_res_mix,
                 int64_t T, int hc_mult, int64_t hidden, void* out, void* stream);

/* ---- expert parallelism over peer memory ---------------------------------------------
 * No counterpart in the reference.  cnt_all int32 [G][G*E_local]: cnt_all[s][v] = rows that
 * source rank s routes to virtual expert v = dest_rank*E_local + slot (all-gather of the
 * per-rank histograms taken with id_map).  moe_ep_plan derives this rank's tables:
 *   offsets  int32 [E_local+1]  expert-major start of each local expert in the receive buffer
 *   dst_base int32 [G*E_local]  start of this rank's rows for v inside the destination's buffer
 *   ret_rank, ret_row int32 [rows received]: source rank and row in the source's return
 *            buffer (its sorted order) for the row held at expert-major position q.
 * moe_ep_dispatch copies the activation row of every routed entry (this rank's sorted order,
 * perm / topk_idx / id_map / offsets from moe_route_histogram) into peer_recv[dest] at its
 * expert-major row: plain stores to peer memory, no collective library.  peer_recv: host
 * array of G device pointers (one receive buffer per rank, this rank's own included).
 * Only rows bound for local expert slots [slot_lo, slot_hi) of their destination are moved, so
 * the dispatch of a second group of experts can overlap the GEMMs of the first.
 * moe_grouped_gemm_peer_scatter is moe_grouped_gemm(MOE_GEMM_PLAIN) whose epilogue stores row r
 * into peer_base[row_rank[r]] at row dst_rows[r]: the combine exchange fused into the down GEMM.
 * Callers order the phases across ranks (a barrier after dispatch and after the scatter).
 */
int moe_ep_plan(const int32_t* cnt_all, int G, int E_local, int my_rank, int32_t* offsets,
                int32_t* dst_base, int32_t* ret_rank, int32_t* ret_row, void* stream);
int moe_ep_dispatch(const void* x, const int32_t* perm, const int32_t* topk_idx,
                    const int32_t* id_map, const int32_t* offsets, const int32_t* dst_base, int k,
                    int E_local, int slot_lo, int slot_hi, int64_t n, int64_t H,
                    void* const* peer_recv, int G, void* stream);
/* De-duplicated dispatch: a token row travels to a destination rank once, whatever the number of its k experts
 * there (bytes over NVLink fall by k / E[distinct ranks per token]); the destination's up GEMM then gathers its
 * expert-major rows through an index list that the sources write beside the rows (moe_grouped_gemm_gathered with
 * gather_div = 1 on the receive buffer).
 *   moe_ep_unique: urank int32 [Tl, G]: u(t,d) = tokens t' < t of this rank with an expert on rank d, or -1 if token
 *     t has none there; ucount int32 [G] = tokens per destination.  The histogram all-gather then carries
 *     E + G integers per rank: counts, then ucount.
 *   moe_ep_plan_dedup: moe_ep_plan on that [G][E+G] table, plus u_base int32 [G]: first row of this rank's tokens in
 *     each destination's receive buffer.
 *   moe_ep_dispatch_dedup: stores row x[t] to peer_recv[d] at row u_base[d] + u(t,d) for every (t,d) with u >= 0,
 *     and for every routed entry p the received-row number into peer_gidx[d] (int32 [capacity]) at the entry's
 *     expert-major position dst_base[v] + (p - offsets[v]).
 */
int moe_ep_unique(const int32_t* topk_idx, const int32_t* id_map, int64_t Tl, int k, int E_local, int G,
                  int32_t* urank, int32_t* ucount, void* stream);
int moe_ep_plan_dedup(const int32_t* cnt_all, int G, int E_local, int my_rank, int32_t* offsets,
                      int32_t* dst_base, int32_t* ret_rank, int32_t* ret_row, int32_t* u_base, void* stream);
int moe_ep_dispatch_dedup(const void* x, const int32_t* perm, const int32_t* topk_idx, const int32_t* id_map,
                          const int32_t* offsets, const int32_t* dst_base, const int32_t* urank,
                          const int32_t* u_base, int k, int E_local, int64_t n, int64_t Tl, int64_t H,
                          void* const* peer_recv, void* const* peer_gidx, int G, void* stream);
/* Barrier between the G ranks over peer memory, with a time limit.  No counterpart in the reference.
 *   peer_flags: host array of G device pointers; entry g addresses rank g's flag block, int32 [4][16] (channel, slot),
 *     zero-filled once, writable by every rank (symmetric / peer-mapped memory).
 *   epoch: the number of this barrier on `channel` (1, 2, 3, ... the same on every rank).  Each rank stores the epoch
 *     into slot [my_rank] of every peer's block - after a system-scope fence, so the rows it wrote into peer buffers
 *     before the call are visible first - and waits until all G slots of its own block have reached it.
 *   A wait longer than timeout_us gives up: status = {2, 40 + channel, peer} and the kernel returns (never a hang);
 *     kernels enqueued behind it then run on incomplete data, so the caller must check `status` before using results.
 */
int moe_ep_barrier(void* const* peer_flags, int G, int my_rank, int channel, int32_t epoch, int64_t timeout_us,
                   int32_t* status, void* stream);
/* All-gather of the ranks' routing histograms over peer memory, closed by the same time-limited barrier: one launch
 * instead of a collective library call.  No counterpart in the reference.
 *   counts [n_counts] (+ extra [n_extra], may be null with n_extra = 0): this rank's vector, on the device.
 *   peer_tables: host array of G device pointers; entry g addresses rank g's table, int32 [2][G][n_counts + n_extra],
 *     writable by every rank.  The kernel stores this rank's vector into row [slot][my_rank] of every table, then
 *     runs barrier `epoch` of `channel` (see moe_ep_barrier); behind it, table [slot] of this rank holds every rank's
 *     vector.  slot alternates 0, 1 from step to step so that a rank one step ahead does not overwrite rows in use.
 *   A wait that runs out leaves status = {2, 40 + channel, peer}, as in moe_ep_barrier.
 */
int moe_ep_share_counts(const int32_t* counts, int n_counts, const int32_t* extra, int n_extra,
                        void* const* peer_tables, int slot, void* const* peer_flags, int G, int my_rank,
                        int channel, int32_t epoch, int64_t timeout_us, int32_t* status, void* stream);
int moe_grouped_gemm_peer_scatter(const void* A, const void* B, const int32_t* offsets,
                                  const int32_t* row_rank, const int32_t* dst_rows,
                                  void* const* peer_base, int n_peers, int64_t ldy, int64_t max_rows,
                                  int64_t expected_rows, int K, int N, int E, int dtype,
                                  int32_t* status, void* stream);

/* ---- self-test of the bounded waits ---------------------------------------------------------
 * No counterpart in the reference.  Launches one warp that waits, through the GEMM kernels' own barrier-wait
 * routine, on a barrier nobody arrives on, with a limit of limit_us microseconds (1 .. 1 000 000).  The wait runs
 * out: status (device int32[MOE_STATUS_WORDS]) receives {2, 99, 0}, *outcome (device int32, may be NULL) 0, and
 * the kernel returns.  Lets a test see the give-up path without a faulty GEMM; the stream stays usable.
 */
int moe_debug_wait_probe(int64_t limit_us, int32_t* status, int32_t* outcome, void* stream);

/* ---- index checks of the checked build ---------------------------------------------------------
 * No counterpart in the reference.  A build of the library with -DMOE_BOUNDS_CHECK (python -m tilelang_moe_b200.build
 * --check -> libmoe_b200_check.so, same ABI) compares every row index it takes out of an index table with the size of
 * the buffer it addresses before following it: scatter destinations (site 1) and gather sources (site 2) of the
 * grouped GEMMs, the row table of moe_combine (site 3).  An index outside the buffer is not followed (the store is
 * skipped, the gather reads the last row instead, the combine adds nothing) and the first one is remembered.
 * This call waits for `stream`, writes {4, site, index} of the first such index since the last call (or {0,0,0})
 * to the host array out3, clears the record, and returns 1 in the checked build, 0 in the normal one (whose kernels
 * carry no checks and always report {0,0,0}).
 */
int moe_debug_bounds_status(int32_t* out3, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_B200_H_ */
