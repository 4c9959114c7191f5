// Fused top-k + softmax router kernels for sm_100a.
//
// Three kernels behind one entry point:
//   * topk_tile_kernel   rows staged in shared memory by cp.async, 1-8 threads per row keep a sorted
//                        k-entry list in registers; N <= 1024, k <= 8, aligned rows, M >= 64.
//   * topk_warp_kernel   one warp per row, the row lives in registers; k rounds of
//                        warp-wide arg-max by redux; N <= 1024, k <= 64.
//   * topk_radix_kernel  a thread-block cluster per row; each CTA stages its slice
//                        of the row in shared memory once, the cluster runs a
//                        3-pass (11/11/10 bit) radix select on order-preserving
//                        keys with histograms combined over distributed shared
//                        memory, the selected entries are gathered into the leading
//                        CTA, sorted (bitonic, 64-bit key|index) and normalised.
// Both read every logit exactly once from global memory.
//
// Ordering contract: descending by value, equal values lowest index first,
// -0.0 == +0.0, NaN above every number.
#include "common.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace moe {

// ------------------------------------------------------------------------------------
// warp-per-row kernel
// ------------------------------------------------------------------------------------
template <int ELTS, int VEC>
__device__ __forceinline__ uint32_t warp_col(int i, int lane) {
  if (VEC == 4) return (uint32_t)((i >> 2) * 128 + lane * 4 + (i & 3));
  return (uint32_t)(i * 32 + lane);
}

template <int ELTS, int VEC>
__global__ void __launch_bounds__(128)
topk_warp_kernel(const float* __restrict__ logits, int64_t M, int N, int64_t ld, int k, int mode,
                 float* __restrict__ scores, int64_t* __restrict__ idx64, int32_t* __restrict__ idx32) {
  const unsigned FULL = 0xFFFFFFFFu;
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * 4;
  for (int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5); row < M; row += nwarps) {
    const float* p = logits + row * ld;
    uint32_t key[ELTS];
    if (VEC == 4) {
#pragma unroll
      for (int c = 0; c < ELTS / 4; ++c) {
        const int col0 = c * 128 + lane * 4;
        if (col0 < N) {  // N % 4 == 0 on this path: the whole vector is in range
          const float4 v = __ldg(reinterpret_cast<const float4*>(p + col0));
          key[c * 4 + 0] = float_to_key(v.x);
          key[c * 4 + 1] = float_to_key(v.y);
          key[c * 4 + 2] = float_to_key(v.z);
          key[c * 4 + 3] = float_to_key(v.w);
        } else {
          key[c * 4 + 0] = key[c * 4 + 1] = key[c * 4 + 2] = key[c * 4 + 3] = 0u;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < ELTS; ++i) {
        const int col = i * 32 + lane;
        key[i] = col < N ? float_to_key(__ldg(p + col)) : 0u;
      }
    }

    // lane-local best (strict > keeps the lowest column among equals: columns grow with i)
    uint32_t bk = 0u, bc = 0xFFFFFFFFu;
#pragma unroll
    for (int i = 0; i < ELTS; ++i) {
      if (key[i] > bk) { bk = key[i]; bc = warp_col<ELTS, VEC>(i, lane); }
    }
    const uint32_t maxkey = __reduce_max_sync(FULL, bk);
    const float vmax = key_to_float(maxkey);

    float rowsum = 0.f;
    if (mode != MOE_TOPK_MODE_B) {
#pragma unroll
      for (int i = 0; i < ELTS; ++i)
        if (key[i] != 0u) rowsum += expf(key_to_float(key[i]) - vmax);
      rowsum = warp_sum(rowsum);
    }

    uint32_t selk0 = 0u, selk1 = 0u, selc0 = 0u, selc1 = 0u;
    for (int r = 0; r < k; ++r) {
      const uint32_t m = __reduce_max_sync(FULL, bk);
      const uint32_t c = __reduce_min_sync(FULL, (bk == m) ? bc : 0xFFFFFFFFu);
      if (lane == (r & 31)) {
        if (r < 32) { selk0 = m; selc0 = c; } else { selk1 = m; selc1 = c; }
      }
      if (bk == m && bc == c) {  // the owning lane retires the winner and rescans its registers
        bk = 0u; bc = 0xFFFFFFFFu;
#pragma unroll
        for (int i = 0; i < ELTS; ++i) {
          if (warp_col<ELTS, VEC>(i, lane) == c) key[i] = 0u;
          if (key[i] > bk) { bk = key[i]; bc = warp_col<ELTS, VEC>(i, lane); }
        }
      }
    }

    const bool v0 = lane < k, v1 = lane + 32 < k;
    float e0 = v0 ? expf(key_to_float(selk0) - vmax) : 0.f;
    float e1 = v1 ? expf(key_to_float(selk1) - vmax) : 0.f;
    float s0, s1;
    if (mode == MOE_TOPK_MODE_B) {
      const float denom = warp_sum(e0 + e1);
      s0 = e0 / denom; s1 = e1 / denom;
    } else {
      s0 = e0 / rowsum; s1 = e1 / rowsum;
      if (mode == MOE_TOPK_MODE_A_RENORM) {
        const float s = warp_sum(s0 + s1);
        s0 = s0 / s; s1 = s1 / s;
      }
    }
    const int64_t o = row * (int64_t)k;
    if (v0) {
      scores[o + lane] = s0;
      if (idx64) idx64[o + lane] = (int64_t)selc0;
      if (idx32) idx32[o + lane] = (int32_t)selc0;
    }
    if (v1) {
      scores[o + lane + 32] = s1;
      if (idx64) idx64[o + lane + 32] = (int64_t)selc1;
      if (idx32) idx32[o + lane + 32] = (int32_t)selc1;
    }
  }
}

template <int ELTS, int VEC>
static int launch_warp(const float* logits, int64_t M, int N, int64_t ld, int k, int mode, float* scores,
                       int64_t* idx64, int32_t* idx32, int sm_count, cudaStream_t st) {
  int64_t blocks = ceil_div64(M, 4);
  const int64_t cap = (int64_t)sm_count * 16;
  if (blocks > cap) blocks = cap;
  topk_warp_kernel<ELTS, VEC><<<(unsigned)blocks, 128, 0, st>>>(logits, M, N, ld, k, mode, scores, idx64, idx32);
  MOE_CHECK_LAUNCH("topk_warp_kernel");
  return MOE_OK;
}


// ------------------------------------------------------------------------------------
// thread-per-row kernel for small k (k <= 8, N <= 1024, 16-byte aligned rows)
//
// A CTA of 128 threads stages a tile of rows in shared memory with 16-byte cp.async (coalesced, the only
// read of the logits), then TPR = 1, 2, 4 or 8 adjacent threads share one row: each scans its part with a
// sorted k-entry list in registers (compare against the k-th best, insert by a compare-exchange chain),
// partial lists are merged over shuffles, and the first thread of the row normalises and writes.
// The instruction cost per row is a quarter of the warp-per-row kernel's; three CTAs per SM keep ~190 KB of
// loads in flight.  Keys are signed integers ordered like the floats: x + 0.0f folds -0.0 into +0.0 and every
// NaN into the canonical positive NaN, which ranks above +inf.
// ------------------------------------------------------------------------------------
constexpr int TILE_THREADS = 128;
constexpr int MAX_PART_VECS = 32;   // 16-byte vectors one thread scans: at most 128 floats of a row per thread


template <int K, int TPR>
__global__ void __launch_bounds__(TILE_THREADS)
topk_tile_kernel(const float* __restrict__ logits, int64_t M, int N, int64_t ld, int k, int mode, int rows_per_tile,
                 float* __restrict__ scores, int64_t* __restrict__ idx64, int32_t* __restrict__ idx32) {
  extern __shared__ __align__(16) float tile[];
  __shared__ unsigned char queue[(2 * K - 1) * TILE_THREADS];   // per thread: vectors that can hold one of its K largest
  const int tid = threadIdx.x;
  const int pitch = N + 4;                         // floats; 16-byte aligned rows, conflict-free 16-byte reads
  const int vec_per_row = N >> 2;
  const int row_in_tile = tid / TPR, part = tid % TPR;
  const int part_vecs = (vec_per_row + TPR - 1) / TPR;
  const int64_t n_tiles = (M + rows_per_tile - 1) / rows_per_tile;
  // staging walk of this thread: first vector, and the step of 128 vectors in rows / columns / bytes
  const int ld_r0 = tid / vec_per_row, ld_c0 = tid % vec_per_row;
  const int ld_dr = TILE_THREADS / vec_per_row, ld_dc = TILE_THREADS % vec_per_row;
  const int64_t ld_dsrc = (int64_t)ld_dr * ld + ld_dc * 4;
  const uint32_t ld_ddst = (uint32_t)(ld_dr * pitch + ld_dc * 4) * 4u;
  const uint32_t tile_s = (uint32_t)__cvta_generic_to_shared(tile);

  for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
    const int64_t row0 = t * rows_per_tile;
    const int rows = (int)((M - row0) < rows_per_tile ? (M - row0) : rows_per_tile);
    __syncthreads();                               // previous tile fully consumed
    {   // thread t copies vectors t, t + 128, ... of the tile; (row, column) advance by a fixed step, no division
      int r = ld_r0, c = ld_c0;
      const float* src = logits + (row0 + r) * ld + c * 4;
      uint32_t dst = tile_s + (uint32_t)(r * pitch + c * 4) * 4u;
      while (r < rows) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        r += ld_dr; c += ld_dc;
        src += ld_dsrc; dst += ld_ddst;
        if (c >= vec_per_row) { c -= vec_per_row; r += 1; src += ld - N; dst += (uint32_t)(pitch - N) * 4u; }
      }
    }
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    const bool active = row_in_tile < rows;
    int kv[K], ki[K];
#pragma unroll
    for (int j = 0; j < K; ++j) { kv[j] = (int)0x80000000; ki[j] = 0; }
    const float* rowp = tile + row_in_tile * pitch;
    const int v_lo = part * part_vecs, v_hi = min(vec_per_row, v_lo + part_vecs);
    if (active) {
      // Pass 1, branch-free: the largest key of every 4-element vector, and the K largest of those (keys only: a
      // max / min pair per list entry).  The K largest elements of the part sit in vectors whose largest key is at
      // least the K-th largest vector maximum V: at most K-1 vectors lie above V, and of those equal to V only the
      // first K in column order can matter.
      int vm[MAX_PART_VECS];
      constexpr int CH = 2;                   // independent lists (two dependency chains in flight), one per half of the part
      constexpr int QV = MAX_PART_VECS / CH;
      int va[CH][K];
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int j = 0; j < K; ++j) va[c][j] = (int)0x80000000;
#pragma unroll
      for (int u = 0; u < QV; ++u) {
        int m[CH];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          m[c] = (int)0x80000000;
          if (v_lo + u + c * QV < v_hi) {
            const float4 x = *reinterpret_cast<const float4*>(rowp + (v_lo + u + c * QV) * 4);
            m[c] = max(max(float_to_ikey(x.x), float_to_ikey(x.y)), max(float_to_ikey(x.z), float_to_ikey(x.w)));
          }
          vm[u + c * QV] = m[c];
        }
#pragma unroll
        for (int j = 0; j < K; ++j) {
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            const int hi = max(va[c][j], m[c]);
            m[c] = min(va[c][j], m[c]);
            va[c][j] = hi;
          }
        }
      }
#pragma unroll
      for (int c = 1; c < CH; ++c) {          // the K largest of all lists end up in va[0]
#pragma unroll
        for (int i = 0; i < K; ++i) {
          int m = va[c][i];
#pragma unroll
          for (int j = 0; j < K; ++j) {
            const int hi = max(va[0][j], m);
            m = min(va[0][j], m);
            va[0][j] = hi;
          }
        }
      }
      // Pass 2, predicated: queue the vectors that can hold a winner (this thread's slots in shared memory)
      const int V = va[0][K - 1];
      int cnt = 0, n_eq = 0;
#pragma unroll
      for (int u = 0; u < MAX_PART_VECS; ++u) {
        const bool eq = vm[u] == V && n_eq < K && v_lo + u < v_hi;
        const bool take = (vm[u] > V) || eq;
        if (take) queue[cnt * TILE_THREADS + tid] = (unsigned char)u;
        cnt += take ? 1 : 0;
        n_eq += eq ? 1 : 0;
      }
      // Pass 3: the queued vectors (about K of them) go through the sorted list with their columns, largest element
      // first, lowest column first among equal ones
      for (int q = 0; q < cnt; ++q) {
        const int v = v_lo + (int)queue[q * TILE_THREADS + tid];
        const float4 x = *reinterpret_cast<const float4*>(rowp + v * 4);
        int c0 = float_to_ikey(x.x), c1 = float_to_ikey(x.y), c2 = float_to_ikey(x.z), c3 = float_to_ikey(x.w);
        int m = max(max(c0, c1), max(c2, c3));
        while (m >= V && m > kv[K - 1]) {     // nothing below V can be among the K largest: K vector maxima are >= V
          const int sel = c0 == m ? 0 : (c1 == m ? 1 : (c2 == m ? 2 : 3));
          list_insert<K>(kv, ki, m, v * 4 + sel);
          c0 = sel == 0 ? (int)0x80000000 : c0;
          c1 = sel == 1 ? (int)0x80000000 : c1;
          c2 = sel == 2 ? (int)0x80000000 : c2;
          c3 = sel == 3 ? (int)0x80000000 : c3;
          m = max(max(c0, c1), max(c2, c3));
        }
      }
    }
    // merge the parts of a row: the lower part keeps its entries ahead of equal ones from higher columns
#pragma unroll
    for (int d = 1; d < TPR; d <<= 1) {
      int ok[K], oi[K];
#pragma unroll
      for (int j = 0; j < K; ++j) {
        ok[j] = __shfl_xor_sync(0xFFFFFFFFu, kv[j], d);
        oi[j] = __shfl_xor_sync(0xFFFFFFFFu, ki[j], d);
      }
      if ((part & d) == 0) {
#pragma unroll
        for (int j = 0; j < K; ++j) list_insert<K>(kv, ki, ok[j], oi[j]);
      }
    }
    // full-row softmax denominator for the conventions that normalise over all N
    float rowsum = 0.f;
    const float vmax = ikey_to_float(TPR == 1 ? kv[0] : __shfl_sync(0xFFFFFFFFu, kv[0], (tid & 31) - part));
    if (mode != MOE_TOPK_MODE_B) {
      if (active)
        for (int v = v_lo; v < v_hi; ++v) {
          const float4 x = *reinterpret_cast<const float4*>(rowp + v * 4);
          rowsum += expf(x.x - vmax) + expf(x.y - vmax) + expf(x.z - vmax) + expf(x.w - vmax);
        }
#pragma unroll
      for (int d = 1; d < TPR; d <<= 1) rowsum += __shfl_xor_sync(0xFFFFFFFFu, rowsum, d);
    }
    if (active && part == 0) {
      float e[K];
      float denom = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        e[j] = j < k ? expf(ikey_to_float(kv[j]) - vmax) : 0.f;
        denom += e[j];
      }
      if (mode != MOE_TOPK_MODE_B) denom = rowsum;
      float renorm = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) { e[j] = e[j] / denom; renorm += e[j]; }
      const int64_t o = (row0 + row_in_tile) * (int64_t)k;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (j < k) {
          scores[o + j] = mode == MOE_TOPK_MODE_A_RENORM ? e[j] / renorm : e[j];
          if (idx64) idx64[o + j] = (int64_t)ki[j];
          if (idx32) idx32[o + j] = (int32_t)ki[j];
        }
      }
    }
  }
}

template <int K, int TPR>
static int launch_tile(const float* logits, int64_t M, int N, int64_t ld, int k, int mode, float* scores,
                       int64_t* idx64, int32_t* idx32, int sm_count, cudaStream_t st) {
  const int rows_per_tile = TILE_THREADS / TPR;
  const size_t smem = (size_t)rows_per_tile * (N + 4) * sizeof(float);
  if (smem > 48 * 1024)   // per device, cheap: set on every such launch
    MOE_CUDA_CHECK(cudaFuncSetAttribute(topk_tile_kernel<K, TPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024));
  int64_t blocks = ceil_div64(M, rows_per_tile);
  const int64_t cap = (int64_t)sm_count * 3;
  if (blocks > cap) blocks = cap;
  topk_tile_kernel<K, TPR><<<(unsigned)blocks, TILE_THREADS, smem, st>>>(logits, M, N, ld, k, mode, rows_per_tile, scores,
                                                                        idx64, idx32);
  MOE_CHECK_LAUNCH("topk_tile_kernel");
  return MOE_OK;
}

// ------------------------------------------------------------------------------------
// cluster radix-select kernel
// ------------------------------------------------------------------------------------
constexpr int RT = 512;             // threads per CTA
constexpr int RWARPS = RT / 32;
constexpr int RBINS = 2048;         // histogram bins (11-bit digit)
constexpr int RBPT = RBINS / RT;    // bins owned by one thread in the scan (4)
constexpr int RCTRL_BYTES = 256;
constexpr int RMAX_SLICE = 16384;   // keys one CTA stages (64 KB)
constexpr int RMAX_KPAD = 4096;

struct RadixCtrl {
  uint32_t warp_tot[RWARPS];
  double warp_d[RWARPS];
  uint32_t sel_bin;
  uint32_t k_rem;
  uint32_t sel_count;
  uint32_t blk_maxkey;
  uint32_t loc_count;   // selected entries compacted in this CTA
  uint32_t loc_base;    // their first slot in the leading CTA's buffer
  double blk_sum;
};
static_assert(sizeof(RadixCtrl) <= RCTRL_BYTES, "control block too large");

__device__ __forceinline__ uint64_t pack_entry(uint32_t key, uint32_t col) {
  return ((uint64_t)key << 32) | (uint64_t)(0xFFFFFFFFu - col);
}

// Sum of one value per thread over the CTA in a fixed order; result valid in every thread.
// Softmax denominators over thousands of terms are accumulated in fp64 so that the only
// rounding left in a score is that of expf and of the final division.
__device__ __forceinline__ double block_sum_ordered(double v, RadixCtrl* ctrl, int lane, int wid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  __syncthreads();
  if (lane == 0) ctrl->warp_d[wid] = v;
  __syncthreads();
  double t = 0.0;
#pragma unroll
  for (int w = 0; w < RWARPS; ++w) t += ctrl->warp_d[w];
  return t;
}

// Descending bitonic sort of RT*EPT 64-bit entries held EPT per thread (entry g = tid*EPT + e).
// Exchanges at distance < EPT stay in registers, distance < 32*EPT go through warp shuffles, and only the
// few long-distance stages of the last merges use shared memory with a block barrier.
template <int EPT>
__device__ __forceinline__ void block_sort_desc(uint64_t* sbuf, int tid) {
  constexpr int NSORT = RT * EPT;
  uint64_t v[EPT];
#pragma unroll
  for (int e = 0; e < EPT; ++e) v[e] = sbuf[tid * EPT + e];
  for (int size = 2; size <= NSORT; size <<= 1) {
    int stride = size >> 1;
    // long distance: through shared memory
    for (; stride >= 32 * EPT; stride >>= 1) {
      __syncthreads();
#pragma unroll
      for (int e = 0; e < EPT; ++e) sbuf[tid * EPT + e] = v[e];
      __syncthreads();
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        const int g = tid * EPT + e;
        const uint64_t o = sbuf[g ^ stride];
        const bool keep_max = ((g & stride) == 0) == ((g & size) == 0);
        v[e] = keep_max ? (v[e] > o ? v[e] : o) : (v[e] < o ? v[e] : o);
      }
    }
    // inside a warp: shuffles
    for (; stride >= EPT; stride >>= 1) {
      const int lx = stride / EPT;
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        const int g = tid * EPT + e;
        const uint64_t o = __shfl_xor_sync(0xFFFFFFFFu, v[e], lx);
        const bool keep_max = ((g & stride) == 0) == ((g & size) == 0);
        v[e] = keep_max ? (v[e] > o ? v[e] : o) : (v[e] < o ? v[e] : o);
      }
    }
    // inside a thread: registers (compile-time distances)
#pragma unroll
    for (int st = EPT / 2; st > 0; st >>= 1) {
      if (st <= (size >> 1)) {
#pragma unroll
        for (int e = 0; e < EPT; ++e) {
          if ((e & st) == 0) {
            const int g = tid * EPT + e;
            const bool desc = (g & size) == 0;
            const uint64_t a = v[e], b = v[e | st];
            const bool swap = (a < b) == desc;
            v[e] = swap ? b : a;
            v[e | st] = swap ? a : b;
          }
        }
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int e = 0; e < EPT; ++e) sbuf[tid * EPT + e] = v[e];
  __syncthreads();
}

__global__ void __launch_bounds__(RT)
topk_radix_kernel(const float* __restrict__ logits, int64_t M, int N, int64_t ld, int k, int kpad, int mode,
                  int slice, int vec_ok, float* __restrict__ scores, int64_t* __restrict__ idx64,
                  int32_t* __restrict__ idx32, int32_t* __restrict__ status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const unsigned FULL = 0xFFFFFFFFu;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned C = cluster.num_blocks();
  const unsigned crank = cluster.block_rank();
  const int64_t row = blockIdx.x / C;

  RadixCtrl* ctrl = reinterpret_cast<RadixCtrl*>(smem_raw);
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem_raw + RCTRL_BYTES);
  uint64_t* sbuf = reinterpret_cast<uint64_t*>(smem_raw + RCTRL_BYTES + 2 * RBINS * 4);
  uint64_t* lbuf = sbuf + kpad;                      // this CTA's selected entries before they go to the leader
  uint32_t* keys = reinterpret_cast<uint32_t*>(lbuf + kpad);

  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const unsigned lt_mask = (1u << lane) - 1u;
  const int begin = (int)crank * slice;
  int len = N - begin;
  if (len > slice) len = slice;
  if (len < 0) len = 0;

  if (tid == 0) { ctrl->sel_count = 0u; ctrl->blk_maxkey = 0u; ctrl->blk_sum = 0.0; ctrl->sel_bin = 0u; ctrl->k_rem = 0u; }
  for (int i = tid; i < 2 * RBINS; i += RT) hist[i] = 0u;
  if (crank == 0)
    for (int i = k + tid; i < kpad; i += RT) sbuf[i] = 0ull;

  // ---- stage the slice as keys (the only read of the logits)
  const float* p = logits + row * ld + begin;
  uint32_t lmax = 0u;
  if (vec_ok) {
    for (int i = tid * 4; i < len; i += RT * 4) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p + i));
      uint4 kk;
      kk.x = float_to_key(v.x); kk.y = float_to_key(v.y); kk.z = float_to_key(v.z); kk.w = float_to_key(v.w);
      *reinterpret_cast<uint4*>(keys + i) = kk;
      lmax = max(max(lmax, kk.x), max(kk.y, max(kk.z, kk.w)));
    }
  } else {
    for (int i = tid; i < len; i += RT) {
      const uint32_t kk = float_to_key(__ldg(p + i));
      keys[i] = kk;
      lmax = max(lmax, kk);
    }
  }
  __syncthreads();  // ctrl initialised, keys staged
  if (mode != MOE_TOPK_MODE_B) {
    lmax = __reduce_max_sync(FULL, lmax);
    if (lane == 0) atomicMax(&ctrl->blk_maxkey, lmax);
  }

  // ---- radix select: after three passes `prefix` is the key of the k-th largest value
  uint32_t prefix = 0u, pmask = 0u, k_rem = (uint32_t)k, bin = 0u;
  double rowsum = 0.0;
  uint32_t* h = hist;
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const uint32_t dmask = pass == 2 ? 1023u : 2047u;
    h = hist + (pass & 1) * RBINS;
    if (pass == 2) {  // buffer 0 again: every remote read of pass 0 ended before pass 1's cluster barrier
      for (int i = tid; i < RBINS; i += RT) h[i] = 0u;
      __syncthreads();
    }
    for (int i = tid; i < len; i += RT) {
      const uint32_t kk = keys[i];
      if ((kk & pmask) == prefix) atomicAdd(&h[(kk >> shift) & dmask], 1u);
    }
    cluster.sync();

    uint32_t g[RBPT];
#pragma unroll
    for (int j = 0; j < RBPT; ++j) g[j] = 0u;
#pragma unroll
    for (unsigned c = 0; c < 8; ++c) {   // all remote loads are issued before the first is consumed
      if (c < C) {
        const uint32_t* rh = cluster.map_shared_rank(h, c);
        const uint4 v = *reinterpret_cast<const uint4*>(rh + tid * RBPT);
        g[0] += v.x; g[1] += v.y; g[2] += v.z; g[3] += v.w;
      }
    }
    const uint32_t tsum = g[0] + g[1] + g[2] + g[3];
    uint32_t inc = tsum;  // suffix-inclusive sum over lanes >= lane
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_down_sync(FULL, inc, o);
      if (lane + o < 32) inc += n;
    }
    if (lane == 0) ctrl->warp_tot[wid] = inc;
    __syncthreads();
    uint32_t S = inc - tsum;
    for (int w = wid + 1; w < RWARPS; ++w) S += ctrl->warp_tot[w];
#pragma unroll
    for (int j = RBPT - 1; j >= 0; --j) {
      if (S < k_rem && k_rem <= S + g[j]) { ctrl->sel_bin = (uint32_t)(tid * RBPT + j); ctrl->k_rem = k_rem - S; }
      S += g[j];
    }
    __syncthreads();
    bin = ctrl->sel_bin;
    k_rem = ctrl->k_rem;
    prefix |= bin << shift;
    pmask |= dmask << shift;

    if (pass == 0 && mode != MOE_TOPK_MODE_B) {
      // full-row softmax denominator: cluster max, then this CTA's share of sum exp(v - max)
      uint32_t gmax = 0u;
      for (unsigned c = 0; c < C; ++c) gmax = max(gmax, cluster.map_shared_rank(ctrl, c)->blk_maxkey);
      const float vmax = key_to_float(gmax);
      double part = 0.0;
      for (int i = tid; i < len; i += RT) part += (double)expf(key_to_float(keys[i]) - vmax);
      part = block_sum_ordered(part, ctrl, lane, wid);
      if (tid == 0) ctrl->blk_sum = part;  // published by the next cluster barrier
    }
  }
  const uint32_t thr = prefix;        // key of the k-th largest element
  const uint32_t need_eq = k_rem;     // how many entries equal to it are taken (lowest indices first)

  // equal-to-threshold entries per CTA sit in the last histogram; CTAs hold ascending index ranges
  uint32_t eq_before = 0u;
  const uint32_t eq_local = h[bin];
  for (unsigned c = 0; c < crank; ++c) eq_before += cluster.map_shared_rank(h, c)[bin];
  uint32_t take = 0u;
  if (need_eq > eq_before) { take = need_eq - eq_before; if (take > eq_local) take = eq_local; }
  const bool take_all = (take == eq_local);
  if (mode != MOE_TOPK_MODE_B && crank == 0) {
    for (unsigned c = 0; c < C; ++c) rowsum += cluster.map_shared_rank(ctrl, c)->blk_sum;
  }

  // ---- gather the selected entries into the leading CTA: compact them locally first (shared-memory atomics are
  //      cheap, remote ones are not), reserve their place in the leader's buffer with one remote atomic, copy
  uint64_t* lead_sbuf = cluster.map_shared_rank(sbuf, 0);
  uint32_t* lead_count = cluster.map_shared_rank(&ctrl->sel_count, 0);
  if (tid == 0) ctrl->loc_count = 0u;
  __syncthreads();
  for (int base = 0; base < len; base += RT) {
    const int i = base + tid;
    const uint32_t kk = i < len ? keys[i] : 0u;
    const bool sel = i < len && (kk > thr || (take_all && kk == thr));
    const unsigned m = __ballot_sync(FULL, sel);
    if (m) {
      uint32_t b = 0u;
      if (lane == 0) b = atomicAdd(&ctrl->loc_count, (uint32_t)__popc(m));
      b = __shfl_sync(FULL, b, 0);
      if (sel) lbuf[b + __popc(m & lt_mask)] = pack_entry(kk, (uint32_t)(begin + i));
    }
  }
  if (!take_all && take > 0u) {  // block-uniform: only the first `take` equal entries, in index order
    uint32_t running = 0u;
    for (int base = 0; base < len && running < take; base += RT) {
      const int i = base + tid;
      const bool eq = i < len && keys[i] == thr;
      const unsigned m = __ballot_sync(FULL, eq);
      __syncthreads();
      if (lane == 0) ctrl->warp_tot[wid] = (uint32_t)__popc(m);
      __syncthreads();
      uint32_t before = running, total = 0u;
      for (int w = 0; w < RWARPS; ++w) {
        const uint32_t t = ctrl->warp_tot[w];
        if (w < wid) before += t;
        total += t;
      }
      const uint32_t myrank = before + (uint32_t)__popc(m & lt_mask);
      if (eq && myrank < take) {
        const uint32_t slot = atomicAdd(&ctrl->loc_count, 1u);
        lbuf[slot] = pack_entry(thr, (uint32_t)(begin + i));
      }
      running += total;
    }
  }
  __syncthreads();
  if (tid == 0) ctrl->loc_base = atomicAdd(lead_count, ctrl->loc_count);
  __syncthreads();
  {
    const uint32_t cnt = ctrl->loc_count, base0 = ctrl->loc_base;
    for (uint32_t i = tid; i < cnt; i += RT) lead_sbuf[base0 + i] = lbuf[i];
  }
  cluster.sync();
  if (crank != 0) return;  // nobody reads another CTA's shared memory past this point

  if (tid == 0 && ctrl->sel_count != (uint32_t)k && status) {
    status[0] = ST_INTERNAL; status[1] = (int32_t)ctrl->sel_count; status[2] = (int32_t)row;
  }

  // ---- bitonic sort, descending, of kpad 64-bit entries (padding entries are 0 and sink to the end):
  //      in registers + shuffles when there is at least one entry per thread, else the plain shared-memory network
  if (kpad >= RT) {   // block-uniform
    if (kpad == RT) block_sort_desc<1>(sbuf, tid);
    else if (kpad == 2 * RT) block_sort_desc<2>(sbuf, tid);
    else if (kpad == 4 * RT) block_sort_desc<4>(sbuf, tid);
    else block_sort_desc<8>(sbuf, tid);
  } else {
    for (int size = 2; size <= kpad; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int t = tid; t < (kpad >> 1); t += RT) {
          const int i = 2 * t - (t & (stride - 1));
          const int j = i + stride;
          const bool desc = (i & size) == 0;
          const uint64_t a = sbuf[i], b = sbuf[j];
          if ((a < b) == desc) { sbuf[i] = b; sbuf[j] = a; }
        }
        __syncthreads();
      }
    }
  }

  // ---- softmax over the k selected (mode B) or against the full-row denominator (modes A)
  const float vmax = key_to_float((uint32_t)(sbuf[0] >> 32));
  float denom;
  if (mode == MOE_TOPK_MODE_B) {
    double part = 0.0;
    for (int r = tid; r < k; r += RT) part += (double)expf(key_to_float((uint32_t)(sbuf[r] >> 32)) - vmax);
    denom = (float)block_sum_ordered(part, ctrl, lane, wid);
  } else {
    denom = (float)rowsum;
  }
  float renorm = 1.f;
  if (mode == MOE_TOPK_MODE_A_RENORM) {
    double part = 0.0;
    for (int r = tid; r < k; r += RT) part += (double)(expf(key_to_float((uint32_t)(sbuf[r] >> 32)) - vmax) / denom);
    renorm = (float)block_sum_ordered(part, ctrl, lane, wid);
  }
  const int64_t o = row * (int64_t)k;
  for (int r = tid; r < k; r += RT) {
    const uint64_t ent = sbuf[r];
    float s = expf(key_to_float((uint32_t)(ent >> 32)) - vmax) / denom;
    if (mode == MOE_TOPK_MODE_A_RENORM) s = s / renorm;
    const uint32_t col = 0xFFFFFFFFu - (uint32_t)(ent & 0xFFFFFFFFull);
    scores[o + r] = s;
    if (idx64) idx64[o + r] = (int64_t)col;
    if (idx32) idx32[o + r] = (int32_t)col;
  }
}

static int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

static int launch_radix(const float* logits, int64_t M, int N, int64_t ld, int k, int mode, float* scores,
                        int64_t* idx64, int32_t* idx32, int32_t* status, const DeviceInfo& dev, cudaStream_t st) {
  // cluster size: a slice must fit; beyond that split rows until the grid covers the SMs
  int C = 1;
  while (C < 8 && ((N + C - 1) / C > RMAX_SLICE || (M * C < dev.sm_count && N / (2 * C) >= 2048))) C <<= 1;
  int slice = (N + C - 1) / C;
  slice = (slice + 3) & ~3;
  if (slice > RMAX_SLICE) return fail(MOE_ERR_UNSUPPORTED, "topk_softmax: N=%d exceeds %d", N, 8 * RMAX_SLICE);
  int kpad = next_pow2(k);
  if (kpad < 2) kpad = 2;
  if (kpad > RMAX_KPAD) return fail(MOE_ERR_UNSUPPORTED, "topk_softmax: k=%d exceeds %d", k, RMAX_KPAD);
  const size_t smem = (size_t)RCTRL_BYTES + 2 * RBINS * 4 + (size_t)kpad * 16 + (size_t)slice * 4;
  const int vec_ok = (N % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  MOE_CUDA_CHECK(cudaFuncSetAttribute(topk_radix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(M * C), 1, 1);
  cfg.blockDim = dim3(RT, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MOE_CUDA_CHECK(cudaLaunchKernelEx(&cfg, topk_radix_kernel, logits, M, N, ld, k, kpad, mode, slice, vec_ok, scores,
                                    idx64, idx32, status));
  return MOE_OK;
}

}  // namespace moe

extern "C" int moe_topk_softmax(const float* logits, int64_t M, int64_t N, int64_t ld, int k, int mode, float* scores,
                                int64_t* indices, int32_t* indices32, int32_t* status, void* stream) {
  using namespace moe;
  if (!logits || !scores || (!indices && !indices32)) return fail(MOE_ERR_ARG, "topk_softmax: null pointer");
  if (M < 0 || N < 1 || k < 1 || k > N || ld < N) return fail(MOE_ERR_ARG, "topk_softmax: bad shape M=%lld N=%lld k=%d ld=%lld", (long long)M, (long long)N, k, (long long)ld);
  if (mode < 0 || mode > 2) return fail(MOE_ERR_ARG, "topk_softmax: unknown mode %d", mode);
  if (N > 8 * (int64_t)RMAX_SLICE) return fail(MOE_ERR_UNSUPPORTED, "topk_softmax: N=%lld exceeds %d", (long long)N, 8 * RMAX_SLICE);
  if (M * 8 > 0x7FFFFFFFll) return fail(MOE_ERR_UNSUPPORTED, "topk_softmax: M too large");
  if (M == 0) return MOE_OK;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int n = (int)N;
  if (n <= 1024 && k <= 8 && n >= 8 && (n % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0) &&
      M >= 2048) {
    // enough rows to give every SM a tile; below that the warp-per-row kernel has the shorter critical path
    // thread-per-row tiles: TPR threads share a row so that a tile is always <= 128 x 128 floats
    const int tpr = n <= 128 ? 1 : (n <= 256 ? 2 : (n <= 512 ? 4 : 8));
#define MOE_TILE_CASE(K_, T_) return launch_tile<K_, T_>(logits, M, n, ld, k, mode, scores, indices, indices32, dev.sm_count, st)
#define MOE_TILE_K(K_) { if (tpr == 1) MOE_TILE_CASE(K_, 1); if (tpr == 2) MOE_TILE_CASE(K_, 2); if (tpr == 4) MOE_TILE_CASE(K_, 4); MOE_TILE_CASE(K_, 8); }
    if (k <= 2) MOE_TILE_K(2)
    if (k <= 4) MOE_TILE_K(4)
    if (k <= 6) MOE_TILE_K(6)
    MOE_TILE_K(8)
#undef MOE_TILE_K
#undef MOE_TILE_CASE
  }
  if (n <= 1024 && k <= 64) {
    const bool vec = (n % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
#define MOE_WARP_CASE(E_, V_) return launch_warp<E_, V_>(logits, M, n, ld, k, mode, scores, indices, indices32, dev.sm_count, st)
    if (n <= 32) MOE_WARP_CASE(1, 1);
    if (n <= 64) MOE_WARP_CASE(2, 1);
    if (n <= 128) { if (vec) MOE_WARP_CASE(4, 4); MOE_WARP_CASE(4, 1); }
    if (n <= 256) { if (vec) MOE_WARP_CASE(8, 4); MOE_WARP_CASE(8, 1); }
    if (n <= 512) { if (vec) MOE_WARP_CASE(16, 4); MOE_WARP_CASE(16, 1); }
    if (vec) MOE_WARP_CASE(32, 4);
    MOE_WARP_CASE(32, 1);
#undef MOE_WARP_CASE
  }
  return launch_radix(logits, M, n, ld, k, mode, scores, indices, indices32, status, dev, st);
}
