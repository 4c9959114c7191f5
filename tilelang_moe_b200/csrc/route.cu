// Token permutation / histogram stage, row gather, combine and the small-E router GEMV.
// All of it is HBM- or latency-bound integer / copy work: coalesced 16-byte accesses,
// warp-private shared-memory histograms, no host round trip.
#include "common.cuh"

#include <cuda_fp16.h>
#include <mutex>

namespace moe {

// ------------------------------------------------------------------------------------
// histogram / offsets / stable permutation
//
// The flat list of n = T*k expert ids is cut into units of RUNIT consecutive entries,
// one warp per unit.  (1) every warp counts its unit into unit_counts[u][e];
// (2) one CTA turns the table into start positions: offsets[e] + entries of expert e in
// earlier units; (3) every warp walks its unit again in order and hands out positions,
// which makes the permutation the stable argsort of the ids.
// ------------------------------------------------------------------------------------
constexpr int RUNIT = 1024;        // entries per warp (large inputs)
constexpr int RUNIT_SMALL = 128;   // entries per warp when the whole input is small: more warps, shorter serial walks
constexpr int64_t RSMALL_MAX = 65536;    // up to here the three kernels cut the list into the small units (one warp each) ...
constexpr int64_t RSMALL_TABLE = 131072; // ... as long as the units x experts table the scan kernel walks stays this small
// measured inside a CUDA graph, E = 256 (us, small / large units): n = 32768 18 / 36, 65536 30 / ~45; beyond that the
// table walk of the scan kernel outweighs the extra warps (n = 262144: 90 with small units, 524288: 57 with large)
__host__ __device__ inline bool route_small_units(int64_t n, int E) {
  return n <= RSMALL_MAX && ((n + RUNIT_SMALL - 1) / RUNIT_SMALL) * (int64_t)E <= RSMALL_TABLE;
}
constexpr int64_t RSINGLE_MAX = 4096;    // up to here (half of it with many experts) one CTA does the whole stage in one launch
constexpr int RWPB = 8;            // warps per CTA in the count / scatter kernels

// Expert id of flat entry i; with an id_map (int32 [E]) the id is translated, e.g. to the
// destination-major numbering used by expert parallelism.  Out-of-range ids come back as -1.
// With kx > 0 the list is virtual: every run of kx stored ids (one token's routed experts) is followed by one entry
// that is not stored anywhere and names expert E - 1, the shared expert riding along as one more group.
__device__ __forceinline__ int load_id(const void* ids, int is64, int64_t i, const int32_t* id_map, int E, int kx = 0) {
  if (kx > 0) {
    const int64_t t = i / (kx + 1);
    const int sl = (int)(i - t * (kx + 1));
    if (sl == kx) return E - 1;
    i = t * kx + sl;
    E -= 1;                          // stored ids name the routed experts only
  }
  int e;
  if (is64) {
    const long long v = reinterpret_cast<const long long*>(ids)[i];
    e = (v < 0 || v > 0x7FFFFFFFll) ? -1 : (int)v;
  } else {
    e = reinterpret_cast<const int*>(ids)[i];
  }
  if (e < 0 || e >= E) return -1;
  return id_map ? id_map[e] : e;
}

template <int UNIT>
__global__ void __launch_bounds__(RWPB * 32)
route_count_kernel(const void* __restrict__ ids, int is64, int64_t n, int E, const int32_t* __restrict__ id_map,
                   int32_t* __restrict__ unit_counts, int32_t* __restrict__ status, int kx) {
  extern __shared__ int32_t sh[];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  int32_t* wh = sh + (size_t)w * E;
  const int64_t u = (int64_t)blockIdx.x * RWPB + w;
  const int64_t first = u * UNIT;
  if (first >= n) return;
  // all loads of the unit are issued before the first one is consumed (the walk itself is latency-bound)
  int ev[UNIT / 32];
#pragma unroll
  for (int sidx = 0; sidx < UNIT / 32; ++sidx) {
    const int64_t i = first + sidx * 32 + lane;
    ev[sidx] = i < n ? load_id(ids, is64, i, id_map, E, kx) : -2;
  }
  for (int e = lane; e < E; e += 32) wh[e] = 0;
  __syncwarp();
  bool bad = false;
#pragma unroll
  for (int sidx = 0; sidx < UNIT / 32; ++sidx) {
    const int e = ev[sidx];
    if (e >= 0) atomicAdd(&wh[e], 1);
    else if (e == -1) bad = true;
  }
  if (bad && status) status[0] = ST_BAD_EXPERT_ID;
  __syncwarp();
  for (int e = lane; e < E; e += 32) unit_counts[u * E + e] = wh[e];
}

__global__ void __launch_bounds__(1024)
route_scan_kernel(int32_t* __restrict__ unit_counts, int64_t n_units, int E, int32_t* __restrict__ counts,
                  int32_t* __restrict__ offsets) {
  __shared__ int32_t warp_tot[32];
  __shared__ int32_t carry_s;
  __shared__ int32_t part[1024];     // [P][Ec]: entries of expert e in the p-th share of the units
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  // Up to 1024 experts at a time, consecutive lanes on consecutive experts (coalesced rows of the table); with fewer
  // experts than threads, P threads share an expert's column, each walking a contiguous share of the units
  const int Ec = E >= 1024 ? 1024 : ((E + 31) & ~31);
  const int P = 1024 / Ec;
  const int p = tid / Ec, el = tid - p * Ec;
  const int64_t u_lo = n_units * p / P, u_hi = n_units * (p + 1) / P;
  for (int base = 0; base < E; base += 1024) {
    const int e = base + el;
    int32_t mine = 0;
    if (e < E && p < P)
      for (int64_t u = u_lo; u < u_hi; ++u) mine += unit_counts[u * E + e];
    if (p < P) part[p * Ec + el] = mine;
    __syncthreads();
    int32_t total = 0, ahead = 0;        // whole column; entries in the shares before this thread's
    if (p < P)
      for (int q = 0; q < P; ++q) {
        const int32_t v = part[q * Ec + el];
        total += v;
        if (q < p) ahead += v;
      }
    // exclusive scan of the column totals over this chunk of experts: threads 0 .. Ec-1 carry them, the rest zero
    const int32_t mine_tot = p == 0 ? total : 0;
    int32_t inc = mine_tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += v;
    }
    if (lane == 31) warp_tot[wid] = inc;
    __syncthreads();
    int32_t before = carry_s;
    for (int w2 = 0; w2 < wid; ++w2) before += warp_tot[w2];
    const int32_t start = before + inc - mine_tot;
    if (p == 0) part[el] = start;        // row 0 is free again: every thread has read what it needed
    if (p == 0 && e < E) { counts[e] = total; offsets[e] = start; }
    __syncthreads();
    if (e < E && p < P) {
      int32_t run = part[el] + ahead;
      for (int64_t u = u_lo; u < u_hi; ++u) {
        const int32_t c = unit_counts[u * E + e];
        unit_counts[u * E + e] = run;
        run += c;
      }
    }
    if (tid == 1023) carry_s = before + inc;
    __syncthreads();
  }
  if (tid == 0) offsets[E] = carry_s;
}

template <int UNIT>
__global__ void __launch_bounds__(RWPB * 32)
route_scatter_kernel(const void* __restrict__ ids, int is64, int64_t n, int E, const int32_t* __restrict__ id_map,
                     const int32_t* __restrict__ unit_base, int32_t* __restrict__ perm, int32_t* __restrict__ inv, int kx) {
  extern __shared__ int32_t sh[];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const unsigned lt_mask = (1u << lane) - 1u;
  int32_t* wh = sh + (size_t)w * E;
  const int64_t u = (int64_t)blockIdx.x * RWPB + w;
  const int64_t first = u * UNIT;
  if (first >= n) return;
  int ev[UNIT / 32];
#pragma unroll
  for (int sidx = 0; sidx < UNIT / 32; ++sidx) {
    const int64_t i = first + sidx * 32 + lane;
    ev[sidx] = i < n ? load_id(ids, is64, i, id_map, E, kx) : -2;
  }
  for (int e = lane; e < E; e += 32) wh[e] = unit_base[u * E + e];
  __syncwarp();
#pragma unroll
  for (int sidx = 0; sidx < UNIT / 32; ++sidx) {
    const int64_t i = first + sidx * 32 + lane;
    const int e = ev[sidx];
    const bool valid = e >= 0;
    // lanes without a valid id get a private group so that they match nobody
    const unsigned grp = __match_any_sync(0xFFFFFFFFu, valid ? (unsigned)e : (0x80000000u | (unsigned)lane));
    const int r = __popc(grp & lt_mask);
    int32_t base = 0;
    if (valid) base = wh[e];
    __syncwarp();
    if (valid && r == 0) wh[e] = base + __popc(grp);
    __syncwarp();
    if (valid) {
      const int32_t pos = base + r;
      if (perm) perm[pos] = (int32_t)i;
      if (inv) inv[i] = pos;
    }
  }
}

// Small inputs (n <= RSINGLE_MAX): the whole stage in one CTA and one launch.  Counts by shared-memory atomics, an
// exclusive scan over the experts, then the stable permutation in rounds of 1024 consecutive entries: inside a
// round an entry's place is its expert's running start + the entries of that expert in earlier warps of the round
// (one count per warp and expert, written by the first lane of each match group) + its rank among equal ids of
// its own warp.  Same results as the three-kernel path, two launches fewer on the latency-bound small layers.
__global__ void __launch_bounds__(1024)
route_small_kernel(const void* __restrict__ ids, int is64, int n, int E, const int32_t* __restrict__ id_map,
                   int32_t* __restrict__ counts, int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                   int32_t* __restrict__ inv, int32_t* __restrict__ status, int kx) {
  extern __shared__ int32_t sh[];
  int32_t* base = sh;                 // [E]   counts, then the running start of every expert
  int32_t* wcnt = sh + E;             // [32][E]
  __shared__ int32_t warp_tot[32];
  __shared__ int32_t carry_s;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const unsigned lt_mask = (1u << lane) - 1u;
  for (int i = tid; i < 33 * E; i += 1024) sh[i] = 0;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  // a thread owns entries tid, tid + 1024, ...: at most RSINGLE_MAX / 1024 of them, kept in registers for the
  // permutation rounds below (the loads are independent, so they are all in flight together)
  constexpr int ROUNDS = RSINGLE_MAX / 1024;
  int32_t ereg[ROUNDS];
  bool bad = false;
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    const int i = r * 1024 + tid;
    ereg[r] = i < n ? load_id(ids, is64, i, id_map, E, kx) : -1;
    if (i < n && ereg[r] < 0) bad = true;
  }
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r)
    if (ereg[r] >= 0) atomicAdd(&base[ereg[r]], 1);
  if (bad && status) status[0] = ST_BAD_EXPERT_ID;
  __syncthreads();
  for (int b0 = 0; b0 < E; b0 += 1024) {          // exclusive scan, 1024 experts at a time
    const int e = b0 + tid;
    const int32_t total = e < E ? base[e] : 0;
    int32_t inc = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
      if (lane >= o) inc += v;
    }
    if (lane == 31) warp_tot[w] = inc;
    __syncthreads();
    int32_t before = carry_s;
    for (int w2 = 0; w2 < w; ++w2) before += warp_tot[w2];
    const int32_t start = before + inc - total;
    if (e < E) { counts[e] = total; offsets[e] = start; base[e] = start; }
    __syncthreads();
    if (tid == 1023) carry_s = before + inc;
    __syncthreads();
  }
  if (tid == 0) offsets[E] = carry_s;
  if (!perm && !inv) return;
#pragma unroll
  for (int r = 0; r < ROUNDS; ++r) {
    if (r * 1024 >= n) break;
    const int i = r * 1024 + tid;
    const int e = ereg[r];
    const bool valid = e >= 0;
    const unsigned grp = __match_any_sync(0xFFFFFFFFu, valid ? (unsigned)e : (0x80000000u | (unsigned)lane));
    const int rank = __popc(grp & lt_mask);
    if (valid && rank == 0) wcnt[w * E + e] = __popc(grp);
    __syncthreads();
    if (valid) {
      int32_t pos = base[e] + rank;
      for (int w2 = 0; w2 < w; ++w2) pos += wcnt[w2 * E + e];
      if (perm) perm[pos] = i;
      if (inv) inv[i] = pos;
    }
    __syncthreads();
    if (valid && rank == 0) { atomicAdd(&base[e], __popc(grp)); wcnt[w * E + e] = 0; }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------
// row gather: dst[p,:] = src[perm[p] / div, :]
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ perm, int div, int64_t n_rows,
                   int vec_per_row, uint4* __restrict__ dst, const float* __restrict__ w_src,
                   float* __restrict__ w_dst) {
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  for (int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); p < n_rows; p += nwarps) {
    const int32_t f = perm ? perm[p] : (int32_t)p;
    const int64_t srow = div > 1 ? f / div : f;
    const uint4* s = src + srow * vec_per_row;
    uint4* d = dst + p * vec_per_row;
    // four independent 16-byte loads in flight per lane before the first store
    int v = lane;
    for (; v + 96 < vec_per_row; v += 128) {
      const uint4 a = __ldg(s + v), b = __ldg(s + v + 32), c = __ldg(s + v + 64), e = __ldg(s + v + 96);
      d[v] = a; d[v + 32] = b; d[v + 64] = c; d[v + 96] = e;
    }
    for (; v < vec_per_row; v += 32) d[v] = __ldg(s + v);
    if (w_src && lane == 0) w_dst[p] = w_src[f];
  }
}

// ------------------------------------------------------------------------------------
// combine: out[t,:] = shared[t,:] + sum_s Yk[t*k+s,:]   (fp32 sum in slot order, one rounding)
// ------------------------------------------------------------------------------------
// element-pair conversions for the two 16-bit types (F16 = false: bfloat16, true: half)
template <bool F16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if (F16) return __half22float2(*reinterpret_cast<const __half2*>(&u));
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
}
template <bool F16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if (F16) { __half2 h = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&h); }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <bool F16>
__device__ __forceinline__ void add_x8(float* acc, const uint4& v) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack2<F16>(u[j]);
    acc[2 * j] += f.x;
    acc[2 * j + 1] += f.y;
  }
}

template <bool F16>
__device__ __forceinline__ void fma_x8(float* acc, const uint4& v, float w) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack2<F16>(u[j]);
    acc[2 * j] = fmaf(f.x, w, acc[2 * j]);
    acc[2 * j + 1] = fmaf(f.y, w, acc[2 * j + 1]);
  }
}

template <bool F16>
__global__ void __launch_bounds__(256)
combine_kernel(const uint4* __restrict__ Yk, const uint4* __restrict__ shared, const int32_t* __restrict__ row_of,
               const float* __restrict__ scale, int64_t T, int k, int vec_per_row, uint4* __restrict__ out) {
  const int64_t total = T * vec_per_row;
  for (int64_t g = (int64_t)blockIdx.x * 256 + threadIdx.x; g < total; g += (int64_t)gridDim.x * 256) {
    const int64_t t = g / vec_per_row;
    const int v = (int)(g - t * vec_per_row);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // four slots at a time: the loads of a group are all in flight before the first is added; the additions
    // stay in slot order, so the sum is the same as one slot at a time
    for (int s0 = 0; s0 < k; s0 += 4) {
      uint4 y[4];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u < k) {
          const int64_t f = t * k + s0 + u;
          const int64_t r = row_of ? (int64_t)row_of[f] : f;
          if (!row_of || MOE_INDEX_OK(r, T * k, 3)) y[u] = __ldg(Yk + r * vec_per_row + v);
          else y[u] = make_uint4(0u, 0u, 0u, 0u);            // checked build: a row outside Yk contributes nothing
          w[u] = scale ? scale[f] : 1.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s0 + u < k) {
          if (scale) fma_x8<F16>(acc, y[u], w[u]); else add_x8<F16>(acc, y[u]);
        }
      }
    }
    if (shared) add_x8<F16>(acc, __ldg(shared + g));
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) ou[j] = pack2<F16>(acc[2 * j], acc[2 * j + 1]);
    out[g] = o;
  }
}

// ------------------------------------------------------------------------------------
// router logits for a small expert count: the router weight [E,H] is staged once per CTA in shared memory,
// then each warp takes tokens in turn: one pass over the token row, all E dot products in registers
// ------------------------------------------------------------------------------------
template <bool F16, int EMAX>
__global__ void __launch_bounds__(256)
router_logits_kernel(const uint4* __restrict__ x, const uint4* __restrict__ Wr, int64_t T, int vec_per_row, int E,
                     float* __restrict__ logits, int k, int mode, float* __restrict__ scores,
                     int64_t* __restrict__ idx64, int32_t* __restrict__ idx32) {
  extern __shared__ uint4 wsh[];   // [E][vec_per_row]
  const int lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < E * vec_per_row; i += 256) wsh[i] = __ldg(Wr + i);
  __syncthreads();
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  for (int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); t < T; t += nwarps) {
    const uint4* xr = x + t * vec_per_row;
    float acc[EMAX];
#pragma unroll
    for (int j = 0; j < EMAX; ++j) acc[j] = 0.f;
    // the row is fetched eight vectors per lane at a time, all eight loads in flight before the first is used: a
    // 4 KB row costs one memory round trip instead of eight in a row
    for (int v0 = lane; v0 < vec_per_row; v0 += 256) {
      uint4 xq[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int v = v0 + 32 * u;
        xq[u] = v < vec_per_row ? __ldg(xr + v) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int v = v0 + 32 * u;
        if (v < vec_per_row) {
          const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xq[u]);
          float xf[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = unpack2<F16>(xu[j]);
            xf[2 * j] = f.x; xf[2 * j + 1] = f.y;
          }
#pragma unroll
          for (int j = 0; j < EMAX; ++j) {
            if (j < E) {
              const uint4 wv = wsh[j * vec_per_row + v];
              const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 f = unpack2<F16>(wu[q]);
                acc[j] = fmaf(xf[2 * q], f.x, acc[j]);
                acc[j] = fmaf(xf[2 * q + 1], f.y, acc[j]);
              }
            }
          }
        }
      }
    }
    float mine = 0.f;                                  // lane j ends up with the logit of expert j
#pragma unroll
    for (int j = 0; j < EMAX; ++j) {
      const float sum = warp_sum(acc[j]);
      if (lane == j) mine = sum;
    }
    if (logits && lane < E) logits[t * E + lane] = mine;
    if (k > 0) {
      // fused top-k + softmax over the E <= 32 logits held one per lane: k rounds of warp arg-max, lowest
      // lane first among equals; lane r keeps the r-th winner
      const unsigned FULL = 0xFFFFFFFFu;
      int key = lane < E ? float_to_ikey(mine) : (int)0x80000000;
      int win_key = (int)0x80000000, win_idx = 0;
      for (int r = 0; r < k; ++r) {
        const int m = __reduce_max_sync(FULL, key);
        const int sel = __ffs(__ballot_sync(FULL, key == m)) - 1;
        if (lane == r) { win_key = m; win_idx = sel; }
        if (lane == sel) key = (int)0x80000000;
      }
      const float vmax = ikey_to_float(__shfl_sync(FULL, win_key, 0));
      const float e = lane < k ? expf(ikey_to_float(win_key) - vmax) : 0.f;
      const float denom = mode == MOE_TOPK_MODE_B ? warp_sum(e) : warp_sum(lane < E ? expf(mine - vmax) : 0.f);
      float sc = e / denom;
      if (mode == MOE_TOPK_MODE_A_RENORM) sc = sc / warp_sum(sc);
      if (lane < k) {
        scores[t * k + lane] = sc;
        if (idx64) idx64[t * k + lane] = (int64_t)win_idx;
        if (idx32) idx32[t * k + lane] = (int32_t)win_idx;
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// expert-parallel regroup table
//
// After the dispatch all-to-all a rank holds rows in source-major order: for each source
// rank s, for each local expert j, cnt[s][j] rows.  The expert GEMM wants them expert-major.
// This kernel turns cnt (int32 [G][El]) into offsets[El+1] (expert-major exclusive prefix) and
// src_row[p] = source-major row held at expert-major position p.  src_row serves both as the
// gather list before the up GEMM and as the scatter list of the down GEMM's epilogue.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
ep_regroup_kernel(const int32_t* __restrict__ cnt, int G, int El, int32_t* __restrict__ offsets,
                  int32_t* __restrict__ src_row) {
  extern __shared__ int32_t sh[];
  int32_t* in_start = sh;               // [G*El] source-major exclusive prefix
  int32_t* out_start = sh + G * El;     // [G*El] expert-major start of segment (s, j), stored at [s*El + j]
  __shared__ int32_t part[1024];
  const int tid = threadIdx.x;
  const int n = G * El;
  const int per = (n + 1023) / 1024;

  // pass 1: source-major exclusive scan
  {
    const int lo = tid * per, hi = min(n, lo + per);
    int32_t sum = 0;
    for (int q = lo; q < hi; ++q) sum += cnt[q];
    part[tid] = sum;
    __syncthreads();
    if (tid < 32) {  // one warp scans the 1024 partial sums, 32 per lane
      int32_t loc = 0;
      for (int i = 0; i < 32; ++i) loc += part[tid * 32 + i];
      int32_t inc = loc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (tid >= o) inc += v;
      }
      int32_t run = inc - loc;
      for (int i = 0; i < 32; ++i) { const int32_t v = part[tid * 32 + i]; part[tid * 32 + i] = run; run += v; }
    }
    __syncthreads();
    int32_t run = part[tid];
    for (int q = lo; q < hi; ++q) { in_start[q] = run; run += cnt[q]; }
    __syncthreads();
  }
  // pass 2: expert-major order = flattened index q' = j*G + s
  {
    const int lo = tid * per, hi = min(n, lo + per);
    int32_t sum = 0;
    for (int q = lo; q < hi; ++q) { const int j = q / G, s = q - j * G; sum += cnt[s * El + j]; }
    part[tid] = sum;
    __syncthreads();
    if (tid < 32) {
      int32_t loc = 0;
      for (int i = 0; i < 32; ++i) loc += part[tid * 32 + i];
      int32_t inc = loc;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (tid >= o) inc += v;
      }
      int32_t run = inc - loc;
      for (int i = 0; i < 32; ++i) { const int32_t v = part[tid * 32 + i]; part[tid * 32 + i] = run; run += v; }
      if (tid == 31) offsets[El] = inc;
    }
    __syncthreads();
    int32_t run = part[tid];
    for (int q = lo; q < hi; ++q) {
      const int j = q / G, s = q - j * G;
      out_start[s * El + j] = run;
      if (s == 0) offsets[j] = run;
      run += cnt[s * El + j];
    }
    __syncthreads();
  }
  // fill: one warp per segment
  const int lane = tid & 31;
  for (int q = tid >> 5; q < n; q += 32) {
    const int32_t c = cnt[q], a = in_start[q], b = out_start[q];
    for (int i = lane; i < c; i += 32) src_row[b + i] = a + i;
  }
}

}  // namespace moe

// ====================================================================================
extern "C" size_t moe_route_histogram_workspace(int64_t n, int E) {
  if (n <= 0 || E <= 0) return 0;
  const int64_t units = moe::ceil_div64(n, moe::route_small_units(n, E) ? moe::RUNIT_SMALL : moe::RUNIT);
  return (size_t)units * (size_t)E * sizeof(int32_t);
}

extern "C" int moe_route_histogram(const void* topk_idx, int idx_is_int64, int64_t n, int E, const int32_t* id_map,
                                   int32_t* counts, int32_t* offsets, int32_t* perm, int32_t* inv, void* ws,
                                   size_t ws_bytes, int32_t* status, void* stream) {
  return moe::route_histogram_ex(topk_idx, idx_is_int64, n, E, id_map, counts, offsets, perm, inv, ws, ws_bytes, status,
                                 stream, 0);
}

// kx > 0: n counts a virtual list in which every kx stored ids are followed by one entry of expert E - 1 (declared in
// common.cuh; used by the single-call layer to run the shared expert as one more group of the routed GEMMs)
int moe::route_histogram_ex(const void* topk_idx, int idx_is_int64, int64_t n, int E, const int32_t* id_map,
                            int32_t* counts, int32_t* offsets, int32_t* perm, int32_t* inv, void* ws, size_t ws_bytes,
                            int32_t* status, void* stream, int kx) {
  using namespace moe;
  if (n < 0 || E < 1) return fail(MOE_ERR_ARG, "route_histogram: bad size n=%lld E=%d", (long long)n, E);
  if (!counts || !offsets) return fail(MOE_ERR_ARG, "route_histogram: null counts/offsets");
  if (n > 0 && !topk_idx) return fail(MOE_ERR_ARG, "route_histogram: null ids");
  if (n > 0x7FFFFFFFll) return fail(MOE_ERR_UNSUPPORTED, "route_histogram: n exceeds int32 positions");
  if ((size_t)RWPB * E * 4 > 160 * 1024) return fail(MOE_ERR_UNSUPPORTED, "route_histogram: E=%d too large", E);
  const size_t need = moe_route_histogram_workspace(n, E);
  if (need > 0 && (!ws || ws_bytes < need)) return fail(MOE_ERR_WORKSPACE, "route_histogram: workspace %zu < %zu", ws_bytes, need);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool small = route_small_units(n, E);
  // MOE_B200_ROUTE_SINGLE_MAX moves the size up to which one CTA does the whole stage (for measurements; at most RSMALL_MAX)
  static const int64_t single_max = [] {
    const char* v = getenv("MOE_B200_ROUTE_SINGLE_MAX");
    const int64_t m = v ? atoll(v) : RSINGLE_MAX;
    return m < RSINGLE_MAX ? m : RSINGLE_MAX;
  }();
  // measured inside a CUDA graph (us, one CTA / three kernels): E = 256: n = 2048 8.9 / 7.0, 4096 14.2 / 8.4, 16384
  // 45.6 / 13.6; E = 9: 3072 7.4 / 7.3, 4096 8.7 / 7.8, 16384 23.9 / 14.2.  One launch instead of three is worth
  // a few microseconds of host time outside a graph, so the single CTA keeps the smallest inputs only.
  const bool single = n <= single_max && (n <= RSINGLE_MAX / 2 || E <= 64);
  if (single && n > 0 && E <= 1024) {   // one CTA, one launch
    const size_t smem1 = (size_t)33 * E * 4;
    if (smem1 > 48 * 1024)
      MOE_CUDA_CHECK(cudaFuncSetAttribute(route_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1));
    route_small_kernel<<<1, 1024, smem1, st>>>(topk_idx, idx_is_int64, (int)n, E, id_map, counts, offsets, perm, inv, status, kx);
    MOE_CHECK_LAUNCH("route_small_kernel");
    return MOE_OK;
  }
  const int64_t units = ceil_div64(n, small ? RUNIT_SMALL : RUNIT);
  const size_t smem = (size_t)RWPB * E * 4;
  int32_t* unit_counts = reinterpret_cast<int32_t*>(ws);
  if (smem > 48 * 1024) {
    MOE_CUDA_CHECK(cudaFuncSetAttribute(route_count_kernel<RUNIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MOE_CUDA_CHECK(cudaFuncSetAttribute(route_scatter_kernel<RUNIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MOE_CUDA_CHECK(cudaFuncSetAttribute(route_count_kernel<RUNIT_SMALL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MOE_CUDA_CHECK(cudaFuncSetAttribute(route_scatter_kernel<RUNIT_SMALL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const unsigned blocks = (unsigned)ceil_div64(units, RWPB);
  if (units > 0) {
    if (small) route_count_kernel<RUNIT_SMALL><<<blocks, RWPB * 32, smem, st>>>(topk_idx, idx_is_int64, n, E, id_map, unit_counts, status, kx);
    else route_count_kernel<RUNIT><<<blocks, RWPB * 32, smem, st>>>(topk_idx, idx_is_int64, n, E, id_map, unit_counts, status, kx);
    MOE_CHECK_LAUNCH("route_count_kernel");
  }
  route_scan_kernel<<<1, 1024, 0, st>>>(unit_counts, units, E, counts, offsets);
  MOE_CHECK_LAUNCH("route_scan_kernel");
  if (units > 0 && (perm || inv)) {
    if (small) route_scatter_kernel<RUNIT_SMALL><<<blocks, RWPB * 32, smem, st>>>(topk_idx, idx_is_int64, n, E, id_map, unit_counts, perm, inv, kx);
    else route_scatter_kernel<RUNIT><<<blocks, RWPB * 32, smem, st>>>(topk_idx, idx_is_int64, n, E, id_map, unit_counts, perm, inv, kx);
    MOE_CHECK_LAUNCH("route_scatter_kernel");
  }
  return MOE_OK;
}

extern "C" int moe_gather_rows(const void* src, const int32_t* perm, int div, int64_t n_rows, int64_t cols, void* dst,
                               const float* w_src, float* w_dst, void* stream) {
  using namespace moe;
  if (n_rows < 0 || cols < 8 || cols % 8) return fail(MOE_ERR_ARG, "gather_rows: cols=%lld must be a positive multiple of 8", (long long)cols);
  if (n_rows == 0) return MOE_OK;
  if (!src || !dst) return fail(MOE_ERR_ARG, "gather_rows: null pointer");
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) return fail(MOE_ERR_ARG, "gather_rows: pointers must be 16-byte aligned");
  if (w_src && !w_dst) return fail(MOE_ERR_ARG, "gather_rows: w_src without w_dst");
  if (div < 1) div = 1;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  int64_t blocks = ceil_div64(n_rows, 8);
  const int64_t cap = (int64_t)dev.sm_count * 8;   // 64 warps per SM, each with four row pieces in flight
  if (blocks > cap) blocks = cap;
  gather_rows_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(src), perm, div, n_rows, (int)(cols / 8), reinterpret_cast<uint4*>(dst), w_src, w_dst);
  MOE_CHECK_LAUNCH("gather_rows_kernel");
  return MOE_OK;
}

extern "C" int moe_combine(const void* Yk, const void* shared, const int32_t* row_of, const float* scale, int64_t T,
                           int k, int64_t H, int dtype, void* out, void* stream) {
  using namespace moe;
  if (dtype != MOE_DTYPE_BF16 && dtype != MOE_DTYPE_F16) return fail(MOE_ERR_ARG, "combine: unknown dtype %d", dtype);
  if (T < 0 || k < 0 || H < 8 || H % 8) return fail(MOE_ERR_ARG, "combine: bad shape T=%lld k=%d H=%lld", (long long)T, k, (long long)H);
  if (T == 0) return MOE_OK;
  if ((k > 0 && !Yk) || !out) return fail(MOE_ERR_ARG, "combine: null pointer");
  if ((reinterpret_cast<uintptr_t>(Yk) | reinterpret_cast<uintptr_t>(shared) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(MOE_ERR_ARG, "combine: pointers must be 16-byte aligned");
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  const int64_t total = T * (H / 8);
  int64_t blocks = ceil_div64(total, 256);
  const int64_t cap = (int64_t)dev.sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (dtype == MOE_DTYPE_F16)
    combine_kernel<true><<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4*>(Yk), reinterpret_cast<const uint4*>(shared), row_of, scale, T, k, (int)(H / 8),
        reinterpret_cast<uint4*>(out));
  else
    combine_kernel<false><<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4*>(Yk), reinterpret_cast<const uint4*>(shared), row_of, scale, T, k, (int)(H / 8),
        reinterpret_cast<uint4*>(out));
  MOE_CHECK_LAUNCH("combine_kernel");
  return MOE_OK;
}

// E <= 32 experts whose weight fits shared memory: CUDA cores, one warp per token; k == 0: logits only
static int router_small(const void* x, const void* Wr, int64_t T, int H, int E, int dtype, float* logits, int k, int mode,
                        float* scores, int64_t* idx64, int32_t* idx32, void* stream) {
  using namespace moe;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  // one CTA per SM at most: every CTA stages the whole router weight
  const size_t smem = (size_t)E * H * 2;
  int64_t blocks = ceil_div64(T, 8);      // a token per warp while the SMs last
  if (blocks > dev.sm_count) blocks = dev.sm_count;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define MOE_RL_LAUNCH(F16_, EMAX_)                                                                                       \
  do {                                                                                                                   \
    if (smem > 48 * 1024)                                                                                                \
      MOE_CUDA_CHECK(cudaFuncSetAttribute(router_logits_kernel<F16_, EMAX_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    router_logits_kernel<F16_, EMAX_><<<(unsigned)blocks, 256, smem, st>>>(                                              \
        reinterpret_cast<const uint4*>(x), reinterpret_cast<const uint4*>(Wr), T, H / 8, E, logits, k, mode, scores,     \
        idx64, idx32);                                                                                                   \
  } while (0)
  if (dtype == MOE_DTYPE_F16) { if (E <= 8) MOE_RL_LAUNCH(true, 8); else if (E <= 16) MOE_RL_LAUNCH(true, 16); else MOE_RL_LAUNCH(true, 32); }
  else { if (E <= 8) MOE_RL_LAUNCH(false, 8); else if (E <= 16) MOE_RL_LAUNCH(false, 16); else MOE_RL_LAUNCH(false, 32); }
#undef MOE_RL_LAUNCH
  MOE_CHECK_LAUNCH("router_logits_kernel");
  return MOE_OK;
}

static bool router_small_fits(int H, int E) { return E <= 32 && (size_t)E * H * 2 <= 200 * 1024; }

extern "C" int moe_router_logits(const void* x, const void* Wr, int64_t T, int H, int E, int dtype, float* logits,
                                 int32_t* status, void* stream) {
  using namespace moe;
  (void)status;
  if (dtype != MOE_DTYPE_BF16 && dtype != MOE_DTYPE_F16) return fail(MOE_ERR_ARG, "router_logits: unknown dtype %d", dtype);
  if (T < 0 || H < 8 || H % 8 || E < 1) return fail(MOE_ERR_ARG, "router_logits: bad shape T=%lld H=%d E=%d", (long long)T, H, E);
  if (T == 0) return MOE_OK;
  if (!x || !Wr || !logits) return fail(MOE_ERR_ARG, "router_logits: null pointer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(Wr)) & 15) return fail(MOE_ERR_ARG, "router_logits: pointers must be 16-byte aligned");
  if (E > 32) return fail(MOE_ERR_UNSUPPORTED, "router_logits: E=%d > 32 goes through moe_grouped_gemm (MOE_GEMM_PLAIN_F32)", E);
  if (!router_small_fits(H, E)) return fail(MOE_ERR_UNSUPPORTED, "router_logits: E*H=%lld does not fit shared memory", (long long)E * H);
  return router_small(x, Wr, T, H, E, dtype, logits, 0, 0, nullptr, nullptr, nullptr, stream);
}

extern "C" int moe_router_topk(const void* x, const void* Wr, int64_t T, int H, int E, int k, int mode, int dtype,
                               float* scores, int64_t* indices, int32_t* indices32, float* logits_out, int32_t* status,
                               void* stream) {
  using namespace moe;
  if (dtype != MOE_DTYPE_BF16 && dtype != MOE_DTYPE_F16) return fail(MOE_ERR_ARG, "router_topk: unknown dtype %d", dtype);
  if (T < 0 || H < 8 || H % 8 || E < 1 || k < 1 || k > E)
    return fail(MOE_ERR_ARG, "router_topk: bad shape T=%lld H=%d E=%d k=%d", (long long)T, H, E, k);
  if (mode < 0 || mode > 2) return fail(MOE_ERR_ARG, "router_topk: unknown mode %d", mode);
  if (T == 0) return MOE_OK;
  if (!x || !Wr || !scores || (!indices && !indices32)) return fail(MOE_ERR_ARG, "router_topk: null pointer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(Wr) | reinterpret_cast<uintptr_t>(logits_out)) & 15)
    return fail(MOE_ERR_ARG, "router_topk: x, Wr and logits_out must be 16-byte aligned");
  if (router_small_fits(H, E))
    return router_small(x, Wr, T, H, E, dtype, logits_out, k, mode, scores, indices, indices32, stream);
  if (E % 8 || E < 8 || E > 256 || k > 8)
    return fail(MOE_ERR_UNSUPPORTED, "router_topk: fused kernels take E <= 32 (small H), or E %% 8 == 0, E <= 256, k <= 8 "
                "(E=%d k=%d): use moe_router_logits / moe_grouped_gemm + moe_topk_softmax", E, k);
  return router_topk_gemm(x, Wr, T, H, E, k, mode, dtype, scores, indices, indices32, logits_out, status, stream);
}

// ------------------------------------------------------------------------------------
// Router for few tokens: the GEMM x . Wr^T has only ceil(T/128) row tiles, so it is split along K to give every
// SM a tile (fp32 slices [T, S, E]); this kernel adds the slices of a token (fixed order) and selects the top k
// with softmax.  One warp per token, column c of the row in lane c % 32; each round takes the warp maximum by redux
// and, among equal values, the lowest column.  E <= 256, k <= 32.
// ------------------------------------------------------------------------------------
namespace moe {
__global__ void __launch_bounds__(256)
router_reduce_topk_kernel(const float* __restrict__ part, int S, int64_t T, int E, int k, int mode,
                          float* __restrict__ scores, int64_t* __restrict__ idx64, int32_t* __restrict__ idx32,
                          float* __restrict__ logits_out) {
  const unsigned FULL = 0xFFFFFFFFu;
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  for (int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); t < T; t += nwarps) {
    const float* pp = part + t * (int64_t)S * E;
    float v[8];
    int key[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = lane + 32 * j;
      float a = 0.f;
      if (c < E)
        for (int s = 0; s < S; ++s) a += pp[s * E + c];
      v[j] = a;
      key[j] = c < E ? float_to_ikey(a) : (int)0x80000000;
      if (logits_out && c < E) logits_out[t * E + c] = a;
    }
    int win_key = (int)0x80000000, win_col = 0;
    for (int r = 0; r < k; ++r) {
      int lm = key[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = max(lm, key[j]);
      const int m = __reduce_max_sync(FULL, lm);
      int lc = 0x7FFFFFFF;                       // lowest column of this lane that holds the maximum
#pragma unroll
      for (int j = 7; j >= 0; --j) lc = key[j] == m ? lane + 32 * j : lc;
      const int c = __reduce_min_sync(FULL, lc);
      if (lane == r) { win_key = m; win_col = c; }
      if ((c & 31) == lane) {
#pragma unroll
        for (int j = 0; j < 8; ++j) key[j] = (c >> 5) == j ? (int)0x80000000 : key[j];
      }
    }
    const float vmax = ikey_to_float(__shfl_sync(FULL, win_key, 0));
    const float e = lane < k ? expf(ikey_to_float(win_key) - vmax) : 0.f;
    float denom;
    if (mode == MOE_TOPK_MODE_B) {
      denom = warp_sum(e);
    } else {
      float a = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (lane + 32 * j < E) a += expf(v[j] - vmax);
      denom = warp_sum(a);
    }
    float sc = e / denom;
    if (mode == MOE_TOPK_MODE_A_RENORM) sc = sc / warp_sum(sc);
    if (lane < k) {
      scores[t * k + lane] = sc;
      if (idx64) idx64[t * k + lane] = (int64_t)win_col;
      if (idx32) idx32[t * k + lane] = (int32_t)win_col;
    }
  }
}

int router_splits(int64_t T, int H) {
  const int64_t row_tiles = (T + 127) / 128;
  int S = 1;
  while (S < 16 && row_tiles * S * 2 <= 148 && H % (64 * (S * 2)) == 0 && H / (S * 2) >= 256) S *= 2;
  return S;
}
}  // namespace moe

extern "C" size_t moe_router_topk_splitk_workspace(int64_t T, int H, int E) {
  if (T < 1 || H < 8 || E < 1) return 0;
  return (size_t)T * moe::router_splits(T, H) * E * sizeof(float);
}

extern "C" int moe_router_topk_splitk(const void* x, const void* Wr, int64_t T, int H, int E, int k, int mode, int dtype,
                                      float* scores, int64_t* indices, int32_t* indices32, float* logits_out, void* ws,
                                      size_t ws_bytes, int32_t* status, void* stream) {
  using namespace moe;
  if (dtype != MOE_DTYPE_BF16 && dtype != MOE_DTYPE_F16) return fail(MOE_ERR_ARG, "router_topk_splitk: unknown dtype %d", dtype);
  if (T < 0 || H < 8 || H % 8 || E < 8 || E % 8 || k < 1 || k > E)
    return fail(MOE_ERR_ARG, "router_topk_splitk: bad shape T=%lld H=%d E=%d k=%d", (long long)T, H, E, k);
  if (E > 256 || k > 32) return fail(MOE_ERR_UNSUPPORTED, "router_topk_splitk: E <= 256 and k <= 32 (E=%d k=%d)", E, k);
  if (mode < 0 || mode > 2) return fail(MOE_ERR_ARG, "router_topk_splitk: unknown mode %d", mode);
  if (T == 0) return MOE_OK;
  if (!x || !Wr || !scores || (!indices && !indices32) || !ws) return fail(MOE_ERR_ARG, "router_topk_splitk: null pointer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(Wr) | reinterpret_cast<uintptr_t>(ws)) & 15)
    return fail(MOE_ERR_ARG, "router_topk_splitk: x, Wr and ws must be 16-byte aligned");
  const int S = router_splits(T, H);
  if (ws_bytes < (size_t)T * S * E * sizeof(float)) return fail(MOE_ERR_WORKSPACE, "router_topk_splitk: workspace too small");
  int rc = gemm_splitk_f32(x, Wr, T, H, E, S, reinterpret_cast<float*>(ws), status, stream, dtype);
  if (rc) return rc;
  DeviceInfo dev;
  rc = current_device_info(&dev);
  if (rc) return rc;
  int64_t blocks = ceil_div64(T, 8);
  if (blocks > (int64_t)dev.sm_count * 8) blocks = (int64_t)dev.sm_count * 8;
  router_reduce_topk_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float*>(ws), S, T, E, k, mode, scores, indices, indices32, logits_out);
  MOE_CHECK_LAUNCH("router_reduce_topk_kernel");
  return MOE_OK;
}

extern "C" int moe_ep_regroup(const int32_t* recv_counts, int G, int E_local, int32_t* offsets, int32_t* src_row,
                              void* stream) {
  using namespace moe;
  if (!recv_counts || !offsets || !src_row) return fail(MOE_ERR_ARG, "ep_regroup: null pointer");
  if (G < 1 || E_local < 1 || (int64_t)G * E_local > 20000) return fail(MOE_ERR_UNSUPPORTED, "ep_regroup: G*E_local=%lld out of range", (long long)G * E_local);
  const size_t smem = (size_t)2 * G * E_local * sizeof(int32_t);
  if (smem > 48 * 1024) MOE_CUDA_CHECK(cudaFuncSetAttribute(ep_regroup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  ep_regroup_kernel<<<1, 1024, smem, reinterpret_cast<cudaStream_t>(stream)>>>(recv_counts, G, E_local, offsets, src_row);
  MOE_CHECK_LAUNCH("ep_regroup_kernel");
  return MOE_OK;
}

// ====================================================================================
// Expert parallelism over peer memory: plan tables and the dispatch copy.
//
// Every rank knows cnt[s][v]: how many routed rows source rank s sends to virtual expert
// v = dest_rank * E_local + slot (an all-gather of the per-rank histograms).  From that table alone
// each rank derives, without talking to anyone,
//   offsets[j]   expert-major start of local expert j in its own receive buffer,
//   dst_base[v]  where this rank's rows for virtual expert v start in the destination's buffer
//                (expert-major there: after the rows of lower-ranked sources for the same expert),
//   ret_rank[q], ret_row[q]   for the row it holds at expert-major position q: the source rank and the
//                position in that source's sorted order (= the row of the source's return buffer).
// ====================================================================================
namespace moe {

__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t* __restrict__ cnt_all, int ld, int G, int El, int me, int32_t* __restrict__ offsets,
               int32_t* __restrict__ dst_base, int32_t* __restrict__ ret_rank, int32_t* __restrict__ ret_row,
               int32_t* __restrict__ u_base) {
  extern __shared__ int32_t sh[];
  const int E = G * El;
  int32_t* cnt = sh;                 // [G][E]
  int32_t* dbase = cnt + G * E;      // [E]   expert-major start of virtual expert v on its destination
  int32_t* srcoff = dbase + E;       // [G][El] start of (source s, my expert j) in source s's sorted order
  const int tid = threadIdx.x;
  for (int i = tid; i < G * E; i += 1024) cnt[i] = cnt_all[(i / E) * ld + (i % E)];
  // de-duplicated dispatch: row s of the table also carries, after the E counts, how many distinct tokens source s
  // sends to each destination; this rank's tokens start in destination d's buffer after those of lower ranks
  if (u_base && tid >= 64 && tid < 64 + G) {
    const int d = tid - 64;
    int32_t run = 0;
    for (int s2 = 0; s2 < me; ++s2) run += cnt_all[s2 * ld + E + d];
    u_base[d] = run;
  }
  __syncthreads();
  // per destination d: exclusive scan over its local experts of the rows they receive from all sources
  if (tid < G) {
    int32_t run = 0;
    for (int j = 0; j < El; ++j) {
      const int v = tid * El + j;
      dbase[v] = run;
      for (int s = 0; s < G; ++s) run += cnt[s * E + v];
    }
    if (tid == me) offsets[El] = run;
  }
  // per source s: exclusive prefix over virtual experts up to my range, then inside it
  if (tid >= 32 && tid < 32 + G) {
    const int s = tid - 32;
    int32_t run = 0;
    for (int v = 0; v < me * El; ++v) run += cnt[s * E + v];
    for (int j = 0; j < El; ++j) { srcoff[s * El + j] = run; run += cnt[s * E + me * El + j]; }
  }
  __syncthreads();
  for (int v = tid; v < E; v += 1024) {
    int32_t b = dbase[v];
    for (int s = 0; s < me; ++s) b += cnt[s * E + v];
    dst_base[v] = b;
  }
  for (int j = tid; j < El; j += 1024) offsets[j] = dbase[me * El + j];
  // return table: one warp per (source, local expert) segment
  const int lane = tid & 31;
  for (int seg = tid >> 5; seg < G * El; seg += 32) {
    const int s = seg / El, j = seg - s * El;
    const int v = me * El + j;
    int32_t q0 = dbase[v];
    for (int s2 = 0; s2 < s; ++s2) q0 += cnt[s2 * E + v];
    const int32_t c = cnt[s * E + v], r0 = srcoff[s * El + j];
    for (int i = lane; i < c; i += 32) { ret_rank[q0 + i] = s; ret_row[q0 + i] = r0 + i; }
  }
}

struct PeerPtrs {
  void* p[16];
};

// One warp per routed row p (in this rank's sorted order): copy the token's activation row straight into
// the destination rank's receive buffer at its expert-major position.  Plain 16-byte stores to peer memory.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ perm, const int32_t* __restrict__ topk_idx,
                   const int32_t* __restrict__ id_map, const int32_t* __restrict__ offsets,
                   const int32_t* __restrict__ dst_base, int k, int El, int slot_lo, int slot_hi, int64_t n,
                   int vec_per_row, int E_all, PeerPtrs peers) {
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  // entries whose expert id was out of range were left out of the permutation: only offsets[E_all] of the n are live
  const int64_t n_live = min(n, (int64_t)offsets[E_all]);
  for (int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); p < n_live; p += nwarps) {
    const int32_t f = perm[p];
    const int v = id_map[topk_idx[f]];
    const int dest = v / El;
    const int slot = v - dest * El;
    if (slot < slot_lo || slot >= slot_hi) continue;   // this launch moves only the rows of local experts [lo, hi)
    const int64_t row = (int64_t)dst_base[v] + (p - offsets[v]);
    const uint4* s = x + (int64_t)(f / k) * vec_per_row;
    uint4* d = reinterpret_cast<uint4*>(peers.p[dest]) + row * vec_per_row;
    int i = lane;
    for (; i + 96 < vec_per_row; i += 128) {   // four loads in flight before the first remote store
      const uint4 a = __ldg(s + i), b = __ldg(s + i + 32), c = __ldg(s + i + 64), e = __ldg(s + i + 96);
      d[i] = a; d[i + 32] = b; d[i + 64] = c; d[i + 96] = e;
    }
    for (; i < vec_per_row; i += 32) d[i] = __ldg(s + i);
  }
}

// De-duplicated dispatch, step 1: for every token t of this rank and every destination rank d, u(t,d) = the number
// of tokens t' < t that have at least one of their k experts on d, or -1 if t itself has none there; ucount[d] =
// how many tokens go to d.  A token row then travels to a rank once, whatever the number of its experts there.
// One CTA: the scan over tokens is sequential in chunks of 1024.
__global__ void __launch_bounds__(1024)
ep_unique_kernel(const int32_t* __restrict__ topk_idx, const int32_t* __restrict__ id_map, int Tl, int k, int El, int G,
                 int32_t* __restrict__ urank, int32_t* __restrict__ ucount) {
  __shared__ int32_t wtot[32][16];
  __shared__ int32_t running[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned lt = (1u << lane) - 1u;
  if (tid < 16) running[tid] = 0;
  __syncthreads();
  for (int base = 0; base < Tl; base += 1024) {
    const int t = base + tid;
    unsigned mask = 0;
    if (t < Tl)
      for (int s = 0; s < k; ++s) {
        const int32_t id = topk_idx[t * k + s];
        if ((uint32_t)id < (uint32_t)(G * El)) {            // ids out of range, or mapped to no slot, travel nowhere
          const int v = id_map[id];
          if (v >= 0) mask |= 1u << (v / El);
        }
      }
    int32_t in_warp[16];
#pragma unroll
    for (int d = 0; d < 16; ++d) {
      if (d < G) {
        const unsigned b = __ballot_sync(0xFFFFFFFFu, (mask >> d) & 1u);
        in_warp[d] = __popc(b & lt);
        if (lane == 0) wtot[warp][d] = __popc(b);
      }
    }
    __syncthreads();
    if (t < Tl) {
#pragma unroll
      for (int d = 0; d < 16; ++d) {
        if (d < G) {
          int32_t u = -1;
          if ((mask >> d) & 1u) {
            u = running[d] + in_warp[d];
            for (int w = 0; w < warp; ++w) u += wtot[w][d];
          }
          urank[t * G + d] = u;
        }
      }
    }
    __syncthreads();
    if (tid < G) {
      int32_t add = 0;
      for (int w = 0; w < 32; ++w) add += wtot[w][tid];
      running[tid] += add;
    }
    __syncthreads();
  }
  if (tid < G) ucount[tid] = running[tid];
}

// De-duplicated dispatch, step 2.  Work items of one warp each: first the Tl*G (token, destination) pairs - the
// token's row goes to row u_base[d] + u(t,d) of destination d's receive buffer, once; then the routed entries in
// groups of 32 - entry p (this rank's sorted order) tells its destination which received row it is:
// gidx_d[dst_base[v] + (p - offsets[v])] = u_base[d] + u(t,d).  The destination's up GEMM gathers its expert-major
// rows through that list.  Plain stores to peer memory.
__global__ void __launch_bounds__(256)
ep_dispatch_dedup_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ perm,
                         const int32_t* __restrict__ topk_idx, const int32_t* __restrict__ id_map,
                         const int32_t* __restrict__ offsets, const int32_t* __restrict__ dst_base,
                         const int32_t* __restrict__ urank, const int32_t* __restrict__ u_base, int k, int El, int G,
                         int64_t n, int64_t Tl, int vec_per_row, PeerPtrs recv, PeerPtrs gidx) {
  const int lane = threadIdx.x & 31;
  const int64_t nwarps = (int64_t)gridDim.x * 8;
  const int64_t n_live = min(n, (int64_t)offsets[G * El]);   // entries with an expert id out of range are not in perm
  const int64_t pairs = Tl * G, groups = (n_live + 31) / 32;
  for (int64_t item = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); item < pairs + groups; item += nwarps) {
    if (item < pairs) {
      const int32_t u = urank[item];
      if (u < 0) continue;
      const int64_t t = item / G;
      const int d = (int)(item - t * G);
      const uint4* s = x + t * vec_per_row;
      uint4* dst = reinterpret_cast<uint4*>(recv.p[d]) + (int64_t)(u_base[d] + u) * vec_per_row;
      int i = lane;
      for (; i + 96 < vec_per_row; i += 128) {   // four loads in flight before the first remote store
        const uint4 a = __ldg(s + i), b = __ldg(s + i + 32), c = __ldg(s + i + 64), e = __ldg(s + i + 96);
        dst[i] = a; dst[i + 32] = b; dst[i + 64] = c; dst[i + 96] = e;
      }
      for (; i < vec_per_row; i += 32) dst[i] = __ldg(s + i);
    } else {
      const int64_t p = (item - pairs) * 32 + lane;
      if (p < n_live) {
        const int32_t f = perm[p];
        const int v = id_map[topk_idx[f]];
        const int d = v / El;
        const int64_t t = f / k;
        const int64_t row = (int64_t)dst_base[v] + (p - offsets[v]);
        reinterpret_cast<int32_t*>(gidx.p[d])[row] = u_base[d] + urank[t * G + d];
      }
    }
  }
}

}  // namespace moe

extern "C" int moe_ep_unique(const int32_t* topk_idx, const int32_t* id_map, int64_t Tl, int k, int E_local, int G,
                             int32_t* urank, int32_t* ucount, void* stream) {
  using namespace moe;
  if (!topk_idx || !id_map || !urank || !ucount) return fail(MOE_ERR_ARG, "ep_unique: null pointer");
  if (Tl < 0 || Tl > 0x7FFFFFFFll / 64 || k < 1 || E_local < 1 || G < 1 || G > 16)
    return fail(MOE_ERR_ARG, "ep_unique: bad shape Tl=%lld k=%d E_local=%d G=%d", (long long)Tl, k, E_local, G);
  ep_unique_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(topk_idx, id_map, (int)Tl, k, E_local, G, urank, ucount);
  MOE_CHECK_LAUNCH("ep_unique_kernel");
  return MOE_OK;
}

static int ep_plan_impl(const int32_t* cnt_all, int ld, int G, int E_local, int my_rank, int32_t* offsets,
                        int32_t* dst_base, int32_t* ret_rank, int32_t* ret_row, int32_t* u_base, void* stream) {
  using namespace moe;
  if (!cnt_all || !offsets || !dst_base || !ret_rank || !ret_row) return fail(MOE_ERR_ARG, "ep_plan: null pointer");
  if (G < 1 || G > 16 || E_local < 1 || my_rank < 0 || my_rank >= G) return fail(MOE_ERR_ARG, "ep_plan: bad G=%d E_local=%d rank=%d", G, E_local, my_rank);
  const int E = G * E_local;
  if (ld < E + (u_base ? G : 0)) return fail(MOE_ERR_ARG, "ep_plan: row stride %d too small", ld);
  const size_t smem = ((size_t)G * E + E + (size_t)G * E_local) * sizeof(int32_t);
  if (smem > 200 * 1024) return fail(MOE_ERR_UNSUPPORTED, "ep_plan: G*E=%d too large", G * E);
  if (smem > 48 * 1024) MOE_CUDA_CHECK(cudaFuncSetAttribute(ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  ep_plan_kernel<<<1, 1024, smem, reinterpret_cast<cudaStream_t>(stream)>>>(cnt_all, ld, G, E_local, my_rank, offsets, dst_base,
                                                                            ret_rank, ret_row, u_base);
  MOE_CHECK_LAUNCH("ep_plan_kernel");
  return MOE_OK;
}

extern "C" int moe_ep_plan_dedup(const int32_t* cnt_all, int G, int E_local, int my_rank, int32_t* offsets,
                                 int32_t* dst_base, int32_t* ret_rank, int32_t* ret_row, int32_t* u_base, void* stream) {
  if (!u_base) return moe::fail(MOE_ERR_ARG, "ep_plan_dedup: null pointer");
  return ep_plan_impl(cnt_all, G * E_local + G, G, E_local, my_rank, offsets, dst_base, ret_rank, ret_row, u_base, stream);
}

extern "C" int moe_ep_dispatch_dedup(const void* x, const int32_t* perm, const int32_t* topk_idx, const int32_t* id_map,
                                     const int32_t* offsets, const int32_t* dst_base, const int32_t* urank,
                                     const int32_t* u_base, int k, int E_local, int64_t n, int64_t Tl, int64_t H,
                                     void* const* peer_recv, void* const* peer_gidx, int G, void* stream) {
  using namespace moe;
  if (!x || !perm || !topk_idx || !id_map || !offsets || !dst_base || !urank || !u_base || !peer_recv || !peer_gidx)
    return fail(MOE_ERR_ARG, "ep_dispatch_dedup: null pointer");
  if (G < 1 || G > 16 || k < 1 || E_local < 1 || H < 8 || H % 8 || n < 0 || Tl < 0) return fail(MOE_ERR_ARG, "ep_dispatch_dedup: bad shape");
  if (n == 0) return MOE_OK;
  PeerPtrs pr, pg;
  for (int g = 0; g < 16; ++g) { pr.p[g] = g < G ? peer_recv[g] : nullptr; pg.p[g] = g < G ? peer_gidx[g] : nullptr; }
  for (int g = 0; g < G; ++g)
    if (!pr.p[g] || !pg.p[g] || (reinterpret_cast<uintptr_t>(pr.p[g]) & 15) || (reinterpret_cast<uintptr_t>(pg.p[g]) & 3))
      return fail(MOE_ERR_ARG, "ep_dispatch_dedup: peer buffer %d null or unaligned", g);
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  int64_t blocks = ceil_div64(Tl * G + ceil_div64(n, 32), 8);
  const int64_t cap = (int64_t)dev.sm_count * 8;
  if (blocks > cap) blocks = cap;
  ep_dispatch_dedup_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), perm, topk_idx, id_map, offsets, dst_base, urank, u_base, k, E_local, G, n, Tl,
      (int)(H / 8), pr, pg);
  MOE_CHECK_LAUNCH("ep_dispatch_dedup_kernel");
  return MOE_OK;
}

extern "C" int moe_ep_plan(const int32_t* cnt_all, int G, int E_local, int my_rank, int32_t* offsets, int32_t* dst_base,
                           int32_t* ret_rank, int32_t* ret_row, void* stream) {
  return ep_plan_impl(cnt_all, G * E_local, G, E_local, my_rank, offsets, dst_base, ret_rank, ret_row, nullptr, stream);
}

extern "C" int moe_ep_dispatch(const void* x, const int32_t* perm, const int32_t* topk_idx, const int32_t* id_map,
                               const int32_t* offsets, const int32_t* dst_base, int k, int E_local, int slot_lo,
                               int slot_hi, int64_t n, int64_t H, void* const* peer_recv, int G, void* stream) {
  using namespace moe;
  if (!x || !perm || !topk_idx || !id_map || !offsets || !dst_base || !peer_recv) return fail(MOE_ERR_ARG, "ep_dispatch: null pointer");
  if (G < 1 || G > 16 || k < 1 || E_local < 1 || H < 8 || H % 8 || n < 0) return fail(MOE_ERR_ARG, "ep_dispatch: bad shape");
  if (slot_lo < 0 || slot_hi > E_local || slot_lo >= slot_hi) return fail(MOE_ERR_ARG, "ep_dispatch: bad slot range [%d,%d)", slot_lo, slot_hi);
  if (n == 0) return MOE_OK;
  PeerPtrs pp;
  for (int g = 0; g < 16; ++g) pp.p[g] = g < G ? peer_recv[g] : nullptr;
  for (int g = 0; g < G; ++g)
    if (!pp.p[g] || (reinterpret_cast<uintptr_t>(pp.p[g]) & 15)) return fail(MOE_ERR_ARG, "ep_dispatch: peer buffer %d null or unaligned", g);
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  int64_t blocks = ceil_div64(n, 8);
  const int64_t cap = (int64_t)dev.sm_count * 8;
  if (blocks > cap) blocks = cap;
  ep_dispatch_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(x), perm, topk_idx, id_map, offsets, dst_base, k, E_local, slot_lo, slot_hi, n,
      (int)(H / 8), G * E_local, pp);
  MOE_CHECK_LAUNCH("ep_dispatch_kernel");
  return MOE_OK;
}

// ====================================================================================
// Barrier between the ranks of an expert-parallel group over peer memory, with a time limit.
//
// Every rank owns a row of G 32-bit flags per channel in memory its peers can write.  Arriving = storing this
// barrier's epoch into slot [my rank] of every peer's row (after a system-scope fence, so that the rows this rank
// stored into peer buffers before the barrier are visible first); waiting = polling the own row until every slot has
// reached the epoch.  One thread per peer.  A wait that outlasts the limit writes status = {ST_WAIT_TIMEOUT,
// 40 + channel, peer} and returns: the kernels behind it run on stale data, the host sees the status word, and no
// GPU spins for ever because a peer died.
// ====================================================================================
namespace moe {
// thread j's part of barrier `epoch` on `channel`: tell peer j that this rank has arrived, wait (time-limited) for peer j
__device__ __forceinline__ void ep_barrier_thread(const PeerPtrs& flags, int j, int me, int channel, int32_t epoch,
                                                  unsigned long long limit_ns, int32_t* __restrict__ status);

__global__ void __launch_bounds__(32)
ep_barrier_kernel(PeerPtrs flags, int G, int me, int channel, int32_t epoch, unsigned long long limit_ns,
                  int32_t* __restrict__ status) {
  const int j = threadIdx.x;
  if (j >= G) return;
  ep_barrier_thread(flags, j, me, channel, epoch, limit_ns, status);
}

__device__ __forceinline__ void ep_barrier_thread(const PeerPtrs& flags, int j, int me, int channel, int32_t epoch,
                                                  unsigned long long limit_ns, int32_t* __restrict__ status) {
  __threadfence_system();
  volatile int32_t* theirs = reinterpret_cast<volatile int32_t*>(flags.p[j]) + channel * 16 + me;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const int32_t* mine = reinterpret_cast<const int32_t*>(flags.p[me]) + channel * 16 + j;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v - epoch >= 0) break;                       // epochs only grow (wrap-safe comparison)
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > limit_ns) {
      if (status && atomicCAS(&status[0], 0, ST_WAIT_TIMEOUT) == 0) { status[1] = 40 + channel; status[2] = j; }
      break;
    }
    __nanosleep(64);
  }
  __threadfence_system();
}

// All-gather of every rank's small histogram over peer memory, closed by the barrier: this rank's `na + nb` ints go into
// row `me` of table `slot` on every rank; once the barrier has passed, every rank's row is in this rank's own table.
// Two tables (slot = step parity) so that a rank that is a step ahead never overwrites a row still being read.
__global__ void __launch_bounds__(256)
ep_share_counts_kernel(const int32_t* __restrict__ a, int na, const int32_t* __restrict__ b, int nb, PeerPtrs tables,
                       int slot, PeerPtrs flags, int G, int me, int channel, int32_t epoch, unsigned long long limit_ns,
                       int32_t* __restrict__ status) {
  const int width = na + nb;
  for (int g = 0; g < G; ++g) {
    int32_t* dst = reinterpret_cast<int32_t*>(tables.p[g]) + ((int64_t)slot * G + me) * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = i < na ? a[i] : b[i - na];
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < G) ep_barrier_thread(flags, threadIdx.x, me, channel, epoch, limit_ns, status);
}
}  // namespace moe

extern "C" int moe_ep_barrier(void* const* peer_flags, int G, int my_rank, int channel, int32_t epoch,
                              int64_t timeout_us, int32_t* status, void* stream) {
  using namespace moe;
  if (!peer_flags) return fail(MOE_ERR_ARG, "ep_barrier: null pointer");
  if (G < 1 || G > 16 || my_rank < 0 || my_rank >= G || channel < 0 || channel >= 4 || timeout_us < 1)
    return fail(MOE_ERR_ARG, "ep_barrier: bad G=%d rank=%d channel=%d timeout_us=%lld", G, my_rank, channel, (long long)timeout_us);
  PeerPtrs pf;
  for (int g = 0; g < 16; ++g) pf.p[g] = g < G ? peer_flags[g] : nullptr;
  for (int g = 0; g < G; ++g)
    if (!pf.p[g] || (reinterpret_cast<uintptr_t>(pf.p[g]) & 3)) return fail(MOE_ERR_ARG, "ep_barrier: flag row %d null or unaligned", g);
  ep_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(pf, G, my_rank, channel, epoch,
                                                                          (unsigned long long)timeout_us * 1000ull, status);
  MOE_CHECK_LAUNCH("ep_barrier_kernel");
  return MOE_OK;
}

int moe::bounds_status_route(int32_t* out3, cudaStream_t st) { return moe::bounds_status_read(out3, st); }

extern "C" int moe_debug_bounds_status(int32_t* out3, void* stream) {
  using namespace moe;
  if (!out3) return fail(MOE_ERR_ARG, "debug_bounds_status: null pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int32_t a[3], b[3];
  int rc = bounds_status_gemm(a, st);
  if (rc) return rc;
  rc = bounds_status_route(b, st);
  if (rc) return rc;
  const int32_t* first = a[0] ? a : b;
  out3[0] = first[0]; out3[1] = first[1]; out3[2] = first[2];
#ifdef MOE_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

extern "C" int moe_ep_share_counts(const int32_t* counts, int n_counts, const int32_t* extra, int n_extra,
                                   void* const* peer_tables, int slot, void* const* peer_flags, int G, int my_rank,
                                   int channel, int32_t epoch, int64_t timeout_us, int32_t* status, void* stream) {
  using namespace moe;
  if (!counts || !peer_tables || !peer_flags || (n_extra > 0 && !extra)) return fail(MOE_ERR_ARG, "ep_share_counts: null pointer");
  if (G < 1 || G > 16 || my_rank < 0 || my_rank >= G || channel < 0 || channel >= 4 || timeout_us < 1 || slot < 0 || slot > 1 ||
      n_counts < 1 || n_extra < 0)
    return fail(MOE_ERR_ARG, "ep_share_counts: bad G=%d rank=%d channel=%d slot=%d n=%d+%d timeout_us=%lld", G, my_rank, channel,
                slot, n_counts, n_extra, (long long)timeout_us);
  PeerPtrs pt, pf;
  for (int g = 0; g < 16; ++g) { pt.p[g] = g < G ? peer_tables[g] : nullptr; pf.p[g] = g < G ? peer_flags[g] : nullptr; }
  for (int g = 0; g < G; ++g)
    if (!pt.p[g] || !pf.p[g] || ((reinterpret_cast<uintptr_t>(pt.p[g]) | reinterpret_cast<uintptr_t>(pf.p[g])) & 3))
      return fail(MOE_ERR_ARG, "ep_share_counts: table or flag row %d null or unaligned", g);
  ep_share_counts_kernel<<<1, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      counts, n_counts, extra, n_extra, pt, slot, pf, G, my_rank, channel, epoch, (unsigned long long)timeout_us * 1000ull, status);
  MOE_CHECK_LAUNCH("ep_share_counts_kernel");
  return MOE_OK;
}

// ====================================================================================
// Histogram entry point for callers that have no scratch buffer to give.
//
// The per-unit count table that moe_route_histogram keeps in caller-provided workspace lives
// here in a fixed array inside the library's device image.  The array is 1 MiB, exists once on
// every GPU that loads the library, and is never freed.
// ====================================================================================
namespace moe {
constexpr int64_t STATIC_SCRATCH_INTS = 262144;   // 1 MiB of int32
static __device__ __align__(256) int32_t g_route_static_scratch[STATIC_SCRATCH_INTS];

// In host code the array's name is only a handle for the runtime, not an address a kernel can use;
// the device address is looked up once per GPU (with that GPU current) and remembered.
static int static_scratch_address(int32_t** out) {
  static std::mutex mu;
  static int32_t* cached[64] = {nullptr};
  int dev = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MOE_ERR_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    int32_t* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_route_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_route_static_scratch)");
    if (!ptr) return fail(MOE_ERR_DEVICE, "no device address for the built-in scratch array");
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return MOE_OK;
}
}  // namespace moe

extern "C" int moe_route_histogram_static(const void* topk_idx, int idx_is_int64, int64_t n, int E,
                                          const int32_t* id_map, int32_t* counts, int32_t* offsets, int32_t* perm,
                                          int32_t* inv, int32_t* status, void* stream) {
  using namespace moe;
  if (n < 0 || E < 1) return fail(MOE_ERR_ARG, "route_histogram_static: bad size n=%lld E=%d", (long long)n, E);
  if (!counts || !offsets) return fail(MOE_ERR_ARG, "route_histogram_static: null counts/offsets");
  if (n > 0 && !topk_idx) return fail(MOE_ERR_ARG, "route_histogram_static: null ids");
  if ((size_t)RWPB * E * 4 > 160 * 1024) return fail(MOE_ERR_UNSUPPORTED, "route_histogram_static: E=%d too large", E);
  const int64_t units = ceil_div64(n, RUNIT);
  if (units * (int64_t)E > STATIC_SCRATCH_INTS)
    return fail(MOE_ERR_UNSUPPORTED,
                "route_histogram_static: ceil(n/%d)*E = %lld exceeds the built-in scratch of %lld entries; "
                "use moe_route_histogram with a workspace", RUNIT, (long long)(units * E), (long long)STATIC_SCRATCH_INTS);
  int32_t* unit_counts = nullptr;
  int rc = static_scratch_address(&unit_counts);   // first call on a GPU performs the look-up
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)RWPB * E * 4;
  if (smem > 48 * 1024) {
    MOE_CUDA_CHECK(cudaFuncSetAttribute(route_count_kernel<RUNIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MOE_CUDA_CHECK(cudaFuncSetAttribute(route_scatter_kernel<RUNIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  const unsigned blocks = (unsigned)ceil_div64(units, RWPB);
  // Nothing in the array has to start at zero: the count kernel writes every entry of the
  // units x E table it will later read, so whatever an earlier call left behind is overwritten.
  if (units > 0) {
    route_count_kernel<RUNIT><<<blocks, RWPB * 32, smem, st>>>(topk_idx, idx_is_int64, n, E, id_map, unit_counts, status, 0);
    MOE_CHECK_LAUNCH("route_count_kernel");
  }
  route_scan_kernel<<<1, 1024, 0, st>>>(unit_counts, units, E, counts, offsets);
  MOE_CHECK_LAUNCH("route_scan_kernel");
  if (units > 0 && (perm || inv)) {
    route_scatter_kernel<RUNIT><<<blocks, RWPB * 32, smem, st>>>(topk_idx, idx_is_int64, n, E, id_map, unit_counts, perm, inv, 0);
    MOE_CHECK_LAUNCH("route_scatter_kernel");
  }
  return MOE_OK;
}
