// Ragged expert grouped GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM.
//
//   Y[rows of expert e] = A[rows of expert e] . B[e]^T          (A: [rows,K], B: [E,N,K], K contiguous)
//
// One persistent CTA per SM, 256 threads in four roles (192 threads and the first three roles in the CTA-pair and
// tokens-as-N kernels):
//   warp 0      TMA producer: per k-block one A box (128 rows x 64) and the B box(es) (BN rows x 64),
//               128-byte swizzled, into a ring of shared-memory stages guarded by mbarriers;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) four times per
//               k-block; tcgen05.commit releases the stage and, after the last k-block, publishes
//               the accumulator.  Also owns the TMEM allocation;
//   warps 2..5  epilogue: tcgen05.ld the fp32 accumulator, apply the fused epilogue, store 16-byte
//               vectors with row masks;
//   warps 6..7  row gather (see below); idle otherwise.
//
// Two tile shapes.  MT=1: 128 rows x BN columns, accumulator double-buffered in TMEM so that the next
// tile's main loop overlaps the epilogue.  MT=2: 256 rows x 256 columns as two M=128 MMAs per K step
// that share one B tile in shared memory - a third less operand traffic into the SM per flop, which is
// what limits the MT=1 shape (all 512 TMEM columns hold one tile, so the epilogue is not overlapped).
// A tile whose expert has no more than 128 rows left issues only the first of the two MMAs.
//
// Tiles are enumerated on the device from the expert offsets (no host sync): expert-major, then
// N tile, then M tile, so that CTAs running side by side share one B tile through L2.
//
// Optional row gather (128-row tiles): instead of a TMA box of a pre-gathered A, two more warps copy the
// tile's A rows straight from the un-permuted activation matrix (row = gather[r] / div) with 16-byte
// cp.async into the same 128-byte-swizzled stage layout, completing on the stage's full barrier next to the
// TMA of B.  This removes the separate gather pass (one write and one read of the sorted copy of A).
//
// Epilogues: plain bf16 / fp32, SiLU(gate)*up with gate and up accumulated side by side in TMEM
// by one N=256 instruction, routing-weight scale + scatter to the (token, slot) row, rows stored into other
// GPUs' buffers as 128-byte segments, and the router's top-k + softmax taken straight from the accumulator row.
// Split-K mode (fp32 output): the N-tile index counts K slices, each slice lands in its own column block.
//
// Every barrier wait is bounded in time; on expiry the kernel records a status code, lets the
// copies it issued land, frees its TMEM and returns.
#include "common.cuh"

#include <cuda.h>
#include <cuda_fp16.h>
#include <atomic>
#include <mutex>
#include <stdlib.h>

// -DMOE_GEMM_TRACE (the `--trace` build): the 128-row kernel stamps every tile with %globaltimer at three points
// and every CTA with a clock64 / %globaltimer pair, into fixed device arrays read back by moe_gemm_trace_read.
// Not compiled into the product library.
#ifdef MOE_GEMM_TRACE
#define MOE_TRACE_MAX_TILES 32768
#define MOE_TRACE_MAX_CTAS 256
__device__ unsigned long long g_trace_tile[3][MOE_TRACE_MAX_TILES];   // MMA start, accumulator ready, epilogue done
__device__ int g_trace_cta[MOE_TRACE_MAX_TILES];
__device__ long long g_trace_clk[MOE_TRACE_MAX_CTAS][4];              // clock64, ns at start; clock64, ns at end
#define MOE_TRACE(...) __VA_ARGS__
#else
#define MOE_TRACE(...)
#endif

namespace moe {
namespace gemm {

constexpr int EPI_ROUTER = 17;         // internal: top-k + softmax of each accumulator row (fused router), no matrix output
constexpr int EPI_PEER = 16;           // internal: plain bf16 rows stored into other GPUs' buffers (row_rank / peer_base)
constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int NUM_THREADS_GATHER = 256;   // 128-row kernel: + two warps that gather A rows when asked to
constexpr int MAX_E = 1024;
constexpr uint64_t WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;   // 1 s per barrier wait
constexpr uint64_t DRAIN_LIMIT_NS = 20ull * 1000ull * 1000ull;    // 20 ms when draining after a failure

template <int MT, int BN>
struct Cfg {
  static constexpr int A_HALF_BYTES = BM * BK * 2;         // one 128-row A tile
  static constexpr int A_BYTES = MT * A_HALF_BYTES;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;  // 6, 4 or 3
  static constexpr int ACC_BUFS = (MT * BN * 2 <= 512) ? 2 : 1;
  static constexpr int TMEM_COLS = ACC_BUFS * MT * BN;       // 256 or 512: powers of two >= 32
  // layout: [stages][barriers 256 B][tile tables]
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TABLE_OFFSET = BAR_OFFSET + 256;
  static constexpr int STAGING_OFFSET = (TABLE_OFFSET + 3 * (MAX_E + 1) * 4 + 127) & ~127;   // 16-byte accesses
  static constexpr int SMEM_BYTES = STAGING_OFFSET + 1024;  // + alignment slack
  // peer epilogue: 4 warps x 32 rows x (128 B + 16 B pad) to turn per-thread rows into 128-byte row segments
  static constexpr int STAGING_PITCH = 144;
  static constexpr int SMEM_BYTES_PEER = SMEM_BYTES + 4 * 32 * STAGING_PITCH;
  static_assert(STAGING_OFFSET % 16 == 0 && STAGING_PITCH % 16 == 0, "staging rows are accessed as 16-byte vectors");
  static_assert(SMEM_BYTES_PEER <= 227 * 1024, "shared memory budget");
};

struct Params {
  const int32_t* offsets = nullptr;
  const int32_t* dst_rows = nullptr;
  const float* row_w = nullptr;
  void* Y = nullptr;
  int64_t ldy = 0;
  int K = 0, N = 0, E = 0;
  int num_n_tiles = 0;
  int num_k_blocks = 0;
  int f16 = 0;           // 0: bf16 inputs / outputs, 1: fp16
  int32_t* status = nullptr;
  // optional scatter of output rows into other GPUs' buffers (expert-parallel combine): row r goes to
  // peer_base[row_rank[r]] at row dst_rows[r]; plain stores to peer memory from the epilogue
  const int32_t* row_rank = nullptr;
  void* peer_base[16] = {};
  // optional gather of the A rows (128-row kernel only): sorted row r is row a_gather[r] / a_div of a_src
  const int32_t* a_gather = nullptr;
  const void* a_src = nullptr;
  int a_div = 1;
  int a_src_rows = 0;
  int a_rows = 0;          // entries of a_gather
  int w_by_dst = 0;        // SCALE_SCATTER: row_w is indexed by the destination row instead of the sorted row
  int w_slots = 0;         // > 0: destination rows come in runs of w_slots + 1 per token, row_w has w_slots entries per token
  // fused router (EPI_ROUTER): the N = n_experts accumulator columns of a row are its logits
  int dense_rows = 0;      // offsets == nullptr: one group of this many rows
  float* r_scores = nullptr;     // fp32 [rows, r_k]
  int64_t* r_idx64 = nullptr;    // either may be null
  int32_t* r_idx32 = nullptr;
  float* r_logits = nullptr;     // optional fp32 [rows, N] copy of the logits
  int r_k = 0, r_mode = 0;
  // 128-row kernel: bytes the B box(es) of one stage bring (a box may have fewer rows than the tile has columns)
  int b_tx_bytes = 0;
  // split-K (plain fp32 output only): the N-tile index counts K slices of num_k_blocks blocks each; slice s of
  // row r lands in columns [s*N, (s+1)*N) of Y and the caller adds the slices
  int ksplit = 0;
  int l2_hints = 0;        // 128-row kernel: 0 none, 1 evict-first for weights read once, 2 + evict-last for shared weights
  int mixed = 0;           // 128-row kernel: single-tile and multi-tile experts interleaved in the tile order
  int m64 = 0;             // 128-row kernel: tiles with at most 64 live rows as M = 64 instructions
  int64_t y_rows = 0;      // rows of Y when dst_rows scatters into it (the checked build compares every destination with it)
};

// ------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}

// Bounded wait.  Returns false when the limit expires or another role has already given up
// (*abort_flag != 0); the first to give up records where in status[].
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                            int site, uint64_t limit_ns) {
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > limit_ns) {
      if (atomicExch((int*)abort_flag, 1) == 0 && status) {
        status[0] = ST_WAIT_TIMEOUT;
        status[1] = site;
        status[2] = (int32_t)blockIdx.x;
      }
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          int site, uint64_t limit_ns = WAIT_LIMIT_NS) {
#pragma unroll 1
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, site, limit_ns);
}

// Short bounded wait used only while winding down after a failure: no flag, no status.
__device__ __noinline__ void mbar_wait_drain(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return;
    if (global_timer_ns() - t0 > limit_ns) return;
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// the same load with an L2 eviction-priority hint (a policy from make_policy_*)
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t make_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t make_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// copies src_bytes (16 or 0) from global memory and fills the rest of the 16 bytes with zeros
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// the barrier receives one arrival once every cp.async this thread has issued so far has landed
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// orders shared-memory writes made through the generic proxy before later reads by the async proxy (tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T ; bf16 inputs, fp32 accumulate
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base_lane + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart (SBO), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
  d |= (uint64_t)1 << 46;                    // version
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D fp32, A/B bf16, both K-major, M=128, N=n.
// Instruction descriptor bits: D fp32 (bit 4), A and B format (bits 7.., 10..: 1 = bf16, 0 = fp16), both K-major.
__host__ __device__ constexpr uint32_t make_idesc(int n, int f16 = 0) {
  return (1u << 4) | ((f16 ? 0u : 1u) << 7) | ((f16 ? 0u : 1u) << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
// instruction descriptor for an M x N tile (M counted over the whole pair in cta_group::2 mode)
__host__ __device__ constexpr uint32_t make_idesc_mn(int m, int n, int f16 = 0) {
  return (1u << 4) | ((f16 ? 0u : 1u) << 7) | ((f16 ? 0u : 1u) << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------ tile schedule
struct Tile {
  int e, row0, row_end, n_tile, m_tiles;   // m_tiles: row tiles of the tile's expert
};
// tstart[e] = number of M tiles of experts < e.  Tile ids: expert-major, then N tile, then M tile.
__device__ __forceinline__ Tile decode_tile(int id, const int32_t* tstart, const int32_t* offs, int E, int NT,
                                            int tile_rows) {
  int lo = 0, hi = E - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (tstart[mid + 1] * NT > id) hi = mid; else lo = mid + 1;
  }
  Tile t;
  t.e = lo;
  const int local = id - tstart[lo] * NT;
  const int mt = tstart[lo + 1] - tstart[lo];
  t.n_tile = local / mt;
  const int m_local = local - t.n_tile * mt;
  t.row0 = offs[lo] + m_local * tile_rows;
  t.row_end = offs[lo + 1];
  t.m_tiles = mt;
  return t;
}

// tstart[e] = number of row tiles of the experts before e (tstart[E] = all of them); one warp, each lane a run of
// consecutive experts
__device__ __forceinline__ void tile_prefix(int32_t* tstart, const int32_t* offs, int E, int tile_rows, int lane) {
  const int per = (E + 31) / 32;
  const int e_lo = lane * per, e_hi = min(E, e_lo + per);
  int sum = 0;
  for (int e = e_lo; e < e_hi; ++e) sum += (offs[e + 1] - offs[e] + tile_rows - 1) / tile_rows;
  int inc = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= o) inc += v;
  }
  int run = inc - sum;
  for (int e = e_lo; e < e_hi; ++e) { tstart[e] = run; run += (offs[e + 1] - offs[e] + tile_rows - 1) / tile_rows; }
  if (lane == 31) tstart[E] = inc;
}

// Mixed schedule of the 128-row kernel.  Experts with a single row tile ("light": their tiles stream the weights
// from HBM and leave the tensor pipe waiting) and experts with several ("heavy": weights shared through L2, tensor
// bound) form two tile sequences, each expert-major as above; position g of the launch takes the next tile of one
// or the other in proportion to their lengths, so that at any time the SMs work on both kinds side by side and
// neither HBM nor the tensor pipes sit idle through a run of one kind.
//   hstart[e] = row tiles of the heavy experts before e, lstart[e] = light experts before e.
__device__ __forceinline__ void mixed_prefix(int32_t* hstart, int32_t* lstart, const int32_t* offs, int E, int lane) {
  const int per = (E + 31) / 32;
  const int e_lo = lane * per, e_hi = min(E, e_lo + per);
  int hs = 0, ls = 0;
  for (int e = e_lo; e < e_hi; ++e) {
    const int mt = (offs[e + 1] - offs[e] + BM - 1) / BM;
    if (mt == 1) ++ls; else hs += mt;
  }
  int hi = hs, li = ls;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xFFFFFFFFu, hi, o), b = __shfl_up_sync(0xFFFFFFFFu, li, o);
    if (lane >= o) { hi += a; li += b; }
  }
  int hr = hi - hs, lr = li - ls;
  for (int e = e_lo; e < e_hi; ++e) {
    const int mt = (offs[e + 1] - offs[e] + BM - 1) / BM;
    hstart[e] = hr; lstart[e] = lr;
    if (mt == 1) ++lr; else hr += mt;
  }
  if (lane == 31) { hstart[E] = hi; lstart[E] = li; }
}
__device__ __forceinline__ Tile decode_mixed(int g, const int32_t* hstart, const int32_t* lstart, const int32_t* offs,
                                             int E, int NT) {
  const unsigned long long th = (unsigned long long)hstart[E] * NT, tl = (unsigned long long)lstart[E] * NT;
  const int hc = (int)(((unsigned long long)g * th) / (th + tl));              // heavy tiles before position g
  const int hc1 = (int)(((unsigned long long)(g + 1) * th) / (th + tl));
  if (hc1 > hc) return decode_tile(hc, hstart, offs, E, NT, BM);              // light experts own no tiles of this table
  const int id = g - hc;                                                      // light tile number id
  int lo = 0, hi = E - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (lstart[mid + 1] * NT > id) hi = mid; else lo = mid + 1;
  }
  Tile t;
  t.e = lo;
  t.n_tile = id - lstart[lo] * NT;
  t.row0 = offs[lo];
  t.row_end = offs[lo + 1];
  t.m_tiles = 1;
  return t;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
// two fp32 -> two 16-bit outputs of the tensor's element type
__device__ __forceinline__ uint32_t pack_out(float a, float b, int f16) {
  if (f16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  return pack_bf16(a, b);
}
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + __expf(-g)) * u; }

// ------------------------------------------------------------------------------ kernel
template <int MT, int BN, int EPI, bool GATHER>
__global__ void __launch_bounds__(GATHER ? NUM_THREADS_GATHER : NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmB2, const Params p) {
  using C = Cfg<MT, BN>;
  constexpr int STAGES = C::STAGES;
  constexpr int ACC_BUFS = C::ACC_BUFS;
  constexpr int TILE_ROWS = MT * BM;
  constexpr int OUT_COLS = EPI == MOE_GEMM_SILU_GATE ? BN / 2 : BN;   // output columns per tile
  extern __shared__ unsigned char smem_dyn[];
  // the swizzle pattern needs 1024-byte aligned stage buffers
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty, [2S+4] drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::BAR_OFFSET + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::BAR_OFFSET + 208);
  int32_t* tstart = reinterpret_cast<int32_t*>(smem + C::TABLE_OFFSET);
  int32_t* offs = tstart + (MAX_E + 1);
  int32_t* lstart = offs + (MAX_E + 1);            // mixed schedule: tstart then counts the heavy experts' tiles only
  const bool mixed = p.mixed != 0;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
  const uint32_t drain_bar = smem_u32(bars + 2 * STAGES + 4);
  const int E = p.E, NT = p.num_n_tiles, NKB = p.num_k_blocks;
  constexpr bool gather = GATHER;   // its own instantiation: the copy loops cost every warp of the kernel registers

  // ---- set-up: barriers, TMEM, tile table
  if (threadIdx.x == 0) {
    // full: the TMA producer's arrive (+ one arrival per lane of the two gather warps once its copies have landed)
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, gather ? 65 : 1); mbar_init(empty0 + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (EPI == MOE_GEMM_SILU_GATE) prefetch_tmap(&tmB2);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offs[e] = p.offsets ? p.offsets[e] : (e == 0 ? 0 : p.dense_rows);
  __syncthreads();
  if (warp == 2) { if (mixed) mixed_prefix(tstart, lstart, offs, E, lane); else tile_prefix(tstart, offs, E, TILE_ROWS, lane); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = (tstart[E] + (mixed ? lstart[E] : 0)) * NT;
  MOE_TRACE(if (threadIdx.x == 0 && blockIdx.x < MOE_TRACE_MAX_CTAS) {
    g_trace_clk[blockIdx.x][0] = clock64(); g_trace_clk[blockIdx.x][1] = (long long)global_timer_ns(); })

  if (warp == 0) {
    // ===================================================================== TMA producer
    int stage = 0;
    uint32_t phase = 0;
    uint32_t issued = 0;
    bool ok = true;
    const uint64_t pol_first = make_policy_evict_first(), pol_last = make_policy_evict_last();
    uint64_t pol_normal;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol_normal));
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const Tile t = (mixed ? decode_mixed(tile, tstart, lstart, offs, E, NT) : decode_tile(tile, tstart, offs, E, NT, TILE_ROWS));
      const int n0 = p.ksplit ? 0 : t.n_tile * OUT_COLS;
      const int k0 = p.ksplit ? t.n_tile * NKB * BK : 0;        // first K element of this tile's slice
      // weights of an expert with a single row tile are read exactly once: they should leave L2 first; weights that
      // several row tiles share stay as long as L2 lets them
      const uint64_t b_policy = p.l2_hints == 0 ? pol_normal : (t.m_tiles == 1 ? pol_first : (p.l2_hints == 2 ? pol_last : pol_normal));
      for (int kb = 0; kb < NKB; ++kb) {
        if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
        if (lane == 0) {
          const uint32_t full = full0 + 8 * stage;
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
          mbar_arrive_expect_tx(full, gather ? p.b_tx_bytes : C::A_BYTES + p.b_tx_bytes);
          if (!gather) tma_load_2d(sa, &tmA, full, k0 + kb * BK, t.row0);
          if (EPI == MOE_GEMM_SILU_GATE) {
            tma_load_3d_hint(sb, &tmB, full, kb * BK, n0, t.e, b_policy);
            tma_load_3d_hint(sb + C::B_BYTES / 2, &tmB2, full, kb * BK, n0, t.e, b_policy);
          } else {
            tma_load_3d_hint(sb, &tmB, full, k0 + kb * BK, n0, t.e, b_policy);
          }
        }
        __syncwarp();
        ++issued;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok) {
      // let the copies already issued land before the CTA retires its shared memory
      const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0;
      for (uint32_t j = first; j < issued; ++j)
        mbar_wait_drain(full0 + 8 * (j % STAGES), (j / STAGES) & 1, DRAIN_LIMIT_NS);
    }
  } else if (warp == 1) {
    // ===================================================================== MMA issuer
    const uint32_t idesc = make_idesc(BN, p.f16);
    const uint32_t idesc64 = make_idesc_mn(64, BN, p.f16);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const Tile t = (mixed ? decode_mixed(tile, tstart, lstart, offs, E, NT) : decode_tile(tile, tstart, offs, E, NT, TILE_ROWS));
      const bool second_half = MT == 2 && (t.row_end - t.row0) > BM;   // rows beyond the first 128 exist
      // a tile with at most 64 live rows is issued as M = 64 instructions: same time per instruction, half the rows
      // switching in the tensor core (what counts under the power cap); its accumulator uses lanes 0..15 of every
      // 32-lane quarter of tensor memory
      const uint32_t idesc_t = (MT == 1 && p.m64 && t.row_end - t.row0 <= 64) ? idesc64 : idesc;
      if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, p.status, 2)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * MT * BN);
      for (int kb = 0; kb < NKB; ++kb) {
        if (!mbar_wait(full0 + 8 * stage, phase, abort_flag, p.status, 3)) { ok = false; break; }
        tc_fence_after();
        MOE_TRACE(if (lane == 0 && kb == 0 && tile < MOE_TRACE_MAX_TILES) {
          g_trace_tile[0][tile] = global_timer_ns(); g_trace_cta[tile] = blockIdx.x; })
        if (lane == 0) {
          if (gather) fence_proxy_async();   // the A rows were written by cp.async, not by the TMA unit
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + C::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing K by 16 bf16 = 32 bytes inside the swizzle row: +2 in the (addr >> 4) field
            umma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc_t, (kb | k) != 0 ? 1u : 0u);
            if (second_half)   // rows 128..255 of the tile: next A half (16 KB further), same B, next accumulator
              umma_bf16(d_tmem + BN, adesc + (uint64_t)(C::A_HALF_BYTES >> 4) + (uint64_t)(2 * k),
                        bdesc + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * stage);
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(tfull0 + 8 * acc);
      __syncwarp();
      if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1; }
    }
    if (!ok) {
      // wait (bounded) until the tensor-core work issued so far has retired, so TMEM can be freed
      if (lane == 0) umma_commit(drain_bar);
      __syncwarp();
      mbar_wait_drain(drain_bar, 0, DRAIN_LIMIT_NS);
    }
  } else if (warp >= 6) {
    // ===================================================================== A-row gather (only when asked to)
    // Two warps, 64 tile rows each.  8 lanes cover the 128 bytes of one row, so one cp.async instruction moves
    // four whole 128-byte row pieces; a lane keeps the 16 source pointers it needs for the whole tile.
    if (gather) {
      const unsigned char* src_base = reinterpret_cast<const unsigned char*>(p.a_src);
      const size_t row_bytes = (size_t)p.K * 2;
      const int chunk = lane & 7, sub = lane >> 3;
      const int half_row0 = (warp - 6) * 64;             // first tile row of this warp
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const Tile t = (mixed ? decode_mixed(tile, tstart, lstart, offs, E, NT) : decode_tile(tile, tstart, offs, E, NT, TILE_ROWS));
        // lane l reads the list entries of rows l and l + 32 of this warp's half.  Rows past the end of the
        // expert's group are filled with zeros (nothing is read for them): their products are never stored,
        // and zero operands keep the tensor cores' switching power down on the padding of ragged groups
        uint32_t src_row[2];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          int r = t.row0 + half_row0 + lane + 32 * s;
          if (r > p.a_rows - 1) r = p.a_rows - 1;
          uint32_t v = (uint32_t)p.a_gather[r] / (uint32_t)p.a_div;
          if (v >= (uint32_t)p.a_src_rows) {      // never followed: the last row stands in (the checked build reports it)
            (void)MOE_INDEX_OK(v, p.a_src_rows, 2);
            v = (uint32_t)(p.a_src_rows - 1);
          }
          src_row[s] = v;
        }
        const unsigned char* rp[16];
        uint32_t live = 0;                                                  // bit `it`: that row belongs to the group
#pragma unroll
        for (int it = 0; it < 16; ++it) {
          const int row = it * 4 + sub;                                     // row within this warp's half
          const uint32_t sr = __shfl_sync(0xFFFFFFFFu, src_row[it >> 3], row & 31);
          rp[it] = src_base + (size_t)sr * row_bytes + chunk * 16;
          if (t.row0 + half_row0 + row < t.row_end) live |= 1u << it;
        }
        for (int kb = 0; kb < NKB; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 5)) { ok = false; break; }
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES) + half_row0 * 128;
          const size_t koff = (size_t)kb * (BK * 2);
#pragma unroll
          for (int it = 0; it < 16; ++it) {
            const int row = it * 4 + sub;
            // 128-byte swizzle: 16-byte chunk c of row r sits at chunk (c ^ (r & 7)) of that row
            cp_async_16(sa + row * 128 + ((chunk ^ (row & 7)) << 4), rp[it] + koff, (live >> it) & 1u ? 16u : 0u);
          }
          cp_async_arrive_noinc(full0 + 8 * stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      cp_async_wait_all();   // nothing of this warp's is still in flight when the CTA retires its shared memory
    }
  } else {
    // ===================================================================== epilogue (warps 2..5)
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const Tile t = (mixed ? decode_mixed(tile, tstart, lstart, offs, E, NT) : decode_tile(tile, tstart, offs, E, NT, TILE_ROWS));
      if (!mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, p.status, 4)) { ok = false; break; }
      tc_fence_after();
      MOE_TRACE(if (warp == 2 && lane == 0 && tile < MOE_TRACE_MAX_TILES) g_trace_tile[1][tile] = global_timer_ns();)
#pragma unroll 1
      for (int half = 0; half < MT; ++half) {
      if (half == 1 && t.row0 + BM >= t.row_end) break;   // nothing was accumulated for rows 128..255
      // sorted row handled by this thread; an M = 64 tile keeps rows 16q .. 16q+15 in the first 16 lanes of quarter q
      const bool m64 = MT == 1 && p.m64 && t.row_end - t.row0 <= 64;
      const int grow = m64 ? t.row0 + q * 16 + lane : t.row0 + half * BM + q * 32 + lane;
      bool row_ok = grow < t.row_end && (!m64 || lane < 16);
      const int n0 = p.ksplit ? 0 : t.n_tile * OUT_COLS;
      int64_t out_row = grow;
      float w = 1.0f;
      void* ybase = p.Y;
      if (row_ok) {
        if (EPI != MOE_GEMM_SILU_GATE && p.dst_rows) {
          out_row = p.dst_rows[grow];
          if (EPI != EPI_PEER && !MOE_INDEX_OK(out_row, p.y_rows, 1)) { row_ok = false; out_row = grow; }
        }
      }
      if (row_ok) {
        if (EPI == MOE_GEMM_SCALE_SCATTER) {
          if (p.w_slots > 0) {   // destination rows in runs of w_slots + 1 per token; the run's last row weighs 1
            const int64_t tok = out_row / (p.w_slots + 1);
            const int sl = (int)(out_row - tok * (p.w_slots + 1));
            w = sl < p.w_slots ? p.row_w[tok * p.w_slots + sl] : 1.0f;
          } else {
            w = p.row_w[p.w_by_dst ? out_row : (int64_t)grow];
          }
        }
        if (EPI == EPI_PEER) ybase = p.peer_base[p.row_rank[grow]];
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * MT * BN + half * BN);
      if (EPI == EPI_ROUTER) {
        // This thread's accumulator row holds the N logits of one token: keep the k largest in a sorted list
        // (ascending column scan + strict comparison = lowest index first among equals), then normalise.
        constexpr int KMAX = 8;
        int kv[KMAX], ki[KMAX];
#pragma unroll
        for (int j = 0; j < KMAX; ++j) { kv[j] = (int)0x80000000; ki[j] = 0; }
        const int chunks = (p.N + 31) / 32;
#pragma unroll 1
        for (int c = 0; c < chunks; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = c * 32 + j;
            const int key = float_to_ikey(__uint_as_float(v[j]));
            if (col < p.N && key > kv[KMAX - 1]) list_insert<KMAX>(kv, ki, key, col);
          }
          if (p.r_logits && row_ok) {
            float* dst = p.r_logits + (int64_t)grow * p.N + c * 32;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (c * 32 + j * 4 < p.N)   // N % 8 == 0: whole 16-byte vectors
                *reinterpret_cast<uint4*>(dst + j * 4) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          }
        }
        const float vmax = ikey_to_float(kv[0]);
        float rowsum = 0.f;
        if (p.r_mode != MOE_TOPK_MODE_B) {       // conventions that normalise over all experts: second pass over TMEM
          double total = 0.0;                    // 32-term fp32 sums added up in fp64: the denominator of up to 256 terms
#pragma unroll 1                                  // keeps the scores within 1e-6 of an exactly summed softmax
          for (int c = 0; c < chunks; ++c) {
            uint32_t v[32];
            tmem_ld32(taddr + c * 32, v);
            tmem_ld_wait();
            float part = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c * 32 + j < p.N) part += expf(__uint_as_float(v[j]) - vmax);
            total += (double)part;
          }
          rowsum = (float)total;
        }
        if (row_ok) {
          float e[KMAX];
          float denom = 0.f;
#pragma unroll
          for (int j = 0; j < KMAX; ++j) {
            e[j] = j < p.r_k ? expf(ikey_to_float(kv[j]) - vmax) : 0.f;
            denom += e[j];
          }
          if (p.r_mode != MOE_TOPK_MODE_B) denom = rowsum;
          float renorm = 0.f;
#pragma unroll
          for (int j = 0; j < KMAX; ++j) { e[j] = e[j] / denom; renorm += e[j]; }
          const int64_t o = (int64_t)grow * p.r_k;
#pragma unroll
          for (int j = 0; j < KMAX; ++j) {
            if (j < p.r_k) {
              p.r_scores[o + j] = p.r_mode == MOE_TOPK_MODE_A_RENORM ? e[j] / renorm : e[j];
              if (p.r_idx64) p.r_idx64[o + j] = (int64_t)ki[j];
              if (p.r_idx32) p.r_idx32[o + j] = (int32_t)ki[j];
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < OUT_COLS / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        if (EPI == MOE_GEMM_SILU_GATE) {
          uint32_t u[32];
          tmem_ld32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(silu_mul(__uint_as_float(v[j]), __uint_as_float(u[j])));
        } else {
          tmem_ld_wait();
          if (EPI == MOE_GEMM_SCALE_SCATTER) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * w);
          }
        }
        const int col = n0 + c * 32;
        if (EPI == EPI_PEER) {
          // Remote rows: NVLink wants long contiguous writes.  Two 32-column chunks of every row are parked in
          // shared memory (this warp's 32 rows x 128 bytes), then written out with 8 lanes per row, so that each
          // store instruction carries four 128-byte row segments instead of thirty-two 16-byte pieces.
          unsigned char* stg = smem + C::STAGING_OFFSET + (warp - 2) * 32 * C::STAGING_PITCH;
          uint4* mine = reinterpret_cast<uint4*>(stg + lane * C::STAGING_PITCH + (c & 1) * 64);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_out(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]), p.f16);
            o.y = pack_out(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]), p.f16);
            o.z = pack_out(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]), p.f16);
            o.w = pack_out(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]), p.f16);
            mine[j] = o;
          }
          if (c & 1) {
            __syncwarp();
            const unsigned long long row_ptr = row_ok
                ? reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16*>(ybase) + out_row * p.ldy) : 0ull;
            const int col0 = n0 + (c - 1) * 32;          // first of the 64 columns parked
            const int seg = lane & 7;                    // 16-byte piece of the 128-byte segment
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int r = it * 4 + (lane >> 3);
              const unsigned long long rp = __shfl_sync(0xFFFFFFFFu, row_ptr, r);
              const uint4 val = *reinterpret_cast<const uint4*>(stg + r * C::STAGING_PITCH + seg * 16);
              if (rp != 0ull && col0 + seg * 8 < p.N)
                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(rp) + col0 + seg * 8) = val;
            }
            __syncwarp();
          }
        } else
        if (row_ok && col < p.N) {
          if (EPI == MOE_GEMM_PLAIN_F32) {
            float* dst = reinterpret_cast<float*>(p.Y) + out_row * p.ldy + col + (p.ksplit ? t.n_tile * p.N : 0);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col + j * 4 < p.N)
                *reinterpret_cast<uint4*>(dst + j * 4) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(ybase) + out_row * p.ldy + col;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col + j * 8 < p.N) {
                uint4 o;
                o.x = pack_out(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]), p.f16);
                o.y = pack_out(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]), p.f16);
                o.z = pack_out(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]), p.f16);
                o.w = pack_out(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]), p.f16);
                *reinterpret_cast<uint4*>(dst + j * 8) = o;
              }
            }
          }
        }
      }
      }  // not the router epilogue
      }  // halves
      MOE_TRACE(if (warp == 2 && lane == 0 && tile < MOE_TRACE_MAX_TILES) g_trace_tile[2][tile] = global_timer_ns();)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      if (++acc == ACC_BUFS) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  MOE_TRACE(if (threadIdx.x == 0 && blockIdx.x < MOE_TRACE_MAX_CTAS) {
    g_trace_clk[blockIdx.x][2] = clock64(); g_trace_clk[blockIdx.x][3] = (long long)global_timer_ns(); })
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------ CTA-pair kernel
// The same pipeline on a cluster of two CTAs driving tcgen05 in cta_group::2 mode.  Two tile shapes in one
// launch (a kernel may use only one cta_group, so the ragged tail has to run under cta_group::2 as well):
//
//   256-row tile   one M=256 x N=256 instruction per K step, 128 rows per CTA;
//   128-row tile   the last tile of an expert when it holds no more than 128 rows: M=128 x N=256, 64 rows per
//                  CTA.  The pair finishes it in half the time of a 256-row tile (measured: 70.8 against 133.9
//                  clocks per K step), so row padding costs what it costs the single-CTA kernel, at most 127
//                  rows per expert.  Its accumulator sits folded in tensor memory: lanes 0..63 of a CTA hold
//                  its 64 rows x columns 0..127, lanes 64..127 the same rows x columns 128..255.
//
// Each CTA stages only its own rows of A and its own half of the B tile (128 of the 256 N rows), 32 KB per
// k-block instead of the 48 KB of the single-CTA shape.  Operand staging (TMA writes) and operand reads (MMA)
// share the SM's shared-memory bandwidth, 128 bytes per clock: 96 KB per k-block against 535 tensor clocks caps
// the single-CTA shape near 70 % of the tensor pipe; 64 KB per k-block does not.
//
// SiLU-gate epilogue: the 256 N rows are ordered [gate f..f+63 | up f..f+63 | gate f+64..f+127 | up f+64..f+127]
// (CTA 0 stages the first two boxes, CTA 1 the last two), so that gate and up of one output element meet in one
// thread for both tile shapes.
//
//   full[s]    lives in CTA 0: its producer posts the byte count of both CTAs, both CTAs' TMA loads
//              complete on it (cta_group::2 loads may signal the peer's barrier);
//   empty[s]   one per CTA, released by the leader's tcgen05.commit (one commit per CTA's barrier);
//   tfull[b]   one per CTA, same way; tempty[b] lives in CTA 0 and collects the epilogue warps of both.
// Row gather: warps 6..7 of each CTA copy their CTA's rows with cp.async.  In CTA 0 every lane's copies complete
// on full[s] directly; cp.async cannot signal another CTA's barrier, so in CTA 1 they complete on a local
// barrier gfull[s], and warp 1 of CTA 1 (idle otherwise: only the leader issues MMAs) waits for it, makes the
// rows visible to the async proxy and arrives on the leader's full[s] across the cluster.
// No multicast load anywhere: every CTA fetches its own boxes.
struct PairCfg {
  static constexpr int BN = 256;
  static constexpr int A_BYTES = BM * BK * 2;            // 16 KB: this CTA's rows (128, or 64 of a 128-row tile)
  static constexpr int B_BYTES = (BN / 2) * BK * 2;      // 16 KB: this CTA's half of the N rows
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TABLE_OFFSET = BAR_OFFSET + 256;
  static constexpr int STAGING_OFFSET = (TABLE_OFFSET + 2 * (MAX_E + 1) * 4 + 127) & ~127;
  static constexpr int SMEM_BYTES = STAGING_OFFSET + 1024;
  static constexpr int STAGING_PITCH = 144;
  static constexpr int SMEM_BYTES_PEER = SMEM_BYTES + 4 * 32 * STAGING_PITCH;
  static_assert((3 * STAGES + 5) * 8 <= 200, "barriers fit below the tensor-memory slot");
  static_assert(SMEM_BYTES_PEER <= 227 * 1024, "shared memory budget");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// arrive on a barrier (shared::cluster address, either CTA's) once the pair's MMAs issued so far retire
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 consecutive output columns of one row, fp32 in registers -> 16-byte stores of the output type
template <int EPI>
__device__ __forceinline__ void store_row_chunk(const Params& p, void* ybase, int64_t out_row, int col, const uint32_t (&v)[32]) {
  if (EPI == MOE_GEMM_PLAIN_F32) {
    float* dst = reinterpret_cast<float*>(ybase) + out_row * p.ldy + col;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (col + j * 4 < p.N)
        *reinterpret_cast<uint4*>(dst + j * 4) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(ybase) + out_row * p.ldy + col;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (col + j * 8 < p.N) {
        uint4 o;
        o.x = pack_out(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]), p.f16);
        o.y = pack_out(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]), p.f16);
        o.z = pack_out(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]), p.f16);
        o.w = pack_out(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]), p.f16);
        *reinterpret_cast<uint4*>(dst + j * 8) = o;
      }
    }
  }
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA64,
                         const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
                         const Params p) {
  using C = PairCfg;
  constexpr int STAGES = C::STAGES;
  constexpr int BN = C::BN;
  constexpr int TILE_ROWS = 2 * BM;
  constexpr bool GATE = EPI == MOE_GEMM_SILU_GATE;
  constexpr int OUT_COLS = GATE ? BN / 2 : BN;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFFSET);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty, [2S+4] drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::BAR_OFFSET + 200);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::BAR_OFFSET + 208);
  volatile uint32_t* tile_light = reinterpret_cast<volatile uint32_t*>(smem + C::BAR_OFFSET + 216);   // ring of 8
  int32_t* tstart = reinterpret_cast<int32_t*>(smem + C::TABLE_OFFSET);
  int32_t* offs = tstart + (MAX_E + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
  const uint32_t tfull0 = smem_u32(bars + 2 * STAGES), tempty0 = smem_u32(bars + 2 * STAGES + 2);
  const uint32_t drain_bar = smem_u32(bars + 2 * STAGES + 4);
  const uint32_t lead_full0 = map_to_cta(full0, 0), lead_tempty0 = map_to_cta(tempty0, 0);
  const int E = p.E, NT = p.num_n_tiles, NKB = p.num_k_blocks;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    // full (used in CTA 0): the producer's arrive; the copies of both CTAs count their bytes on it
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 8); }
    mbar_init(drain_bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmA64);
    prefetch_tmap(&tmB);
    if (GATE) prefetch_tmap(&tmB2);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offs[e] = p.offsets ? p.offsets[e] : (e == 0 ? 0 : p.dense_rows);
  __syncthreads();
  if (warp == 2) tile_prefix(tstart, offs, E, TILE_ROWS, lane);
  tc_fence_before();
  __syncthreads();
  cluster_barrier();   // both CTAs' barriers are initialised before anything remote touches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_tiles = tstart[E] * NT;

  if (warp == 0) {
    // ===================================================================== TMA producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    uint32_t issued = 0;
    uint32_t seq = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < total_tiles; tile += n_clusters) {
      const Tile t = decode_tile(tile, tstart, offs, E, NT, TILE_ROWS);
      const bool light = t.row_end - t.row0 <= BM;           // 128-row tile: 64 rows per CTA
      const int n0 = t.n_tile * OUT_COLS;
      const int a_row = t.row0 + (int)rank * (light ? BM / 2 : BM);
      const uint32_t tx = light ? 2u * (C::A_BYTES / 2 + C::B_BYTES) : 2u * C::STAGE_BYTES;
      // read by the MMA issuer after the first full barrier of the tile; the producer runs at most STAGES (< 8) k-blocks,
      // hence tiles, ahead of it
      if (leader && lane == 0) tile_light[seq & 7] = light ? 1u : 0u;
      ++seq;
      for (int kb = 0; kb < NKB; ++kb) {
        if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
        if (lane == 0) {
          const uint32_t lead_full = lead_full0 + 8 * stage;
          const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
          const uint32_t sb = sa + C::A_BYTES;
          if (leader) mbar_arrive_expect_tx(full0 + 8 * stage, tx);
          tma_load_2d_pair(sa, light ? &tmA64 : &tmA, lead_full, kb * BK, a_row);
          if (GATE) {   // this CTA's 64 gate rows, then its 64 up rows of the same output columns
            tma_load_3d_pair(sb, &tmB, lead_full, kb * BK, n0 + (int)rank * (OUT_COLS / 2), t.e);
            tma_load_3d_pair(sb + C::B_BYTES / 2, &tmB2, lead_full, kb * BK, n0 + (int)rank * (OUT_COLS / 2), t.e);
          } else {
            tma_load_3d_pair(sb, &tmB, lead_full, kb * BK, n0 + (int)rank * (BN / 2), t.e);
          }
        }
        __syncwarp();
        ++issued;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (ok) {
      // tail: the leader's tcgen05.commit arrives on this CTA's empty barriers from the other SM; let the
      // last of those arrivals land before this CTA may retire (bounded like every other wait)
      const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0;
      for (uint32_t j = first; j < issued && ok; ++j)
        ok = mbar_wait(empty0 + 8 * (j % STAGES), (j / STAGES) & 1, abort_flag, p.status, 15);
    }
    if (!ok && leader) {
      // the leader's full barriers count the copies of both CTAs: wait (bounded) for the outstanding ones
      const uint32_t first = issued > (uint32_t)STAGES ? issued - STAGES : 0;
      for (uint32_t j = first; j < issued; ++j)
        mbar_wait_drain(full0 + 8 * (j % STAGES), (j / STAGES) & 1, DRAIN_LIMIT_NS);
    }
  } else if (warp == 1) {
    if (leader) {
      // ===================================================================== MMA issuer (leader CTA only)
      const uint32_t idesc_h = make_idesc_mn(2 * BM, BN, p.f16), idesc_l = make_idesc_mn(BM, BN, p.f16);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t seq = 0;                      // tiles this cluster has started
      bool ok = true;
      for (int tile = cluster_id; ok && tile < total_tiles; tile += n_clusters) {
        uint32_t idesc = idesc_h;
        if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, p.status, 12)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < NKB; ++kb) {
          // the peer's copies count their bytes on this barrier through the TMA unit: the CTA-scope wait is enough
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag, p.status, 13)) { ok = false; break; }
          tc_fence_after();
          // the tile's shape comes from the producer (written before its first arrive on this barrier): a table look-up
          // here would sit between two tiles' instruction streams with the tensor pipe idle
          if (kb == 0) idesc = tile_light[seq & 7] ? idesc_l : idesc_h;
          if (lane == 0) {
            const uint32_t sa = smem_u32(smem + stage * C::STAGE_BYTES);
            const uint64_t adesc = make_smem_desc(sa);
            const uint64_t bdesc = make_smem_desc(sa + C::A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_bf16_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit_pair(empty0 + 8 * stage);                  // this CTA's stage
            umma_commit_pair(map_to_cta(empty0 + 8 * stage, 1));   // the peer's stage
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (lane == 0) {
          umma_commit_pair(tfull0 + 8 * acc);
          umma_commit_pair(map_to_cta(tfull0 + 8 * acc, 1));
        }
        __syncwarp();
        ++seq;
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
      if (!ok) {
        if (lane == 0) umma_commit_pair(drain_bar);
        __syncwarp();
        mbar_wait_drain(drain_bar, 0, DRAIN_LIMIT_NS);
      }
    }
  } else {
    // ===================================================================== epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;                  // tensor-memory lane quarter this warp may read
    const int l = q * 32 + lane;             // this thread's lane
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = cluster_id; ok && tile < total_tiles; tile += n_clusters) {
      const Tile t = decode_tile(tile, tstart, offs, E, NT, TILE_ROWS);
      const bool light = t.row_end - t.row0 <= BM;
      if (!mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, p.status, 14)) { ok = false; break; }
      tc_fence_after();
      // 256-row tile: lane = row of this CTA's 128; 128-row tile: lanes 0..63 and 64..127 both hold this CTA's 64 rows,
      // the upper lanes the second half of the columns
      const int grow = t.row0 + (light ? (int)rank * (BM / 2) + (l & 63) : (int)rank * BM + l);
      const int col_half = light ? (l >> 6) : 0;
      bool row_ok = grow < t.row_end;
      const bool any_rows = t.row0 + (light ? (int)rank * (BM / 2) + (q & 1) * 32 : (int)rank * BM + q * 32) < t.row_end;
      const int n0 = t.n_tile * OUT_COLS;
      int64_t out_row = grow;
      float w = 1.0f;
      void* ybase = p.Y;
      if (row_ok) {
        if (!GATE && p.dst_rows) {
          out_row = p.dst_rows[grow];
          if (EPI != EPI_PEER && !MOE_INDEX_OK(out_row, p.y_rows, 1)) { row_ok = false; out_row = grow; }
        }
      }
      if (row_ok) {
        if (EPI == MOE_GEMM_SCALE_SCATTER) {
          if (p.w_slots > 0) {   // destination rows in runs of w_slots + 1 per token; the run's last row weighs 1
            const int64_t tok = out_row / (p.w_slots + 1);
            const int sl = (int)(out_row - tok * (p.w_slots + 1));
            w = sl < p.w_slots ? p.row_w[tok * p.w_slots + sl] : 1.0f;
          } else {
            w = p.row_w[p.w_by_dst ? out_row : (int64_t)grow];
          }
        }
        if (EPI == EPI_PEER) ybase = p.peer_base[p.row_rank[grow]];
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
      if (GATE) {
        // accumulator columns: [gate 64 | up 64] per group of 64 output columns; a 256-row tile holds two groups,
        // a 128-row tile one per lane half
        const int groups = light ? 1 : 2;
#pragma unroll 1
        for (int g = 0; any_rows && g < groups; ++g) {
          const int cg = light ? 0 : g * 128;
          const int fo = light ? col_half * 64 : g * 64;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32], u[32];
            tmem_ld32(taddr + cg + c * 32, v);
            tmem_ld32(taddr + cg + 64 + c * 32, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(silu_mul(__uint_as_float(v[j]), __uint_as_float(u[j])));
            const int col = n0 + fo + c * 32;
            if (row_ok && col < p.N) store_row_chunk<MOE_GEMM_PLAIN>(p, ybase, out_row, col, v);
          }
        }
      } else {
        const int chunks = light ? 4 : 8;
        const int cb = n0 + col_half * 128;
#pragma unroll 1
        for (int c = 0; any_rows && c < chunks; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
          if (EPI == MOE_GEMM_SCALE_SCATTER) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * w);
          }
          const int col = cb + c * 32;
          if (EPI == EPI_PEER) {
            // two 32-column chunks of every row are parked in shared memory (this warp's 32 rows x 128 bytes), then
            // written out with 8 lanes per row: each store instruction carries four 128-byte row segments
            unsigned char* stg = smem + C::STAGING_OFFSET + (warp - 2) * 32 * C::STAGING_PITCH;
            uint4* mine = reinterpret_cast<uint4*>(stg + lane * C::STAGING_PITCH + (c & 1) * 64);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_out(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]), p.f16);
              o.y = pack_out(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]), p.f16);
              o.z = pack_out(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]), p.f16);
              o.w = pack_out(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]), p.f16);
              mine[j] = o;
            }
            if (c & 1) {
              __syncwarp();
              const unsigned long long row_ptr = row_ok
                  ? reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16*>(ybase) + out_row * p.ldy) : 0ull;
              const int col0 = col - 32;
              const int seg = lane & 7;
#pragma unroll
              for (int it = 0; it < 8; ++it) {
                const int r = it * 4 + (lane >> 3);
                const unsigned long long rp = __shfl_sync(0xFFFFFFFFu, row_ptr, r);
                const uint4 val = *reinterpret_cast<const uint4*>(stg + r * C::STAGING_PITCH + seg * 16);
                if (rp != 0ull && col0 + seg * 8 < p.N)
                  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(rp) + col0 + seg * 8) = val;
              }
              __syncwarp();
            }
          } else if (row_ok && col < p.N) {
            store_row_chunk<EPI>(p, ybase, out_row, col, v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---- teardown: neither CTA may retire its shared memory or TMEM while the other still uses them
  tc_fence_before();
  __syncthreads();
  cluster_barrier();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// bf16 tensor [d2][d1][d0] (d0 contiguous), box [1][box1][64], 128-byte swizzle, zero fill out of bounds
static int make_tmap(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t box1,
                     int f16 = 0) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return fail(MOE_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {(cuuint32_t)BK, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = d2 > 0 ? 3 : 2;
  CUresult r = fn(m, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MOE_ERR_ARG, "cuTensorMapEncodeTiled failed with %d (dims %llu,%llu,%llu box1 %u)", (int)r,
                                     (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, box1);
  return MOE_OK;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel: one flag per (kernel, device)
template <class Kernel>
static int allow_dynamic_smem(Kernel kernel, int bytes, std::atomic<bool>* done_per_device) {
  int dev = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MOE_ERR_DEVICE, "device ordinal %d out of range", dev);
  if (!done_per_device[dev].load(std::memory_order_acquire)) {
    MOE_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done_per_device[dev].store(true, std::memory_order_release);
  }
  return MOE_OK;
}

template <int MT, int BN, int EPI, bool GATHER>
static int launch_g(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const Params& p, int grid,
                    cudaStream_t st) {
  using C = Cfg<MT, BN>;
  constexpr int SMEM = EPI == EPI_PEER ? C::SMEM_BYTES_PEER : C::SMEM_BYTES;
  static std::atomic<bool> attr_set[64];
  int rc = allow_dynamic_smem(grouped_gemm_kernel<MT, BN, EPI, GATHER>, SMEM, attr_set);
  if (rc) return rc;
  grouped_gemm_kernel<MT, BN, EPI, GATHER><<<grid, GATHER ? NUM_THREADS_GATHER : NUM_THREADS, SMEM, st>>>(tA, tB, tB2, p);
  MOE_CHECK_LAUNCH("grouped_gemm_kernel");
  return MOE_OK;
}
template <int MT, int BN, int EPI>
static int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const Params& p, int grid,
                  cudaStream_t st) {
  // the row gather is compiled for the matrix epilogues only (the fused router has none)
  if (EPI != EPI_ROUTER && p.a_gather) return launch_g<MT, BN, EPI == EPI_ROUTER ? MOE_GEMM_PLAIN : EPI, true>(tA, tB, tB2, p, grid, st);
  return launch_g<MT, BN, EPI, false>(tA, tB, tB2, p, grid, st);
}

template <int EPI>
static int launch_pair(const CUtensorMap& tA, const CUtensorMap& tA64, const CUtensorMap& tB, const CUtensorMap& tB2,
                       const Params& p, int grid, cudaStream_t st) {
  constexpr int SMEM = EPI == EPI_PEER ? PairCfg::SMEM_BYTES_PEER : PairCfg::SMEM_BYTES;
  static std::atomic<bool> attr_set[64];
  int rc = allow_dynamic_smem(grouped_gemm_pair_kernel<EPI>, SMEM, attr_set);
  if (rc) return rc;
  grouped_gemm_pair_kernel<EPI><<<grid, NUM_THREADS, SMEM, st>>>(tA, tA64, tB, tB2, p);
  MOE_CHECK_LAUNCH("grouped_gemm_pair_kernel");
  return MOE_OK;
}

}  // namespace gemm
}  // namespace moe

struct GatherArgs {           // A rows fetched through an index list instead of a pre-gathered matrix
  const int32_t* idx = nullptr;
  int div = 1;
  int64_t src_rows = 0;
  int64_t dense_rows = 0;     // > 0 with offsets == nullptr: one group of this many rows (E must be 1)
  int w_slots = 0;            // see Params::w_slots
};

static int grouped_gemm_impl(int epilogue, const void* A, const void* B, const void* B2, const int32_t* offsets,
                             const int32_t* dst_rows, const float* row_w, void* Y, int64_t ldy, int64_t max_rows,
                             int K, int N, int E, int32_t* status, void* stream, const int32_t* row_rank,
                             void* const* peer_base, int n_peers, int64_t expected_rows, int dtype,
                             const GatherArgs& ga = GatherArgs());

extern "C" int moe_grouped_gemm(int epilogue, const void* A, const void* B, const void* B2, const int32_t* offsets,
                                const int32_t* dst_rows, const float* row_w, void* Y, int64_t ldy, int64_t max_rows,
                                int64_t expected_rows, int K, int N, int E, int dtype, int32_t* status, void* stream) {
  return grouped_gemm_impl(epilogue, A, B, B2, offsets, dst_rows, row_w, Y, ldy, max_rows, K, N, E, status, stream,
                           nullptr, nullptr, 0, expected_rows, dtype);
}

extern "C" int moe_grouped_gemm_gathered(int epilogue, const void* X, int64_t x_rows, const int32_t* gather_idx,
                                         int gather_div, const void* B, const void* B2, const int32_t* offsets,
                                         const int32_t* dst_rows, const float* row_w, void* Y, int64_t ldy,
                                         int64_t max_rows, int64_t expected_rows, int K, int N, int E, int dtype,
                                         int32_t* status, void* stream) {
  using namespace moe;
  if (!gather_idx) return fail(MOE_ERR_ARG, "grouped_gemm_gathered: null index list");
  if (gather_div < 1 || x_rows < 1 || x_rows > 0x7FFFFFFFll)
    return fail(MOE_ERR_ARG, "grouped_gemm_gathered: bad gather_div=%d or x_rows=%lld", gather_div, (long long)x_rows);
  if (K % 64) return fail(MOE_ERR_UNSUPPORTED, "grouped_gemm_gathered: K=%d must be a multiple of 64", K);
  GatherArgs ga;
  ga.idx = gather_idx; ga.div = gather_div; ga.src_rows = x_rows;
  return grouped_gemm_impl(epilogue, X, B, B2, offsets, dst_rows, row_w, Y, ldy, max_rows, K, N, E, status, stream,
                           nullptr, nullptr, 0, expected_rows, dtype, ga);
}

// Router GEMM with the top-k + softmax of every logits row done in the epilogue (declared in common.cuh; the
// public entry point moe_router_topk validates the arguments and picks between this and the CUDA-core kernel).
int moe::router_topk_gemm(const void* x, const void* Wr, int64_t T, int H, int E, int k, int mode, int dtype,
                          float* scores, int64_t* indices, int32_t* indices32, float* logits_out,
                          int32_t* status, void* stream) {
  using namespace moe::gemm;
  if (dtype != MOE_DTYPE_BF16 && dtype != MOE_DTYPE_F16) return fail(MOE_ERR_ARG, "router_topk: unknown dtype %d", dtype);
  if (T < 0 || H < 8 || (H % 8) || E < 8 || (E % 8) || k < 1 || k > E)
    return fail(MOE_ERR_ARG, "router_topk: bad shape T=%lld H=%d E=%d k=%d (H, E multiples of 8)", (long long)T, H, E, k);
  if (E > 256 || k > 8) return fail(MOE_ERR_UNSUPPORTED, "router_topk: the fused kernel takes E <= 256 and k <= 8 (E=%d k=%d)", E, k);
  if (mode < 0 || mode > 2) return fail(MOE_ERR_ARG, "router_topk: unknown mode %d", mode);
  if (T == 0) return MOE_OK;
  if (T > 0x7FFFFF00ll) return fail(MOE_ERR_UNSUPPORTED, "router_topk: too many rows");
  if (!x || !Wr || !scores || (!indices && !indices32)) return fail(MOE_ERR_ARG, "router_topk: null pointer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(Wr) | reinterpret_cast<uintptr_t>(logits_out)) & 15)
    return fail(MOE_ERR_ARG, "router_topk: x, Wr and logits_out must be 16-byte aligned");
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  const int f16 = dtype == MOE_DTYPE_F16;
  const int BN = E > 128 ? 256 : 128;
  Params p;
  p.K = H; p.N = E; p.E = 1;
  p.num_n_tiles = 1;
  p.num_k_blocks = (H + BK - 1) / BK;
  p.status = status;
  p.f16 = f16;
  p.dense_rows = (int)T;
  p.r_scores = scores; p.r_idx64 = indices; p.r_idx32 = indices32; p.r_logits = logits_out;
  p.r_k = k; p.r_mode = mode;
  CUtensorMap tA, tB;
  rc = make_tmap(&tA, x, (uint64_t)H, (uint64_t)T, 0, (uint32_t)BM, f16);
  if (rc) return rc;
  rc = make_tmap(&tB, Wr, (uint64_t)H, (uint64_t)E, 1, (uint32_t)E, f16);    // only the E weight rows are fetched
  if (rc) return rc;
  p.b_tx_bytes = E * BK * 2;
  const int64_t tiles = (T + BM - 1) / BM;
  const int grid = (int)(tiles < dev.sm_count ? tiles : dev.sm_count);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (BN == 256) return launch<1, 256, EPI_ROUTER>(tA, tB, tB, p, grid, st);
  return launch<1, 128, EPI_ROUTER>(tA, tB, tB, p, grid, st);
}

int moe::grouped_gemm_scatter_slots(const void* A, const void* B, const int32_t* offsets, const int32_t* dst_rows,
                                    const float* row_w, int w_slots, void* Y, int64_t ldy, int64_t max_rows, int K, int N,
                                    int E, int dtype, int32_t* status, void* stream) {
  GatherArgs ga;
  ga.w_slots = w_slots;
  return grouped_gemm_impl(MOE_GEMM_SCALE_SCATTER_DSTW, A, B, nullptr, offsets, dst_rows, row_w, Y, ldy, max_rows, K, N, E,
                           status, stream, nullptr, nullptr, 0, 0, dtype, ga);
}

// One dense group: Y[rows, N] = epilogue(A[rows, K] . B[N, K]^T) without a device-side offsets table (declared in
// common.cuh; used for the shared expert of the single-call layer).
int moe::dense_gemm(int epilogue, const void* A, const void* B, const void* B2, int64_t rows, int K, int N, void* Y,
                    int64_t ldy, int dtype, int32_t* status, void* stream) {
  GatherArgs ga;
  ga.dense_rows = rows;
  return grouped_gemm_impl(epilogue, A, B, B2, nullptr, nullptr, nullptr, Y, ldy, rows, K, N, 1, status, stream, nullptr,
                           nullptr, 0, 0, dtype, ga);
}

// Y[T, S*N] fp32: slice s of the K dimension of A[T,K] . B[N,K]^T in columns [s*N, (s+1)*N) (declared in common.cuh).
// Split-K gives a skinny GEMM (few row tiles, long K) one tile per SM; the caller adds the S slices.
int moe::gemm_splitk_f32(const void* A, const void* B, int64_t T, int K, int N, int S, float* Y, int32_t* status,
                         void* stream, int dtype) {
  using namespace moe::gemm;
  if (T < 1 || N < 8 || N > 256 || (N % 8) || S < 1 || K < 8 || (K % 8) || (S > 1 && (K % (64 * S))))
    return fail(MOE_ERR_ARG, "gemm_splitk: bad shape T=%lld K=%d N=%d S=%d", (long long)T, K, N, S);
  if (T > 0x7FFFFF00ll) return fail(MOE_ERR_UNSUPPORTED, "gemm_splitk: too many rows");
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  const int f16 = dtype == MOE_DTYPE_F16;
  Params p;
  p.K = K; p.N = N; p.E = 1;
  p.num_n_tiles = S;
  p.num_k_blocks = (K / S + BK - 1) / BK;
  p.ksplit = S > 1;
  p.status = status;
  p.f16 = f16;
  p.dense_rows = (int)T;
  p.Y = Y; p.ldy = (int64_t)S * N;
  p.b_tx_bytes = N * BK * 2;
  CUtensorMap tA, tB;
  rc = make_tmap(&tA, A, (uint64_t)K, (uint64_t)T, 0, (uint32_t)BM, f16);
  if (rc) return rc;
  rc = make_tmap(&tB, B, (uint64_t)K, (uint64_t)N, 1, (uint32_t)N, f16);
  if (rc) return rc;
  const int64_t tiles = ((T + BM - 1) / BM) * S;
  const int grid = (int)(tiles < dev.sm_count ? tiles : dev.sm_count);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (N > 128) return launch<1, 256, MOE_GEMM_PLAIN_F32>(tA, tB, tB, p, grid, st);
  return launch<1, 128, MOE_GEMM_PLAIN_F32>(tA, tB, tB, p, grid, st);
}

extern "C" int moe_grouped_gemm_peer_scatter(const void* A, const void* B, const int32_t* offsets,
                                             const int32_t* row_rank, const int32_t* dst_rows, void* const* peer_base,
                                             int n_peers, int64_t ldy, int64_t max_rows, int64_t expected_rows,
                                             int K, int N, int E, int dtype, int32_t* status, void* stream) {
  using namespace moe;
  if (!row_rank || !dst_rows || !peer_base) return fail(MOE_ERR_ARG, "grouped_gemm_peer_scatter: null table");
  if (n_peers < 1 || n_peers > 16) return fail(MOE_ERR_ARG, "grouped_gemm_peer_scatter: n_peers=%d out of range", n_peers);
  for (int g = 0; g < n_peers; ++g)
    if (!peer_base[g] || (reinterpret_cast<uintptr_t>(peer_base[g]) & 15))
      return fail(MOE_ERR_ARG, "grouped_gemm_peer_scatter: peer buffer %d null or unaligned", g);
  return grouped_gemm_impl(MOE_GEMM_PLAIN, A, B, nullptr, offsets, dst_rows, nullptr, peer_base[0], ldy, max_rows, K, N, E,
                           status, stream, row_rank, peer_base, n_peers, expected_rows, dtype);
}

static int grouped_gemm_impl(int epilogue, const void* A, const void* B, const void* B2, const int32_t* offsets,
                             const int32_t* dst_rows, const float* row_w, void* Y, int64_t ldy, int64_t max_rows,
                             int K, int N, int E, int32_t* status, void* stream, const int32_t* row_rank,
                             void* const* peer_base, int n_peers, int64_t expected_rows, int dtype,
                             const GatherArgs& ga) {
  using namespace moe;
  using namespace moe::gemm;
  if (dtype != MOE_DTYPE_BF16 && dtype != MOE_DTYPE_F16) return fail(MOE_ERR_ARG, "grouped_gemm: unknown dtype %d", dtype);
  const int f16 = dtype == MOE_DTYPE_F16;
  // rows the caller expects to be live (<= max_rows, which may be a buffer capacity): steers the tile rule
  const int64_t live_rows = (expected_rows > 0 && expected_rows < max_rows) ? expected_rows : max_rows;
  if (epilogue < 0 || epilogue > 4) return fail(MOE_ERR_ARG, "grouped_gemm: unknown epilogue %d", epilogue);
  const int w_by_dst = epilogue == MOE_GEMM_SCALE_SCATTER_DSTW;
  if (w_by_dst) {
    if (!dst_rows) return fail(MOE_ERR_ARG, "grouped_gemm: SCALE_SCATTER_DSTW needs dst_rows");
    epilogue = MOE_GEMM_SCALE_SCATTER;
  }
  if (max_rows < 0 || K < 8 || N < 8 || (K % 8) || (N % 8) || E < 1)
    return fail(MOE_ERR_ARG, "grouped_gemm: bad shape rows=%lld K=%d N=%d E=%d (K, N multiples of 8)", (long long)max_rows, K, N, E);
  if (E > MAX_E) return fail(MOE_ERR_UNSUPPORTED, "grouped_gemm: E=%d exceeds %d", E, MAX_E);
  if (max_rows == 0) return MOE_OK;
  if (max_rows > 0x7FFFFF00ll) return fail(MOE_ERR_UNSUPPORTED, "grouped_gemm: too many rows");
  if (!A || !B || !Y || (!offsets && !(ga.dense_rows > 0 && E == 1))) return fail(MOE_ERR_ARG, "grouped_gemm: null pointer");
  if (epilogue == MOE_GEMM_SILU_GATE && !B2) return fail(MOE_ERR_ARG, "grouped_gemm: SILU_GATE needs the up weight");
  if (epilogue == MOE_GEMM_SCALE_SCATTER && !row_w) return fail(MOE_ERR_ARG, "grouped_gemm: SCALE_SCATTER needs row weights");
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(B2) |
       reinterpret_cast<uintptr_t>(Y)) & 15)
    return fail(MOE_ERR_ARG, "grouped_gemm: pointers must be 16-byte aligned");
  const int out_elem = epilogue == MOE_GEMM_PLAIN_F32 ? 4 : 2;
  if (ldy < N || (ldy * out_elem) % 16) return fail(MOE_ERR_ARG, "grouped_gemm: ldy=%lld must be >= N and 16-byte aligned", (long long)ldy);
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;

  // Tile shape: a fixed rule on the problem size.  The CTA-pair kernel (256-row and 128-row tiles under
  // cta_group::2, half the B staging per SM) is the default once there is enough work for every SM pair;
  // smaller problems and narrow outputs take the single-CTA kernel with 128-row tiles, which spreads few
  // tiles over twice as many independent CTAs.  MOE_B200_GEMM_TILE_ROWS = "128" | "pair" overrides (tests, measurement).
  const bool gate = epilogue == MOE_GEMM_SILU_GATE;
  const int n_tiles_256 = gate ? (N + 127) / 128 : (N + 255) / 256;
  const int64_t m_tiles_128 = live_rows / BM + E, m_tiles_256 = live_rows / (2 * BM) + E;
  int BN = 128;
  if (gate || (N % 256 == 0 && m_tiles_128 * n_tiles_256 >= dev.sm_count)) BN = 256;
  // the pair kernel reads its A rows through TMA only: a row gather by cp.async needs a relay from the second CTA to the
  // leader's barrier (measured: 15 % behind the 128-row kernel with a relaxed arrive, 2.4x behind with a releasing one)
  const bool pair_ok = (gate ? N % 64 == 0 : N % 256 == 0) && epilogue != MOE_GEMM_PLAIN_F32 && !ga.idx;
  // measured on B200 under its power cap: the pair kernel gains 3-10 % where groups are uniformly large and loses
  // where most experts own a single tile (their weight stream wants the deeper per-SM ring of the single-CTA kernel)
  bool pair = pair_ok && live_rows / E >= 512 && (live_rows / (2 * BM)) * n_tiles_256 * 2 >= (int64_t)dev.sm_count;
  if (const char* force = getenv("MOE_B200_GEMM_TILE_ROWS")) {
    if (force[0] == 'p') pair = pair_ok;
    else if (atoi(force) == 128) pair = false;
  }
  const int out_cols = gate ? BN / 2 : BN;

  Params p;
  p.offsets = offsets; p.dst_rows = dst_rows; p.row_w = row_w; p.Y = Y; p.ldy = ldy;
  p.K = K; p.N = N; p.E = E;
  p.num_n_tiles = pair ? n_tiles_256 : (N + out_cols - 1) / out_cols;
  p.num_k_blocks = (K + BK - 1) / BK;
  p.status = status;
  p.f16 = f16;
  p.row_rank = row_rank;
  for (int g = 0; g < 16; ++g) p.peer_base[g] = (peer_base && g < n_peers) ? peer_base[g] : nullptr;
  p.w_by_dst = w_by_dst;
  p.w_slots = ga.w_slots;
  p.y_rows = max_rows;     // a scatter permutes the sorted rows: the output has as many rows as the sorted input
  p.dense_rows = (int)ga.dense_rows;
  p.a_gather = ga.idx; p.a_src = A; p.a_div = ga.div; p.a_src_rows = (int)ga.src_rows; p.a_rows = (int)max_rows;
  // measured on the DeepSeek-V3-shaped layer: eviction hints on the weight loads 3 % of the step, the mixed tile order
  // another 1-3 % of each GEMM; MOE_B200_L2_HINTS / MOE_B200_MIXED = 0 switch them off for such measurements
  static const int env_hints = [] { const char* h = getenv("MOE_B200_L2_HINTS"); return h ? atoi(h) : 2; }();
  static const int env_mixed = [] { const char* h = getenv("MOE_B200_MIXED"); return h ? atoi(h) : 1; }();
  // measured on the DeepSeek-V3-shaped layer, ten alternating runs of 20 steps: 7.56 -> 7.29 ms per step (-3.6 %) and the
  // median SM clock of the power-capped steps back at its maximum; MOE_B200_M64=0 switches it off for such comparisons
  static const int env_m64 = [] { const char* h = getenv("MOE_B200_M64"); return h ? atoi(h) : 1; }();
  p.m64 = env_m64;
  p.l2_hints = env_hints;
  p.mixed = env_mixed && offsets != nullptr;

  CUtensorMap tA, tA64, tB, tB2;
  // with a row gather A is the un-permuted matrix (src_rows rows) and its tensor maps are never used by the kernel
  const uint64_t a_map_rows = ga.idx ? (uint64_t)ga.src_rows : (uint64_t)max_rows;
  rc = make_tmap(&tA, A, (uint64_t)K, a_map_rows, 0, (uint32_t)BM, f16);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (pair) {
    rc = make_tmap(&tA64, A, (uint64_t)K, a_map_rows, 0, (uint32_t)(BM / 2), f16);
    if (rc) return rc;
    // a CTA of the pair stages 128 of the 256 N rows: one box, or a 64-row gate box and a 64-row up box
    const uint32_t box = gate ? 64u : 128u;
    rc = make_tmap(&tB, B, (uint64_t)K, (uint64_t)N, (uint64_t)E, box, f16);
    if (rc) return rc;
    tB2 = tB;
    if (gate) {
      rc = make_tmap(&tB2, B2, (uint64_t)K, (uint64_t)N, (uint64_t)E, box, f16);
      if (rc) return rc;
    }
    const int64_t units = m_tiles_256 * p.num_n_tiles;
    int pgrid = (int)(2 * units < dev.sm_count ? 2 * units : dev.sm_count) & ~1;
    if (pgrid < 2) pgrid = 2;
    if (row_rank) return launch_pair<EPI_PEER>(tA, tA64, tB, tB2, p, pgrid, st);
    switch (epilogue) {
      case MOE_GEMM_PLAIN: return launch_pair<MOE_GEMM_PLAIN>(tA, tA64, tB, tB2, p, pgrid, st);
      case MOE_GEMM_SCALE_SCATTER: return launch_pair<MOE_GEMM_SCALE_SCATTER>(tA, tA64, tB, tB2, p, pgrid, st);
      default: return launch_pair<MOE_GEMM_SILU_GATE>(tA, tA64, tB, tB2, p, pgrid, st);
    }
  }
  uint32_t b_box_rows = (uint32_t)out_cols;
  // fewer weight rows than tile columns: fetch only those (the rest of the B stage keeps whatever it held; the
  // accumulator columns it feeds are never stored)
  if (!gate && N < out_cols) b_box_rows = (uint32_t)N;
  p.b_tx_bytes = (int)b_box_rows * BK * 2 * (gate ? 2 : 1);
  rc = make_tmap(&tB, B, (uint64_t)K, (uint64_t)N, (uint64_t)E, b_box_rows, f16);
  if (rc) return rc;
  tB2 = tB;
  if (gate) {
    rc = make_tmap(&tB2, B2, (uint64_t)K, (uint64_t)N, (uint64_t)E, b_box_rows, f16);
    if (rc) return rc;
  }
  const int64_t tiles_bound = m_tiles_128 * p.num_n_tiles;
  int grid = (int)(tiles_bound < dev.sm_count ? tiles_bound : dev.sm_count);
  if (grid < 1) grid = 1;
  if (row_rank) {   // combine exchange fused into the epilogue
    if (BN == 256) return launch<1, 256, EPI_PEER>(tA, tB, tB2, p, grid, st);
    return launch<1, 128, EPI_PEER>(tA, tB, tB2, p, grid, st);
  }
#define MOE_GEMM_CASE(EPI_)                                                                  \
  if (BN == 256) return launch<1, 256, EPI_>(tA, tB, tB2, p, grid, st);                        \
  return launch<1, 128, EPI_>(tA, tB, tB2, p, grid, st)
  switch (epilogue) {
    case MOE_GEMM_PLAIN: MOE_GEMM_CASE(MOE_GEMM_PLAIN);
    case MOE_GEMM_SCALE_SCATTER: MOE_GEMM_CASE(MOE_GEMM_SCALE_SCATTER);
    case MOE_GEMM_PLAIN_F32: MOE_GEMM_CASE(MOE_GEMM_PLAIN_F32);
    default: return launch<1, 256, MOE_GEMM_SILU_GATE>(tA, tB, tB2, p, grid, st);
  }
#undef MOE_GEMM_CASE
}

// Exercises the bounded barrier wait of the GEMM kernels on purpose: one warp waits, with the given limit, on an
// mbarrier that nothing ever arrives on.  The wait runs out, records {ST_WAIT_TIMEOUT, 99, block} in status and the
// kernel returns normally - the same path a GEMM takes when a copy it waits for never lands.  Nothing faults or hangs.
namespace moe {
namespace gemm {
__global__ void __launch_bounds__(32) wait_probe_kernel(unsigned long long limit_ns, int32_t* status, int32_t* outcome) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, 99, limit_ns);
  if (threadIdx.x == 0 && outcome) *outcome = ok ? 1 : 0;
}
}  // namespace gemm
}  // namespace moe

int moe::bounds_status_gemm(int32_t* out3, cudaStream_t st) { return moe::bounds_status_read(out3, st); }

extern "C" int moe_debug_wait_probe(int64_t limit_us, int32_t* status, int32_t* outcome, void* stream) {
  using namespace moe;
  if (limit_us < 1 || limit_us > 1000000) return fail(MOE_ERR_ARG, "wait_probe: limit_us=%lld outside [1, 1000000]", (long long)limit_us);
  if (!status) return fail(MOE_ERR_ARG, "wait_probe: null status");
  gemm::wait_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>((unsigned long long)limit_us * 1000ull, status, outcome);
  MOE_CHECK_LAUNCH("wait_probe_kernel");
  return MOE_OK;
}

#ifdef MOE_GEMM_TRACE
// tile_ns: 3 x MOE_TRACE_MAX_TILES uint64, tile_cta: MOE_TRACE_MAX_TILES int32, cta_clk: MOE_TRACE_MAX_CTAS x 4 int64
// (host buffers); the stamps of the most recent launch of the 128-row kernel on the current device.
extern "C" int moe_gemm_trace_read(unsigned long long* tile_ns, int* tile_cta, long long* cta_clk) {
  using namespace moe;
  MOE_CUDA_CHECK(cudaDeviceSynchronize());
  MOE_CUDA_CHECK(cudaMemcpyFromSymbol(tile_ns, g_trace_tile, sizeof(unsigned long long) * 3 * MOE_TRACE_MAX_TILES));
  MOE_CUDA_CHECK(cudaMemcpyFromSymbol(tile_cta, g_trace_cta, sizeof(int) * MOE_TRACE_MAX_TILES));
  MOE_CUDA_CHECK(cudaMemcpyFromSymbol(cta_clk, g_trace_clk, sizeof(long long) * 4 * MOE_TRACE_MAX_CTAS));
  return MOE_OK;
}
#endif
