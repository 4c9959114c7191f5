// Shared host/device helpers for the moe_b200 library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/moe_b200.h"

namespace moe {

// Thread-local message for the last failing call (returned by moe_last_error()).
char* last_error_buffer();
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define MOE_CUDA_CHECK(expr)                                  \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::moe::cuda_fail(_e, #expr); \
  } while (0)

#define MOE_CHECK_LAUNCH(name)                                       \
  do {                                                               \
    cudaError_t _e = cudaGetLastError();                             \
    if (_e != cudaSuccess) return ::moe::cuda_fail(_e, name);        \
  } while (0)

// Cached per-device attributes.
struct DeviceInfo {
  int sm_count;
  int cc_major;
  int cc_minor;
  int max_smem_optin;
};
int current_device_info(DeviceInfo* out);

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Device status codes written to status[0]; status[1..3] carry detail.
enum : int {
  ST_OK = 0,
  ST_BAD_EXPERT_ID = 1,     // an expert id outside [0,E) was seen
  ST_WAIT_TIMEOUT = 2,      // a bounded barrier wait gave up; status[1] = site
  ST_INTERNAL = 3,
  ST_BAD_INDEX = 4,         // checked build only: an index-driven access outside its buffer was skipped
};

// ---- index checks of the checked build (-DMOE_BOUNDS_CHECK) ---------------------
// Every store or load whose row comes out of an index table (scatter destinations and gather sources of the grouped
// GEMMs, the row table of the combine) is compared with the size of its buffer first.  An index outside it is not
// followed: the access is skipped, and {ST_BAD_INDEX, site, index} is left in a status block of the translation unit
// (read and cleared by moe_debug_bounds_status).  Sites: 1 GEMM scatter destination, 2 GEMM gather source, 3 combine
// row table.  The normal build compiles the checks away.
#ifdef MOE_BOUNDS_CHECK
static __device__ int32_t g_bounds_status[4];
__device__ __forceinline__ bool moe_index_ok(int64_t i, int64_t n, int site) {
  if (i >= 0 && i < n) return true;
  if (atomicCAS(&g_bounds_status[0], 0, (int)ST_BAD_INDEX) == 0) { g_bounds_status[1] = site; g_bounds_status[2] = (int32_t)i; }
  return false;
}
#define MOE_INDEX_OK(i, n, site) ::moe::moe_index_ok((int64_t)(i), (int64_t)(n), (site))
// host side of one translation unit: copy the block out (after the stream's work) and clear it
static inline int bounds_status_read(int32_t* out3, cudaStream_t st) {
  int32_t h[4] = {0, 0, 0, 0};
  const int32_t zero[4] = {0, 0, 0, 0};
  MOE_CUDA_CHECK(cudaStreamSynchronize(st));
  MOE_CUDA_CHECK(cudaMemcpyFromSymbol(h, g_bounds_status, sizeof(h)));
  MOE_CUDA_CHECK(cudaMemcpyToSymbol(g_bounds_status, zero, sizeof(zero)));
  out3[0] = h[0]; out3[1] = h[1]; out3[2] = h[2];
  return MOE_OK;
}
#else
#define MOE_INDEX_OK(i, n, site) true
static inline int bounds_status_read(int32_t* out3, cudaStream_t) { out3[0] = out3[1] = out3[2] = 0; return MOE_OK; }
#endif
int bounds_status_gemm(int32_t* out3, cudaStream_t st);     // gemm_sm100.cu
int bounds_status_route(int32_t* out3, cudaStream_t st);    // route.cu

// ---- order-preserving float <-> uint32 key -----------------------------------
// Larger float -> larger key.  -0.0 is folded into +0.0 and every NaN maps to the
// top key, so that key equality is exactly "compares equal in a descending sort
// that ranks NaN first".
__device__ __forceinline__ uint32_t float_to_key(float x) {
  if (x != x) return 0xFFFFFFFFu;
  if (x == 0.0f) x = 0.0f;
  uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  uint32_t b = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(b);
}

// Signed-integer keys ordered like the floats (thread-per-row selection lists): x + 0.0f folds -0.0 into +0.0 and
// every NaN into the canonical positive NaN, which ranks above +inf.
__device__ __forceinline__ int float_to_ikey(float x) {
  const int b = __float_as_int(x + 0.0f);
  return b ^ ((b >> 31) & 0x7FFFFFFF);
}
__device__ __forceinline__ float ikey_to_float(int k) { return __int_as_float(k ^ ((k >> 31) & 0x7FFFFFFF)); }

template <int K>
__device__ __forceinline__ void list_insert(int (&kv)[K], int (&ki)[K], int ck, int ci) {
  // shift chain: the candidate enters at the first entry it strictly exceeds (equal keys keep the earlier column
  // ahead); from there on every entry moves down one place, so entries that tie with each other keep their order
  bool p = false;
#pragma unroll
  for (int j = 0; j < K; ++j) {
    p = p || (ck > kv[j]);
    const int tv = kv[j], ti = ki[j];
    kv[j] = p ? ck : tv;
    ki[j] = p ? ci : ti;
    ck = p ? tv : ck;
    ci = p ? ti : ci;
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// tcgen05 router GEMM whose epilogue does top-k + softmax per row (gemm_sm100.cu); E <= 256, E % 8 == 0, k <= 8
int router_topk_gemm(const void* x, const void* Wr, int64_t T, int H, int E, int k, int mode, int dtype, float* scores,
                     int64_t* indices, int32_t* indices32, float* logits_out, int32_t* status, void* stream);

// split-K GEMM with fp32 slices (gemm_sm100.cu): Y[T, S*N], N <= 256, K % (64*S) == 0
int gemm_splitk_f32(const void* A, const void* B, int64_t T, int K, int N, int S, float* Y, int32_t* status, void* stream,
                    int dtype = MOE_DTYPE_BF16);

// dense single-group GEMM through the grouped kernel, no offsets table on the device (gemm_sm100.cu)
int dense_gemm(int epilogue, const void* A, const void* B, const void* B2, int64_t rows, int K, int N, void* Y,
               int64_t ldy, int dtype, int32_t* status, void* stream);

// moe_route_histogram over a virtual id list: every kx stored ids are followed by one entry of expert E - 1 (route.cu)
int route_histogram_ex(const void* topk_idx, int idx_is_int64, int64_t n, int E, const int32_t* id_map, int32_t* counts,
                       int32_t* offsets, int32_t* perm, int32_t* inv, void* ws, size_t ws_bytes, int32_t* status,
                       void* stream, int kx);

// moe_grouped_gemm(MOE_GEMM_SCALE_SCATTER_DSTW) whose destination rows come in runs of w_slots + 1 per token: the
// first w_slots of a run read row_w[token * w_slots + slot], the last one (the shared expert's row) weighs 1 (gemm_sm100.cu)
int grouped_gemm_scatter_slots(const void* A, const void* B, const int32_t* offsets, const int32_t* dst_rows,
                               const float* row_w, int w_slots, void* Y, int64_t ldy, int64_t max_rows, int K, int N, int E,
                               int dtype, int32_t* status, void* stream);

// K slices of the few-token router GEMM (route.cu): 1..16 from the token count and the hidden size alone
int router_splits(int64_t T, int H);

}  // namespace moe
