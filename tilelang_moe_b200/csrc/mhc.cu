// mHC pre / post blocks (the operators on either side of the MoE layer in the model the reference targets).
//
//   pre :  mixes = (residual_flat . fn^T) * rsqrt(mean(residual_flat^2) + eps) * scale + base      [T, 2*hc + hc*hc]
//          pre_mix = sigmoid(mixes[:hc]) + eps, post_mix = sigmoid(mixes[hc:2hc]) * mult,
//          comb_mix = Sinkhorn(mixes[2hc:].view(hc, hc)), layer_input = sum_m pre_mix[m] * residual[m]   (bf16)
//   post:  out[m] = x * post_mix[m] + sum_j comb_mix[j][m] * residual[j]                                  (bf16)
//
// The skinny GEMM (T x hc*hidden x 24) runs on the tensor cores in bf16 without giving up fp32 accuracy: the
// fp32 matrix fn is split once into three bf16 matrices hi + mid + lo (24 mantissa bits between them), stacked
// as 3*24 weight rows; residual is bf16 already, so every product is exact and the sums are fp32.  Few row
// tiles and a long K: the GEMM is split along K so that every SM gets a tile, and the finishing kernel adds
// the slices.  The finishing kernel keeps the token's residual row in shared memory: one read of it serves
// the sum of squares and, once the mixes are known, the weighted sum of the hc streams.
#include "common.cuh"

#include <cuda_bf16.h>

namespace moe {

__global__ void __launch_bounds__(256)
mhc_split_weights_kernel(const float* __restrict__ fn, int rows, int64_t K, __nv_bfloat16* __restrict__ fn3) {
  const int64_t n = (int64_t)rows * K;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
    const float v = fn[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(mid);
    fn3[i] = hi;
    fn3[n + i] = mid;
    fn3[2 * n + i] = __float2bfloat16_rn(r2);
  }
}

__device__ __forceinline__ float sigmoidf(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 p = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[j]));
    f[2 * j] = p.x;
    f[2 * j + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  uint32_t* u = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    u[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  return o;
}

// One CTA per token.  part: [T, S, 3, R] fp32 slices of the split GEMM (R = 2*HC + HC*HC).
template <int HC>
__global__ void __launch_bounds__(256)
mhc_pre_finish_kernel(const uint4* __restrict__ residual, const float* __restrict__ part, int S,
                      const float* __restrict__ hc_scale, const float* __restrict__ hc_base, int hidden_vecs,
                      float rms_eps, float pre_eps, float sk_eps, float post_mult, int repeat,
                      float* __restrict__ post_mix, float* __restrict__ comb_mix, uint4* __restrict__ layer_input) {
  constexpr int R = 2 * HC + HC * HC;
  extern __shared__ uint4 row[];                 // the token's HC x hidden residual row
  __shared__ float red[8];
  __shared__ float mix[R];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t t = blockIdx.x;
  const int vecs = HC * hidden_vecs;
  const uint4* src = residual + t * vecs;
  float ss = 0.f;
  // eight independent 16-byte loads per thread in flight (a whole 32 KB row per pass of the CTA): the kernel is
  // a stream of the residual
  for (int v0 = tid; v0 < vecs; v0 += 8 * 256) {
    uint4 x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (v0 + u * 256 < vecs) x[u] = __ldg(src + v0 + u * 256);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (v0 + u * 256 < vecs) {
        row[v0 + u * 256] = x[u];
        float f[8];
        unpack8(x[u], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
      }
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  float m = 0.f;                      // the GEMM slices of this thread's mix, fetched before the barrier
  if (tid < R) {
    const float* pp = part + t * (int64_t)(S * 3 * R);
    for (int s = 0; s < S; ++s) m += (pp[(s * 3 + 0) * R + tid] + pp[(s * 3 + 1) * R + tid]) + pp[(s * 3 + 2) * R + tid];
  }
  __syncthreads();
  if (tid < R) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += red[w];
    const float rms = rsqrtf(total / (float)(vecs * 8) + rms_eps);
    const float sc = tid < HC ? hc_scale[0] : (tid < 2 * HC ? hc_scale[1] : hc_scale[2]);
    mix[tid] = m * rms * sc + hc_base[tid];
  }
  __syncthreads();
  if (tid < HC) post_mix[t * HC + tid] = sigmoidf(mix[HC + tid]) * post_mult;
  // weighted sum of the hc streams from the cached row (every thread evaluates the hc gate values itself: no
  // second barrier), then one warp runs the Sinkhorn iteration while the others are already done
  float pm[HC];
#pragma unroll
  for (int m = 0; m < HC; ++m) pm[m] = sigmoidf(mix[m]) + pre_eps;
  uint4* dst = layer_input + t * hidden_vecs;
  for (int v = tid; v < hidden_vecs; v += 256) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int m = 0; m < HC; ++m) {
      float f[8];
      unpack8(row[m * hidden_vecs + v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j] * pm[m];      // the reference multiplies, then sums over the streams
    }
    dst[v] = pack8(acc);
  }
  if (warp == 7 && lane < HC * HC) {
    // Sinkhorn on the HC x HC block: lane = i*HC + j; rows are groups of HC neighbouring lanes, columns stride HC
    const unsigned mask = HC * HC == 32 ? 0xFFFFFFFFu : ((1u << (HC * HC)) - 1u);
    float x = mix[2 * HC + lane];
    float mx = x;
#pragma unroll
    for (int o = 1; o < HC; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(mask, mx, o));
    x = expf(x - mx);
    float rs = x;
#pragma unroll
    for (int o = 1; o < HC; o <<= 1) rs += __shfl_xor_sync(mask, rs, o);
    x = x / rs + sk_eps;
    float cs = x;
#pragma unroll
    for (int o = HC; o < HC * HC; o <<= 1) cs += __shfl_xor_sync(mask, cs, o);
    x = x / (cs + sk_eps);
    for (int it = 1; it < repeat; ++it) {
      rs = x;
#pragma unroll
      for (int o = 1; o < HC; o <<= 1) rs += __shfl_xor_sync(mask, rs, o);
      x = x / (rs + sk_eps);
      cs = x;
#pragma unroll
      for (int o = HC; o < HC * HC; o <<= 1) cs += __shfl_xor_sync(mask, cs, o);
      x = x / (cs + sk_eps);
    }
    comb_mix[t * (HC * HC) + lane] = x;
  }
}

// One CTA per token: out[m] = x * post[m] + sum_j comb[j][m] * residual[j]
template <int HC>
__global__ void __launch_bounds__(256)
mhc_post_kernel(const uint4* __restrict__ x, const uint4* __restrict__ residual, const float* __restrict__ post,
                const float* __restrict__ comb, int hidden_vecs, uint4* __restrict__ out) {
  const int64_t t = blockIdx.x;
  float pm[HC], cm[HC][HC];
#pragma unroll
  for (int m = 0; m < HC; ++m) pm[m] = post[t * HC + m];
#pragma unroll
  for (int j = 0; j < HC; ++j)
#pragma unroll
    for (int m = 0; m < HC; ++m) cm[j][m] = comb[t * (HC * HC) + j * HC + m];
  const uint4* xr = x + t * hidden_vecs;
  const uint4* rr = residual + t * (int64_t)(HC * hidden_vecs);
  uint4* orow = out + t * (int64_t)(HC * hidden_vecs);
  for (int v = threadIdx.x; v < hidden_vecs; v += 256) {
    float xf[8];
    unpack8(__ldg(xr + v), xf);
    float acc[HC][8];
#pragma unroll
    for (int m = 0; m < HC; ++m)
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[m][q] = xf[q] * pm[m];
    // the reference adds term1 to the finished matrix product: keep that association
    float mm[HC][8];
#pragma unroll
    for (int m = 0; m < HC; ++m)
#pragma unroll
      for (int q = 0; q < 8; ++q) mm[m][q] = 0.f;
#pragma unroll
    for (int j = 0; j < HC; ++j) {
      float rf[8];
      unpack8(__ldg(rr + j * hidden_vecs + v), rf);
#pragma unroll
      for (int m = 0; m < HC; ++m)
#pragma unroll
        for (int q = 0; q < 8; ++q) mm[m][q] = fmaf(cm[j][m], rf[q], mm[m][q]);
    }
#pragma unroll
    for (int m = 0; m < HC; ++m) {
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[m][q] += mm[m][q];
      orow[m * hidden_vecs + v] = pack8(acc[m]);
    }
  }
}

static int mhc_splits(int64_t T, int64_t K) {
  // K slices: enough tiles for every SM of a 148-SM part (the rule may not depend on the device: the
  // workspace size is derived from it), K divisible into whole 64-element blocks per slice
  const int64_t row_tiles = (T + 127) / 128;
  int S = 1;
  while (S < 16 && row_tiles * S * 2 <= 148 && K % (64 * (S * 2)) == 0 && K / (S * 2) >= 512) S *= 2;   // one wave of tiles
  return S;
}

}  // namespace moe

extern "C" size_t moe_mhc_pre_workspace(int64_t T, int hc_mult, int64_t hidden) {
  if (T < 1 || hc_mult < 1 || hidden < 1) return 0;
  const int R = 2 * hc_mult + hc_mult * hc_mult;
  return (size_t)T * moe::mhc_splits(T, (int64_t)hc_mult * hidden) * 3 * R * sizeof(float);
}

extern "C" int moe_mhc_split_weights(const float* fn, int rows, int64_t K, void* fn3, void* stream) {
  using namespace moe;
  if (!fn || !fn3) return fail(MOE_ERR_ARG, "mhc_split_weights: null pointer");
  if (rows < 1 || K < 1) return fail(MOE_ERR_ARG, "mhc_split_weights: bad shape rows=%d K=%lld", rows, (long long)K);
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  int64_t blocks = ceil_div64((int64_t)rows * K, 256);
  if (blocks > (int64_t)dev.sm_count * 8) blocks = (int64_t)dev.sm_count * 8;
  mhc_split_weights_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      fn, rows, K, reinterpret_cast<__nv_bfloat16*>(fn3));
  MOE_CHECK_LAUNCH("mhc_split_weights_kernel");
  return MOE_OK;
}

extern "C" int moe_mhc_pre(const void* residual, const void* fn3, const float* hc_scale, const float* hc_base, int64_t T,
                           int hc_mult, int64_t hidden, float rms_eps, float hc_pre_eps, float hc_sinkhorn_eps,
                           float hc_post_mult_value, int sinkhorn_repeat, void* ws, size_t ws_bytes, float* post_mix,
                           float* comb_mix, void* layer_input, int32_t* status, void* stream) {
  using namespace moe;
  if (T < 0 || hidden < 8 || hidden % 8) return fail(MOE_ERR_ARG, "mhc_pre: bad shape T=%lld hidden=%lld", (long long)T, (long long)hidden);
  if (hc_mult != 2 && hc_mult != 4) return fail(MOE_ERR_UNSUPPORTED, "mhc_pre: hc_mult=%d (2 and 4 are built)", hc_mult);
  if (sinkhorn_repeat < 1) return fail(MOE_ERR_ARG, "mhc_pre: sinkhorn_repeat=%d", sinkhorn_repeat);
  if (T == 0) return MOE_OK;
  if (!residual || !fn3 || !hc_scale || !hc_base || !post_mix || !comb_mix || !layer_input || !ws)
    return fail(MOE_ERR_ARG, "mhc_pre: null pointer");
  if ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(fn3) | reinterpret_cast<uintptr_t>(ws) |
       reinterpret_cast<uintptr_t>(layer_input)) & 15)
    return fail(MOE_ERR_ARG, "mhc_pre: residual, fn3, ws and layer_input must be 16-byte aligned");
  const int64_t K = (int64_t)hc_mult * hidden;
  if (K > 0x7FFFFFFFll) return fail(MOE_ERR_UNSUPPORTED, "mhc_pre: hc_mult*hidden too large");
  const size_t row_bytes = (size_t)K * 2;
  if (row_bytes > 200 * 1024) return fail(MOE_ERR_UNSUPPORTED, "mhc_pre: hc_mult*hidden=%lld exceeds the shared-memory row cache", (long long)K);
  const int R = 2 * hc_mult + hc_mult * hc_mult;
  const int S = mhc_splits(T, K);
  if (ws_bytes < (size_t)T * S * 3 * R * sizeof(float)) return fail(MOE_ERR_ARG, "mhc_pre: workspace too small");
  int rc = gemm_splitk_f32(residual, fn3, T, (int)K, 3 * R, S, reinterpret_cast<float*>(ws), status, stream);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define MOE_MHC_PRE(HC_)                                                                                              \
  do {                                                                                                                \
    if (row_bytes > 48 * 1024)                                                                                        \
      MOE_CUDA_CHECK(cudaFuncSetAttribute(mhc_pre_finish_kernel<HC_>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                          (int)row_bytes));                                                           \
    mhc_pre_finish_kernel<HC_><<<(unsigned)T, 256, row_bytes, st>>>(                                                   \
        reinterpret_cast<const uint4*>(residual), reinterpret_cast<const float*>(ws), S, hc_scale, hc_base,           \
        (int)(hidden / 8), rms_eps, hc_pre_eps, hc_sinkhorn_eps, hc_post_mult_value, sinkhorn_repeat, post_mix,       \
        comb_mix, reinterpret_cast<uint4*>(layer_input));                                                             \
  } while (0)
  if (hc_mult == 4) MOE_MHC_PRE(4); else MOE_MHC_PRE(2);
#undef MOE_MHC_PRE
  MOE_CHECK_LAUNCH("mhc_pre_finish_kernel");
  return MOE_OK;
}

extern "C" int moe_mhc_post(const void* x, const void* residual, const float* post_layer_mix, const float* comb_res_mix,
                            int64_t T, int hc_mult, int64_t hidden, void* out, void* stream) {
  using namespace moe;
  if (T < 0 || hidden < 8 || hidden % 8) return fail(MOE_ERR_ARG, "mhc_post: bad shape T=%lld hidden=%lld", (long long)T, (long long)hidden);
  if (hc_mult != 2 && hc_mult != 4) return fail(MOE_ERR_UNSUPPORTED, "mhc_post: hc_mult=%d (2 and 4 are built)", hc_mult);
  if (T == 0) return MOE_OK;
  if (T > 0x7FFFFFFFll) return fail(MOE_ERR_UNSUPPORTED, "mhc_post: too many tokens");
  if (!x || !residual || !post_layer_mix || !comb_res_mix || !out) return fail(MOE_ERR_ARG, "mhc_post: null pointer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(MOE_ERR_ARG, "mhc_post: x, residual and out must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (hc_mult == 4)
    mhc_post_kernel<4><<<(unsigned)T, 256, 0, st>>>(reinterpret_cast<const uint4*>(x), reinterpret_cast<const uint4*>(residual),
                                                    post_layer_mix, comb_res_mix, (int)(hidden / 8), reinterpret_cast<uint4*>(out));
  else
    mhc_post_kernel<2><<<(unsigned)T, 256, 0, st>>>(reinterpret_cast<const uint4*>(x), reinterpret_cast<const uint4*>(residual),
                                                    post_layer_mix, comb_res_mix, (int)(hidden / 8), reinterpret_cast<uint4*>(out));
  MOE_CHECK_LAUNCH("mhc_post_kernel");
  return MOE_OK;
}
