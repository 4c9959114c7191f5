// Measurement tool, not part of the library: throughput of tcgen05.mma shapes with operands resident in shared memory,
// and the place cta_group::2 M=128 accumulators take in tensor memory.  Built and run by
// `python -m tilelang_moe_b200.probe_mma [rates|layout]`; the figures it prints on a B200 are what the tile shapes of
// the grouped GEMM were chosen from (clocks per K=16 step are counted with clock64, so they do not depend on the
// clock the power cap allows).  Every wait is bounded.
#include <cstdio>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0; d |= (uint64_t)((saddr & 0x3FFFFu) >> 4); d |= (uint64_t)1 << 16; d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46; d |= (uint64_t)2 << 61; return d;
}
__host__ __device__ constexpr uint32_t idesc(int m, int n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }
template <int CG> __device__ __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t acc) {
  if (CG == 1) asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(id), "r"(acc) : "memory");
  else asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(id), "r"(acc) : "memory");
}
template <int CG> __device__ __forceinline__ void commit(uint32_t bar) {
  if (CG == 1) asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  else asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done;
}
// mode: 0 = one MMA (M, N) per step, same D; 1 = two MMAs per step: (A0,B)->D0, (A1,B)->D1 (swapped-operand light tile);
// 2 = two MMAs per step into the same D columns shifted (A0,B)->D0 then (A0,B)->D0 (dependency test)
template <int CG>
__global__ void __launch_bounds__(128, 1) k(int n, int mode, int steps, long long* out, int m) {
  extern __shared__ unsigned char dyn[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)dyn + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar; __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += 128) {
    uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u; h ^= h >> 13; h *= 0x5bd1e995u; h ^= h >> 15;
    ((uint32_t*)smem)[i] = (h & 0x83FF83FFu) | 0x3C003C00u;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x == 0) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar))); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  if (threadIdx.x < 32) {
    if (CG == 1) { asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&slot)) : "memory"); asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
    else { asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&slot)) : "memory"); asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CG == 2) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tm = slot;
  uint32_t rank = 0;
  if (CG == 2) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  long long t0 = 0, t1 = 0;
  if (threadIdx.x == 0 && rank == 0) {
    const uint32_t sa = smem_u32(smem);
    const uint32_t id = idesc(m, n);
    t0 = clock64();
    for (int s = 0; s < steps; ++s) {
      const int st = s & 1;   // two "stages" of 48 KB
      const uint32_t base = sa + st * 48 * 1024;
      for (int kk = 0; kk < 4; ++kk) {
        const uint64_t a0 = make_desc(base) + 2 * kk, a1 = make_desc(base + 16384) + 2 * kk, b = make_desc(base + 32768) + 2 * kk;
        if (mode == 0) mma<CG>(tm, a0, make_desc(base + 16384) + 2 * kk, id, s | kk);
        else if (mode == 1) { mma<CG>(tm, a0, b, id, s | kk); mma<CG>(tm + 128, a1, b, id, s | kk); }
        else { mma<CG>(tm, a0, b, id, s | kk); mma<CG>(tm, a1, b, id, 1); }
      }
    }
    commit<CG>(smem_u32(&bar));
    for (long long spin = 0; spin < (1ll << 28) && !try_wait(smem_u32(&bar), 0); ++spin) {}
    t1 = clock64();
    out[blockIdx.x] = t1 - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CG == 2) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (CG == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
  }
}
template <int CG> void run(int n, int mode, int grid, long long* d_out, int m = 0) {
  if (m == 0) m = CG == 2 ? 256 : 128;
  const int steps = 4096, smem = 98 * 1024;
  cudaFuncSetAttribute(k<CG>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaLaunchConfig_t cfg = {}; cfg.gridDim = dim3(grid); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = CG; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  cudaMemset(d_out, 0, 148 * 8);
  for (int rep = 0; rep < 2; ++rep) {
    cudaError_t e = cudaLaunchKernelEx(&cfg, k<CG>, n, mode, steps, d_out, m);
    if (e != cudaSuccess) { printf("launch failed: %s\n", cudaGetErrorString(e)); return; }
    e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { printf("sync failed: %s\n", cudaGetErrorString(e)); exit(1); }
  }
  long long h[148]; cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost);
  double per_step = (double)h[0] / steps / 4;   // clocks per K=16 step
  const double macs = (double)(m / CG) * n * 16 * (mode == 0 ? 1 : 2);   // per SM per K16 step
  printf("cta_group::%d grid %3d M=%d N=%3d mode %d: %7.1f clk per K16 step, %6.0f MAC/clk/SM (ideal 4096)\n", CG, grid, m, n, mode, per_step, macs / per_step);
}
static int rates_main() {
  long long* d_out; cudaMalloc(&d_out, 148 * 8);
  printf("one MMA per K=16 step, same accumulator\n");
  for (int n : {256, 192, 160, 144, 136, 128, 64, 32, 16}) run<1>(n, 0, 148, d_out, 128);
  for (int n : {256, 128, 64}) run<1>(n, 0, 148, d_out, 64);
  for (int n : {256, 128, 64, 32, 16}) run<2>(n, 0, 148, d_out, 256);
  for (int n : {256, 128, 64}) run<2>(n, 0, 148, d_out, 128);
  printf("two MMAs per K=16 step sharing the N-side operand, two accumulators (operands swapped: weights as M, tokens as N)\n");
  for (int n : {128, 96, 64, 32, 16}) run<1>(n, 1, 148, d_out, 128);
  for (int n : {128, 96, 64, 32, 16}) run<2>(n, 1, 148, d_out, 256);
  return 0;
}

// ------------------------------------------------------------------ accumulator layout of cta_group::2, M = 128
__device__ __forceinline__ uint32_t try_wait_l(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done;
}
__device__ void put(unsigned char* base, int row, int k, float v) {   // K-major, 128-byte swizzle
  const int chunk = (k >> 3) ^ (row & 7);
  *reinterpret_cast<__nv_bfloat16*>(base + row * 128 + chunk * 16 + (k & 7) * 2) = __float2bfloat16(v);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) layout_kernel(int test, int M, int N, float* out) {
  extern __shared__ unsigned char dyn[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)dyn + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar; __shared__ uint32_t slot;
  uint32_t rank; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  for (int i = threadIdx.x; i < 64 * 1024 / 4; i += 128) ((uint32_t*)smem)[i] = 0;
  __syncthreads();
  unsigned char* sA = smem; unsigned char* sB = smem + 32768;
  const int mh = M / 2, nh = N / 2;
  for (int r = threadIdx.x; r < mh; r += 128) put(sA, r, 0, test == 0 ? (float)(rank * mh + r) : 1.0f);
  for (int r = threadIdx.x; r < nh; r += 128) put(sB, r, 0, test == 0 ? 1.0f : (float)(rank * nh + r));
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (threadIdx.x == 0) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar))); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tm = slot;
  // clear the accumulator region first: an M=256 N=256 product of zeros (B = zero region)
  if (threadIdx.x == 0 && rank == 0) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tm), "l"(make_desc(smem_u32(smem + 49152))), "l"(make_desc(smem_u32(smem + 49152))), "r"(idesc(256, 256)), "r"(0) : "memory");
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tm + 256), "l"(make_desc(smem_u32(smem + 49152))), "l"(make_desc(smem_u32(smem + 49152))), "r"(idesc(256, 256)), "r"(0) : "memory");
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tm), "l"(make_desc(smem_u32(sA))), "l"(make_desc(smem_u32(sB))), "r"(idesc(M, N)), "r"(0) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
    for (long long spin = 0; spin < (1ll << 26) && !try_wait_l(smem_u32(&bar), 0); ++spin) {}
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = 0; c < 512; c += 8) {
    uint32_t v[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(tm + ((uint32_t)(warp * 32) << 16) + c) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    for (int j = 0; j < 8; ++j) out[((size_t)rank * 128 + warp * 32 + lane) * 512 + c + j] = __uint_as_float(v[j]);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tm) : "memory");
  }
}
static int layout_main() {
  float* d; cudaMalloc(&d, 2 * 128 * 512 * 4);
  static float h0[2][128][512], h1[2][128][512];
  const int smem = 66 * 1024;
  cudaFuncSetAttribute(layout_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int N : {256, 128, 64, 32}) {
    layout_kernel<<<2, 128, smem>>>(0, 128, N, d); cudaError_t e = cudaDeviceSynchronize(); if (e) { printf("err %s\n", cudaGetErrorString(e)); return 1; }
    cudaMemcpy(h0, d, sizeof(h0), cudaMemcpyDeviceToHost);
    layout_kernel<<<2, 128, smem>>>(1, 128, N, d); e = cudaDeviceSynchronize(); if (e) { printf("err %s\n", cudaGetErrorString(e)); return 1; }
    cudaMemcpy(h1, d, sizeof(h1), cudaMemcpyDeviceToHost);
    printf("=== M=128 (cta_group::2) N=%d: (lane, col) -> D[row][n]; '.' = untouched\n", N);
    for (int r = 0; r < 2; ++r) {
      // summary: for each lane the row id, and the col->n mapping as runs
      int maxcol = -1;
      for (int l = 0; l < 128; ++l) for (int c = 0; c < 512; ++c) if (h1[r][l][c] != 0.f || h0[r][l][c] != 0.f) if (c > maxcol) maxcol = c;
      printf("cta %d: highest touched column %d\n", r, maxcol);
      for (int l : {0, 1, 15, 16, 31, 32, 47, 48, 63, 64, 65, 95, 96, 127}) {
        printf("  lane %3d: row(test0) at col0=%g col1=%g col%d=%g | n(test1): c0=%g c1=%g c2=%g c63=%g c64=%g c127=%g c128=%g c255=%g\n", l, h0[r][l][0], h0[r][l][1],
               N / 2, h0[r][l][N / 2], h1[r][l][0], h1[r][l][1], h1[r][l][2], h1[r][l][63], h1[r][l][64], h1[r][l][127], h1[r][l][128], h1[r][l][255]);
      }
    }
  }
  return 0;
}

int main(int argc, char** argv) {
  if (argc > 1 && !strcmp(argv[1], "layout")) return layout_main();
  return rates_main();
}
