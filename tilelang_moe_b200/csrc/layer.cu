// The whole MoE layer behind one C call: router (given logits, or x . Wr^T) -> top-k + softmax over all experts ->
// histogram / offsets / permutation -> up GEMM (gathering its rows, SiLU gate fused) -> down GEMM (routing weight
// and scatter fused) -> k-way combine with the shared expert.  It only sequences the library's own entry points on
// the caller's stream; the shared expert runs on `side_stream` when one is given (fork / join by two events).
// Same arithmetic as calling the pieces one by one, so results are bit-identical to that.
#include "common.cuh"
#include "../../include/moe_b200.h"

#include <mutex>

namespace moe {

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

struct LayerScratch {
  size_t scores, idx32, counts, offsets, perm, hist, act, yk, logits, xs, wsorted, act_s, y_s, total;
};

// The shared expert can ride along as expert E of the routed GEMMs - every token then has k + 1 routed entries, the
// last with weight 1 - when it has the width of a routed expert and its weights lie directly behind the routed ones
// in memory (one [E+1, ...] tensor per projection), and the up GEMM gathers its rows itself.
static bool shared_rides_along(const void* shared_gate, const void* shared_up, const void* shared_down, const void* routed_gate,
                               const void* routed_up, const void* routed_down, int H, int I, int E, int SI) {
  if (SI != I || SI == 0 || H % 64 || E + 1 > 1024) return false;
  const size_t per = (size_t)I * H * 2;
  return reinterpret_cast<const unsigned char*>(routed_gate) + (size_t)E * per == shared_gate &&
         reinterpret_cast<const unsigned char*>(routed_up) + (size_t)E * per == shared_up &&
         reinterpret_cast<const unsigned char*>(routed_down) + (size_t)E * per == shared_down;
}

static LayerScratch layer_layout(int64_t T, int k, int H, int I, int E, int SI) {
  LayerScratch L;
  const size_t n = (size_t)T * (k + (SI == I ? 1 : 0));   // room for the shared expert's entries when it rides along
  size_t o = 0;
  auto take = [&](size_t bytes) { const size_t at = o; o += align256(bytes); return at; };
  L.scores = take(n * 4);
  L.idx32 = take(n * 4);
  L.counts = take((size_t)(E + 1) * 4);
  L.offsets = take((size_t)(E + 2) * 4);
  L.perm = take(n * 4);
  L.hist = take(moe_route_histogram_workspace((int64_t)n, E + 1));
  L.act = take(n * (size_t)I * 2);
  L.yk = take(n * (size_t)H * 2);
  // router scratch: the logits when the one-kernel router does not apply, or the K slices of the few-token router
  L.logits = take((size_t)T * E * 4 * (size_t)router_splits(T, H));
  const bool fused_gather = H % 64 == 0;
  L.xs = take(fused_gather ? 0 : n * (size_t)H * 2);
  L.wsorted = take(fused_gather ? 0 : n * 4);
  L.act_s = take((size_t)T * SI * 2);
  L.y_s = take(SI > 0 ? (size_t)T * H * 2 : 0);
  L.total = o;
  return L;
}

// two events per device for the fork / join around the shared expert; created once, never destroyed
static int layer_events(cudaEvent_t* fork, cudaEvent_t* join) {
  static cudaEvent_t ev[64][2];
  static bool made[64];
  static std::mutex mu;
  int dev = 0;
  MOE_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MOE_ERR_DEVICE, "layer_forward: device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!made[dev]) {
    MOE_CUDA_CHECK(cudaEventCreateWithFlags(&ev[dev][0], cudaEventDisableTiming));
    MOE_CUDA_CHECK(cudaEventCreateWithFlags(&ev[dev][1], cudaEventDisableTiming));
    made[dev] = true;
  }
  *fork = ev[dev][0];
  *join = ev[dev][1];
  return MOE_OK;
}

}  // namespace moe

extern "C" size_t moe_layer_workspace(int64_t T, int k, int H, int I, int E, int SI) {
  if (T < 1 || k < 1 || H < 1 || I < 1 || E < 1 || SI < 0) return 0;
  return moe::layer_layout(T, k, H, I, E, SI).total;
}

extern "C" int moe_layer_forward(const void* x, const void* router_weight, const float* logits, const void* shared_gate,
                                 const void* shared_up, const void* shared_down, const void* routed_gate,
                                 const void* routed_up, const void* routed_down, int64_t T, int H, int I, int E, int k,
                                 int SI, int dtype, void* ws, size_t ws_bytes, void* out, int32_t* status, void* stream,
                                 void* side_stream) {
  using namespace moe;
  if (T < 0 || H < 8 || (H % 8) || I < 8 || (I % 8) || E < 1 || k < 1 || k > E || SI < 0 || (SI % 8))
    return fail(MOE_ERR_ARG, "layer_forward: bad shape T=%lld H=%d I=%d E=%d k=%d SI=%d", (long long)T, H, I, E, k, SI);
  if (T == 0) return MOE_OK;
  if (!x || (!router_weight && !logits) || !routed_gate || !routed_up || !routed_down || !out || !ws)
    return fail(MOE_ERR_ARG, "layer_forward: null pointer");
  if (SI > 0 && (!shared_gate || !shared_up || !shared_down)) return fail(MOE_ERR_ARG, "layer_forward: shared expert weights missing");
  if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(MOE_ERR_ARG, "layer_forward: workspace must be 256-byte aligned");
  const LayerScratch L = layer_layout(T, k, H, I, E, SI);
  if (ws_bytes < L.total) return fail(MOE_ERR_WORKSPACE, "layer_forward: workspace %zu < %zu", ws_bytes, L.total);
  unsigned char* base = reinterpret_cast<unsigned char*>(ws);
  float* scores = reinterpret_cast<float*>(base + L.scores);
  int32_t* idx32 = reinterpret_cast<int32_t*>(base + L.idx32);
  int32_t* counts = reinterpret_cast<int32_t*>(base + L.counts);
  int32_t* offsets = reinterpret_cast<int32_t*>(base + L.offsets);
  int32_t* perm = reinterpret_cast<int32_t*>(base + L.perm);
  void* act = base + L.act;
  void* yk = base + L.yk;
  const int64_t n = T * k;
  int rc;
  // once the side stream has been forked, every return - also an error - first makes `stream` wait for it again:
  // inside a stream capture an unjoined fork would turn the caller's end-of-capture into an unrelated failure
  bool forked = false;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto leave = [&](int code) {
    if (forked) {
      cudaStream_t side = reinterpret_cast<cudaStream_t>(side_stream);
      if (cudaEventRecord(ev_join, side) == cudaSuccess) cudaStreamWaitEvent(st, ev_join, 0);
      forked = false;
    }
    return code;
  };

  // shared expert: one more group of the routed GEMMs where its weights allow it; else it depends on x only and runs
  // beside the routed path when a second stream is given
  const bool ride = SI > 0 && shared_rides_along(shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down, H, I, E, SI);
  void* shared_out = nullptr;
  if (SI > 0 && !ride) {
    void* sst = stream;
    if (side_stream && side_stream != stream) {
      rc = layer_events(&ev_fork, &ev_join);
      if (rc) return rc;
      MOE_CUDA_CHECK(cudaEventRecord(ev_fork, st));
      MOE_CUDA_CHECK(cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(side_stream), ev_fork, 0));
      sst = side_stream;
      forked = true;
    }
    rc = dense_gemm(MOE_GEMM_SILU_GATE, x, shared_gate, shared_up, T, H, SI, base + L.act_s, SI, dtype, status, sst);
    if (rc) return leave(rc);
    rc = dense_gemm(MOE_GEMM_PLAIN, base + L.act_s, shared_down, nullptr, T, SI, H, base + L.y_s, H, dtype, status, sst);
    if (rc) return leave(rc);
    shared_out = base + L.y_s;
  }

  // router: softmax over all experts, top-k without renormalisation (the reference layer's convention)
  if (logits) {
    rc = moe_topk_softmax(logits, T, E, E, k, MOE_TOPK_MODE_A, scores, nullptr, idx32, status, stream);
    if (rc) return leave(rc);
  } else {
    // one kernel when the shape allows and has enough row tiles to hide the selection, else GEMM then top-k
    const bool small = E <= 32 && (size_t)E * H * 2 <= 200 * 1024;
    const int splits = router_splits(T, H);
    if (!small && splits >= 4 && E % 8 == 0 && E >= 8 && E <= 256 && k <= 32) {
      // few tokens: router GEMM split along K so that every SM gets a tile, then slice sum + selection
      rc = moe_router_topk_splitk(x, router_weight, T, H, E, k, MOE_TOPK_MODE_A, dtype, scores, nullptr, idx32, nullptr,
                                  base + L.logits, (size_t)T * E * 4 * (size_t)splits, status, stream);
      if (rc) return leave(rc);
      goto routed;
    }
    const bool fused = small || (E % 8 == 0 && E >= 8 && E <= 256 && k <= 8 && (E <= 64 || T >= 32 * (int64_t)E));
    if (fused) {
      rc = moe_router_topk(x, router_weight, T, H, E, k, MOE_TOPK_MODE_A, dtype, scores, nullptr, idx32, nullptr, status, stream);
      if (rc) return leave(rc);
    } else {
      float* lg = reinterpret_cast<float*>(base + L.logits);
      if (E % 8) return leave(fail(MOE_ERR_UNSUPPORTED, "layer_forward: E=%d needs E %% 8 == 0 or a router weight within 200 KB", E));
      rc = dense_gemm(MOE_GEMM_PLAIN_F32, x, router_weight, nullptr, T, H, E, lg, E, dtype, status, stream);
      if (rc) return leave(rc);
      rc = moe_topk_softmax(lg, T, E, E, k, MOE_TOPK_MODE_A, scores, nullptr, idx32, status, stream);
      if (rc) return leave(rc);
    }
  }
routed:
  if (ride) {
    // k + 1 entries per token: the k routed ones from idx32 and a virtual one for expert E; five launches in all
    const int64_t n1 = T * (k + 1);
    rc = route_histogram_ex(idx32, 0, n1, E + 1, nullptr, counts, offsets, perm, nullptr, base + L.hist,
                            moe_route_histogram_workspace(n1, E + 1), status, stream, k);
    if (rc) return rc;
    rc = moe_grouped_gemm_gathered(MOE_GEMM_SILU_GATE, x, T, perm, k + 1, routed_gate, routed_up, offsets, nullptr, nullptr, act,
                                   I, n1, 0, H, I, E + 1, dtype, status, stream);
    if (rc) return rc;
    rc = grouped_gemm_scatter_slots(act, routed_down, offsets, perm, scores, k, yk, H, n1, I, H, E + 1, dtype, status, stream);
    if (rc) return rc;
    return moe_combine(yk, nullptr, nullptr, nullptr, T, k + 1, H, dtype, out, stream);
  }
  rc = moe_route_histogram(idx32, 0, n, E, nullptr, counts, offsets, perm, nullptr, base + L.hist,
                           moe_route_histogram_workspace(n, E), status, stream);
  if (rc) return leave(rc);
  if (H % 64 == 0) {
    rc = moe_grouped_gemm_gathered(MOE_GEMM_SILU_GATE, x, T, perm, k, routed_gate, routed_up, offsets, nullptr, nullptr, act, I,
                                   n, 0, H, I, E, dtype, status, stream);
    if (rc) return leave(rc);
    rc = moe_grouped_gemm(MOE_GEMM_SCALE_SCATTER_DSTW, act, routed_down, nullptr, offsets, perm, scores, yk, H, n, 0, I, H, E,
                          dtype, status, stream);
    if (rc) return leave(rc);
  } else {
    float* wsorted = reinterpret_cast<float*>(base + L.wsorted);
    rc = moe_gather_rows(x, perm, k, n, H, base + L.xs, scores, wsorted, stream);
    if (rc) return leave(rc);
    rc = moe_grouped_gemm(MOE_GEMM_SILU_GATE, base + L.xs, routed_gate, routed_up, offsets, nullptr, nullptr, act, I, n, 0, H, I,
                          E, dtype, status, stream);
    if (rc) return leave(rc);
    rc = moe_grouped_gemm(MOE_GEMM_SCALE_SCATTER, act, routed_down, nullptr, offsets, perm, wsorted, yk, H, n, 0, I, H, E,
                          dtype, status, stream);
    if (rc) return leave(rc);
  }
  if (forked) {   // join: the combine reads the shared expert's output
    MOE_CUDA_CHECK(cudaEventRecord(ev_join, reinterpret_cast<cudaStream_t>(side_stream)));
    MOE_CUDA_CHECK(cudaStreamWaitEvent(st, ev_join, 0));
    forked = false;
  }
  return moe_combine(yk, shared_out, nullptr, nullptr, T, k, H, dtype, out, stream);
}
