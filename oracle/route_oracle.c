/*
 * CPU oracle for the integer / index part of the routing path, in plain C.  TEST INFRASTRUCTURE ONLY:
 * it is compiled by oracle/build.py (and by __graft_entry__.build()) and loaded by tests/ alone; the product
 * never calls it.
 *
 * It restates, without any library, what the reference baseline obtains from torch:
 *   - top-k selection (kernels/topk_softmax_baseline.py:31,61: torch.topk), canonicalised to "value
 *     descending, equal values lowest index first, -0.0 == +0.0, NaN above every number";
 *   - bincount / cumsum / argsort of the flattened expert ids (kernels/fusedmoe_baseline.py:123-134),
 *     with the stable argsort as canonical permutation.
 * A second, independent statement of the same definitions as oracle/moe_oracle.py (which goes through
 * torch.sort): the two are checked against each other and against the golden fixtures.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* 1 if a ranks strictly before b in "descending, NaN first"; ties (equal, or both NaN) are not "before" */
static int ranks_before(float a, float b) {
  const int an = isnan(a), bn = isnan(b);
  if (an || bn) return an && !bn;
  return a > b; /* -0.0 > +0.0 is false both ways: they tie */
}

/* indices of the k first rows of a stable descending sort of every row; O(N*k) insertion, small cases only */
int oracle_topk_indices(const float* x, int64_t M, int64_t N, int64_t ld, int k, int64_t* idx) {
  if (k < 1 || k > N) return -1;
  for (int64_t r = 0; r < M; ++r) {
    const float* row = x + r * ld;
    int64_t* out = idx + r * k;
    int filled = 0;
    for (int64_t c = 0; c < N; ++c) {
      int pos = filled;
      while (pos > 0 && ranks_before(row[c], row[out[pos - 1]])) --pos; /* equal values: stay behind */
      if (pos >= k) continue;
      const int last = filled < k ? filled : k - 1;
      for (int j = last; j > pos; --j) out[j] = out[j - 1];
      out[pos] = c;
      if (filled < k) ++filled;
    }
  }
  return 0;
}

/* softmax over the k selected logits of a row, accumulated in double, returned as float */
void oracle_softmax_selected(const float* x, int64_t M, int64_t ld, int k, const int64_t* idx, float* scores) {
  for (int64_t r = 0; r < M; ++r) {
    const float* row = x + r * ld;
    double mx = -INFINITY, sum = 0.0;
    for (int j = 0; j < k; ++j) if (row[idx[r * k + j]] > mx) mx = row[idx[r * k + j]];
    for (int j = 0; j < k; ++j) sum += exp((double)row[idx[r * k + j]] - mx);
    for (int j = 0; j < k; ++j) scores[r * k + j] = (float)(exp((double)row[idx[r * k + j]] - mx) / sum);
  }
}

/* counts[E], exclusive offsets[E+1], stable permutation perm[n] (counting sort) and its inverse inv[n];
 * returns the number of ids outside [0,E) (they are skipped, as the CUDA path does) */
int64_t oracle_route_histogram(const int32_t* ids, int64_t n, int E, int32_t* counts, int32_t* offsets, int32_t* perm,
                               int32_t* inv) {
  int64_t bad = 0;
  memset(counts, 0, sizeof(int32_t) * (size_t)E);
  for (int64_t i = 0; i < n; ++i) {
    if (ids[i] < 0 || ids[i] >= E) { ++bad; continue; }
    ++counts[ids[i]];
  }
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
  int32_t* cursor = (int32_t*)malloc(sizeof(int32_t) * (size_t)E);
  if (!cursor) return -1;
  memcpy(cursor, offsets, sizeof(int32_t) * (size_t)E);
  for (int64_t i = 0; i < n; ++i) {
    if (ids[i] < 0 || ids[i] >= E) continue;
    const int32_t p = cursor[ids[i]]++;
    perm[p] = (int32_t)i;
    inv[i] = p;
  }
  free(cursor);
  return bad;
}
