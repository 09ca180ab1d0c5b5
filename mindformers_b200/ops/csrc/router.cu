// Top-k MoE router (sm_100a): score function, optional expert bias, group-limited selection, top-k,
// renormalisation, scaling and per-expert token counts in one pass; one warp per token.
//
//   scores = softmax(logits) | sigmoid(logits)                                   [T, E] fp32
//   sel    = scores (+ bias); with G groups only the best `group_topk` groups stay eligible, a group being
//            ranked by its best score (no bias) or by the sum of its two best biased scores (bias given)
//   ids    = top-k of sel (ties: lower expert index first);  probs = scores[ids]
//   probs  = probs / (sum(probs) + 1e-20) when `norm`;  probs *= scale;  counts[e] += 1 per selected copy
//
// The backward kernel recomputes the scores from the logits and maps d(probs) (and an optional dense
// d(scores), used by the load-balancing loss) to d(logits). E <= 512 and k <= 32.
#include "common.cuh"

namespace mfb {

constexpr int kRouterMaxPerLane = 16;  // E / 32
constexpr int kRouterMaxK = 32;
constexpr int kRouterWarps = 4;

struct RouterArgs {
  int T, E, k, sigmoid, norm, groups, group_topk;
  float scale;
};

// (value, index) arg-max over the warp; ties go to the lower index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

template <int PER>
__device__ __forceinline__ void router_scores(const float* __restrict__ row, int E, int lane, bool sigmoid,
                                              float (&s)[PER]) {
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    s[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, s[j]);
  }
  if (sigmoid) {
#pragma unroll
    for (int j = 0; j < PER; ++j) s[j] = (lane + 32 * j) < E ? 1.f / (1.f + __expf(-s[j])) : 0.f;
    return;
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    s[j] = (lane + 32 * j) < E ? __expf(s[j] - mx) : 0.f;
    sum += s[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int j = 0; j < PER; ++j) s[j] *= inv;
}

template <int PER>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ probs,
                  long long* __restrict__ ids, float* __restrict__ scores_out, float* __restrict__ counts,
                  RouterArgs a) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (t >= a.T) return;
  float s[PER], sel[PER];
  router_scores<PER>(logits + (long long)t * a.E, a.E, lane, a.sigmoid != 0, s);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    sel[j] = e < a.E ? (bias ? s[j] + bias[e] : s[j]) : -INFINITY;
    if (scores_out && e < a.E) scores_out[(long long)t * a.E + e] = s[j];
  }
  if (a.groups > 1 && a.group_topk > 0 && a.group_topk < a.groups) {
    // group score for every group (computed by the whole warp, group by group), then keep the best ones
    const int gsz = a.E / a.groups;
    float gscore = -INFINITY;  // lane g holds the score of group g (groups <= 32)
    for (int g = 0; g < a.groups; ++g) {
      float b1 = -INFINITY, b2 = -INFINITY;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int e = lane + 32 * j;
        if (e < a.E && e / gsz == g) {
          if (sel[j] > b1) { b2 = b1; b1 = sel[j]; } else if (sel[j] > b2) { b2 = sel[j]; }
        }
      }
      // merge (best, second best) pairs over the warp
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, b1, o), o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        const float n1 = fmaxf(b1, o1);
        const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1; b2 = n2;
      }
      const float sc = bias ? (b1 + (gsz > 1 ? b2 : 0.f)) : b1;
      if (lane == g) gscore = sc;
    }
    unsigned keep = 0;
    for (int r = 0; r < a.group_topk; ++r) {
      float v = gscore; int i = lane;
      warp_argmax(v, i);
      keep |= 1u << i;
      if (lane == i) gscore = -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (e < a.E && !((keep >> (e / gsz)) & 1u)) sel[j] = -INFINITY;
    }
  }
  float psum = 0.f;
  float my_p = 0.f;  // lane r keeps the r-th selected probability
  int my_id = 0;
  for (int r = 0; r < a.k; ++r) {
    float bv = -INFINITY; int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (sel[j] > bv || (sel[j] == bv && e < bi)) { bv = sel[j]; bi = e; }
    }
    warp_argmax(bv, bi);
    // owner lane supplies the unbiased score and retires the expert
    float sv = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (lane + 32 * j == bi) { sv = s[j]; sel[j] = -INFINITY; }
    sv = __shfl_sync(0xffffffffu, sv, bi & 31);
    psum += sv;
    if (lane == r) { my_p = sv; my_id = bi; }
  }
  if (lane < a.k) {
    float p = my_p;
    if (a.norm) p = p / (psum + 1e-20f);
    probs[(long long)t * a.k + lane] = p * a.scale;
    ids[(long long)t * a.k + lane] = my_id;
    if (counts) atomicAdd(counts + my_id, 1.f);
  }
}

template <int PER>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_bwd_kernel(const float* __restrict__ logits, const long long* __restrict__ ids,
                  const float* __restrict__ dprobs, const float* __restrict__ dscores,
                  float* __restrict__ dlogits, RouterArgs a) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (t >= a.T) return;
  float s[PER], ds[PER];
  router_scores<PER>(logits + (long long)t * a.E, a.E, lane, a.sigmoid != 0, s);
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int e = lane + 32 * j;
    ds[j] = (dscores && e < a.E) ? dscores[(long long)t * a.E + e] : 0.f;
  }
  // selected set: D = sum s_sel, A = sum dout_j * s_j
  const int my_id = lane < a.k ? (int)ids[(long long)t * a.k + lane] : -1;
  const float my_do = lane < a.k ? dprobs[(long long)t * a.k + lane] * a.scale : 0.f;
  float my_s = 0.f;
  for (int r = 0; r < a.k; ++r) {
    const int id = __shfl_sync(0xffffffffu, my_id, r);
    float sv = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (lane + 32 * j == id) sv = s[j];
    sv = __shfl_sync(0xffffffffu, sv, id & 31);
    if (lane == r) my_s = sv;
  }
  float D = warp_sum(my_s);
  float A = warp_sum(my_do * my_s);
  float my_ds = my_do;
  if (a.norm) {
    D += 1e-20f;
    my_ds = my_do / D - A / (D * D);
  }
  for (int r = 0; r < a.k; ++r) {
    const int id = __shfl_sync(0xffffffffu, my_id, r);
    const float g = __shfl_sync(0xffffffffu, my_ds, r);
#pragma unroll
    for (int j = 0; j < PER; ++j)
      if (lane + 32 * j == id) ds[j] += g;
  }
  if (a.sigmoid) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (e < a.E) dlogits[(long long)t * a.E + e] = ds[j] * s[j] * (1.f - s[j]);
    }
  } else {
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) dot += ds[j] * s[j];
    dot = warp_sum(dot);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int e = lane + 32 * j;
      if (e < a.E) dlogits[(long long)t * a.E + e] = s[j] * (ds[j] - dot);
    }
  }
}

}  // namespace mfb

extern "C" {
using namespace mfb;

static int router_check(int T, int E, int k, int groups, int group_topk) {
  if (E < 1 || E > 32 * kRouterMaxPerLane || k < 1 || k > kRouterMaxK || k > E) {
    mfb_host::set_error("router: E=%d (max %d) / k=%d (max %d) out of range", E, 32 * kRouterMaxPerLane, k, kRouterMaxK);
    return 1;
  }
  if (groups > 1 && (groups > 32 || E % groups != 0 || group_topk > groups)) {
    mfb_host::set_error("router: %d groups (max 32, must divide E=%d), group_topk=%d", groups, E, group_topk);
    return 1;
  }
  return 0;
}

#define MFB_ROUTER_DISPATCH(KERNEL, ...)                                               \
  do {                                                                                 \
    const int per = (E + 31) / 32;                                                     \
    const unsigned grid = (unsigned)((T + kRouterWarps - 1) / kRouterWarps);           \
    if (per <= 4) KERNEL<4><<<grid, kRouterWarps * 32, 0, stream>>>(__VA_ARGS__);      \
    else if (per <= 8) KERNEL<8><<<grid, kRouterWarps * 32, 0, stream>>>(__VA_ARGS__); \
    else KERNEL<16><<<grid, kRouterWarps * 32, 0, stream>>>(__VA_ARGS__);              \
  } while (0)

// logits [T, E] fp32 (contiguous); bias [E] or null; probs [T, k] fp32; ids [T, k] int64;
// scores_out [T, E] fp32 or null; counts [E] fp32 or null (incremented, not cleared).
int mfb_router_fwd(const float* logits, const float* bias, float* probs, long long* ids, float* scores_out,
                   float* counts, int T, int E, int k, int sigmoid, int norm, int groups, int group_topk,
                   float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (router_check(T, E, k, groups, group_topk)) return 1;
  RouterArgs a{T, E, k, sigmoid, norm, groups, group_topk, scale};
  MFB_ROUTER_DISPATCH(router_fwd_kernel, logits, bias, probs, ids, scores_out, counts, a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// dlogits [T, E] = d(probs) and optional dense d(scores) pulled back through the router.
int mfb_router_bwd(const float* logits, const long long* ids, const float* dprobs, const float* dscores,
                   float* dlogits, int T, int E, int k, int sigmoid, int norm, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (router_check(T, E, k, 0, 0)) return 1;
  RouterArgs a{T, E, k, sigmoid, norm, 0, 0, scale};
  MFB_ROUTER_DISPATCH(router_bwd_kernel, logits, ids, dprobs, dscores, dlogits, a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
