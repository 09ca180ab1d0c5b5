// Cross-entropy (vocab-parallel aware), gradient-norm and fused AdamW kernels for sm_100a.
//
// Cross-entropy works on a [T, V_local] bf16 (or fp32) shard of the logits:
//   ce_stats : per row running (max, sum exp(x - max)) and the target logit if the label falls in
//              this shard. Ranks combine the three [T] vectors, then
//   ce_bwd   : dlogits = (exp(x - lse) - onehot) * gscale[t], written in place or to a new buffer.
//
// AdamW works on flat shards: bf16 parameter + 16-bit remainder (together an exact fp32 master,
// see adamw_kernel), fp32 m and v, fp32 or bf16 gradient. The clip coefficient and the skip flag
// are read from device scalars so that a step needs no host synchronisation.
#include "common.cuh"

namespace mfb {

constexpr int kCeThreads = 512;

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) { s = 0.f; m = nm; return; }
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

template <typename LT>
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const LT* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ row_max,
                float* __restrict__ row_sum, float* __restrict__ row_tgt, int V, long long ld, int vocab_start) {
  __shared__ float sm[32], ss[32];
  const long long row = blockIdx.x;
  const LT* x = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  if (sizeof(LT) == 2 && (ld % 8 == 0)) {
    const int nv = V / 8;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int i = threadIdx.x; i < nv; i += kCeThreads) {
      uint4 u = xv[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = __bfloat1622float2(h[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
      }
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      const float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += kCeThreads) online_merge(m, s, to_f32(x[i]), 1.f);
  } else {
    for (int i = threadIdx.x; i < V; i += kCeThreads) online_merge(m, s, to_f32(x[i]), 1.f);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sm[warp] = m; ss[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    m = lane < kCeThreads / 32 ? sm[lane] : -INFINITY;
    s = lane < kCeThreads / 32 ? ss[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) {
      row_max[row] = m;
      row_sum[row] = s;
      const long long lab = labels[row] - vocab_start;
      row_tgt[row] = (lab >= 0 && lab < V) ? to_f32(x[lab]) : 0.f;
    }
  }
}

template <typename LT>
__global__ void __launch_bounds__(kCeThreads)
ce_bwd_kernel(const LT* __restrict__ logits, LT* __restrict__ dlogits, const long long* __restrict__ labels,
              const float* __restrict__ lse, const float* __restrict__ gscale, int V, long long ld,
              int vocab_start) {
  const long long row = blockIdx.x;
  const LT* x = logits + row * ld;
  LT* d = dlogits + row * ld;
  const float l = lse[row];
  const float g = gscale[row];
  const long long lab = labels[row] - vocab_start;
  if (sizeof(LT) == 2 && (ld % 8 == 0)) {
    const int nv = V / 8;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    uint4* dv = reinterpret_cast<uint4*>(d);
    for (int i = threadIdx.x; i < nv; i += kCeThreads) {
      uint4 u = xv[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = __bfloat1622float2(h[j]);
        float p0 = __expf(t.x - l), p1 = __expf(t.y - l);
        if (i * 8 + 2 * j == lab) p0 -= 1.f;
        if (i * 8 + 2 * j + 1 == lab) p1 -= 1.f;
        op[j] = pack_bf16x2(p0 * g, p1 * g);
      }
      dv[i] = o;
    }
    for (int i = nv * 8 + threadIdx.x; i < V; i += kCeThreads) {
      float p = __expf(to_f32(x[i]) - l) - (i == lab ? 1.f : 0.f);
      d[i] = (LT)(p * g);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += kCeThreads) {
      float p = __expf(to_f32(x[i]) - l) - (i == lab ? 1.f : 0.f);
      d[i] = (LT)(p * g);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// sum of squares of a flat gradient buffer -> partials[grid]; finalize adds them into *out
// ----------------------------------------------------------------------------------------------
template <typename GT>
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const GT* __restrict__ g, long long n,
                                                            float* __restrict__ partials) {
  __shared__ float red[8];
  float acc = 0.f;
  if (sizeof(GT) == 4) {
    const long long nv = n / 4;
    const float4* gv = reinterpret_cast<const float4*>(g);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      float4 v = gv[i];
      acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (long long i = nv * 4; i < n; ++i) { float v = to_f32(g[i]); acc += v * v; }
  } else {
    const long long nv = n / 8;
    const uint4* gv = reinterpret_cast<const uint4*>(g);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      uint4 u = gv[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 t = __bfloat1622float2(h[j]);
        acc += t.x * t.x + t.y * t.y;
      }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (long long i = nv * 8; i < n; ++i) { float v = to_f32(g[i]); acc += v * v; }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
}

__global__ void sumsq_finalize_kernel(const float* __restrict__ partials, int parts, float* __restrict__ out,
                                      int accumulate) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) acc += partials[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) *out = accumulate ? *out + t : t;
  }
}

// ----------------------------------------------------------------------------------------------
// AdamW on a flat shard.
//   master (fp32) bits = (param_bf16_bits << 16) + (int16) lo     -- exact, and param_bf16 is the
//   nearest bf16 of the master (ties up in magnitude), so the model weights need no cast pass.
//   p <- p * (1 - lr*wd);  m,v EMA;  p <- p - lr_t * m / (sqrt(v / bc2) + eps),  lr_t = lr / bc1
// `sumsq` (device scalar, may be null) is the squared global gradient norm; the gradient is scaled
// by min(1, max_norm / (sqrt(sumsq) + 1e-6)) and the whole update is skipped when sumsq is not
// finite or sqrt(sumsq) >= skip_threshold (> 0).
// ----------------------------------------------------------------------------------------------
struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, skip_threshold, grad_scale;
  long long n, decay_end;  // elements [0, decay_end) get weight decay
};

template <typename GT>
__global__ void __launch_bounds__(256)
adamw_kernel(__nv_bfloat16* __restrict__ p, unsigned short* __restrict__ lo, float* __restrict__ m,
             float* __restrict__ v, const GT* __restrict__ g, const float* __restrict__ sumsq,
             int* __restrict__ skipped, AdamArgs a) {
  float clip = a.grad_scale;
  if (sumsq) {
    const float ss = *sumsq;
    const float nrm = sqrtf(ss) * fabsf(a.grad_scale);
    const bool bad = !isfinite(ss) || (a.skip_threshold > 0.f && nrm >= a.skip_threshold);
    if (bad) {
      if (blockIdx.x == 0 && threadIdx.x == 0 && skipped) *skipped = 1;
      return;
    }
    if (a.max_norm > 0.f && nrm >= a.max_norm) clip *= a.max_norm / (nrm + 1e-6f);
  }
  const float lr_t = a.lr / a.bc1;
  const float inv_bc2 = 1.f / a.bc2;
  const float decay = 1.f - a.lr * a.wd;
  // main part: 8 elements per thread and iteration, every stream moved with 16-byte accesses
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(lo) | reinterpret_cast<uintptr_t>(m) |
                        reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(g)) & 15) == 0;
  const long long nvec = vec_ok ? (a.n >> 3) : 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e0 = i * 8;
    const uint4 pv = *reinterpret_cast<const uint4*>(p + e0);
    const uint4 lv = *reinterpret_cast<const uint4*>(lo + e0);
    const unsigned short* ph = reinterpret_cast<const unsigned short*>(&pv);
    const unsigned short* pl = reinterpret_cast<const unsigned short*>(&lv);
    float gg[8], mm[8], vv[8];
    if (sizeof(GT) == 4) {
      *reinterpret_cast<float4*>(gg) = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + e0);
      *reinterpret_cast<float4*>(gg + 4) = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + e0 + 4);
    } else {
      const uint4 gv = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g) + e0);
      const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(g2[j]); gg[2 * j] = f.x; gg[2 * j + 1] = f.y; }
    }
    *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(m + e0);
    *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(m + e0 + 4);
    *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + e0);
    *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + e0 + 4);
    uint4 np, nl;
    unsigned short* nph = reinterpret_cast<unsigned short*>(&np);
    unsigned short* npl = reinterpret_cast<unsigned short*>(&nl);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float w = __uint_as_float(((uint32_t)ph[j] << 16) + (uint32_t)(int32_t)(int16_t)pl[j]);
      const float gr = gg[j] * clip;
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gr;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gr * gr;
      if (e0 + j < a.decay_end) w *= decay;
      w -= lr_t * mm[j] / (sqrtf(vv[j] * inv_bc2) + a.eps);
      const uint32_t wb = __float_as_uint(w);
      const uint32_t nhi = (wb + 0x8000u) >> 16;  // nearest bf16, ties up in magnitude
      nph[j] = (unsigned short)nhi;
      npl[j] = (unsigned short)((wb - (nhi << 16)) & 0xffffu);
    }
    *reinterpret_cast<float4*>(m + e0) = *reinterpret_cast<float4*>(mm);
    *reinterpret_cast<float4*>(m + e0 + 4) = *reinterpret_cast<float4*>(mm + 4);
    *reinterpret_cast<float4*>(v + e0) = *reinterpret_cast<float4*>(vv);
    *reinterpret_cast<float4*>(v + e0 + 4) = *reinterpret_cast<float4*>(vv + 4);
    *reinterpret_cast<uint4*>(p + e0) = np;
    *reinterpret_cast<uint4*>(lo + e0) = nl;
  }
  // scalar tail (and the whole range when a pointer is not 16-byte aligned)
  for (long long i = nvec * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n;
       i += (long long)gridDim.x * blockDim.x) {
    const uint32_t hi = __bfloat16_as_ushort(p[i]);
    const int32_t lov = (int32_t)(int16_t)lo[i];
    float w = __uint_as_float((hi << 16) + (uint32_t)lov);
    const float gr = to_f32(g[i]) * clip;
    float mm = m[i], vv = v[i];
    mm = a.beta1 * mm + (1.f - a.beta1) * gr;
    vv = a.beta2 * vv + (1.f - a.beta2) * gr * gr;
    if (i < a.decay_end) w *= decay;
    w -= lr_t * mm / (sqrtf(vv * inv_bc2) + a.eps);
    m[i] = mm;
    v[i] = vv;
    const uint32_t wb = __float_as_uint(w);
    const uint32_t nhi = (wb + 0x8000u) >> 16;
    p[i] = __ushort_as_bfloat16((unsigned short)nhi);
    lo[i] = (unsigned short)((wb - (nhi << 16)) & 0xffffu);
  }
}

// lo <- remainder so that (p, lo) reproduces `master` exactly; p <- rne(master)
__global__ void split_master_kernel(const float* __restrict__ master, __nv_bfloat16* __restrict__ p,
                                    unsigned short* __restrict__ lo, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float w = master[i];
    const uint32_t wb = __float_as_uint(w);
    const uint32_t nhi = (wb + 0x8000u) >> 16;
    p[i] = __ushort_as_bfloat16((unsigned short)nhi);
    lo[i] = (unsigned short)((wb - (nhi << 16)) & 0xffffu);
  }
}

__global__ void join_master_kernel(const __nv_bfloat16* __restrict__ p, const unsigned short* __restrict__ lo,
                                   float* __restrict__ master, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const uint32_t hi = __bfloat16_as_ushort(p[i]);
    master[i] = __uint_as_float((hi << 16) + (uint32_t)(int32_t)(int16_t)lo[i]);
  }
}

static inline int flat_grid(long long n, int per_thread) {
  long long blocks = (n / per_thread + 255) / 256;
  const long long cap = 148 * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// logits: [T, V] with row pitch ld; dtype 0 = bf16, 1 = fp32. Outputs are [T] fp32.
int mfb_ce_stats(const void* logits, int dtype, const long long* labels, float* row_max, float* row_sum,
                 float* row_tgt, long long T, int V, long long ld, int vocab_start, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == 0)
    ce_stats_kernel<__nv_bfloat16><<<(unsigned)T, kCeThreads, 0, stream>>>(
        (const __nv_bfloat16*)logits, labels, row_max, row_sum, row_tgt, V, ld, vocab_start);
  else
    ce_stats_kernel<float><<<(unsigned)T, kCeThreads, 0, stream>>>((const float*)logits, labels, row_max,
                                                                  row_sum, row_tgt, V, ld, vocab_start);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_ce_bwd(const void* logits, void* dlogits, int dtype, const long long* labels, const float* lse,
               const float* gscale, long long T, int V, long long ld, int vocab_start, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == 0)
    ce_bwd_kernel<__nv_bfloat16><<<(unsigned)T, kCeThreads, 0, stream>>>(
        (const __nv_bfloat16*)logits, (__nv_bfloat16*)dlogits, labels, lse, gscale, V, ld, vocab_start);
  else
    ce_bwd_kernel<float><<<(unsigned)T, kCeThreads, 0, stream>>>((const float*)logits, (float*)dlogits, labels,
                                                                lse, gscale, V, ld, vocab_start);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Number of floats of scratch that mfb_grad_sumsq needs.
int mfb_grad_sumsq_scratch() { return 148 * 8; }

// *out (+)= sum(g^2). dtype 0 = bf16, 1 = fp32. `scratch`: mfb_grad_sumsq_scratch() floats.
int mfb_grad_sumsq(const void* g, int dtype, long long n, float* scratch, float* out, int accumulate,
                   cudaStream_t stream) {
  const int grid = flat_grid(n, 8);
  if (dtype == 0)
    sumsq_partial_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)g, n, scratch);
  else
    sumsq_partial_kernel<float><<<grid, 256, 0, stream>>>((const float*)g, n, scratch);
  sumsq_finalize_kernel<<<1, 256, 0, stream>>>(scratch, grid, out, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_adamw(void* p, void* lo, float* m, float* v, const void* g, int g_dtype, const float* sumsq,
              int* skipped, long long n, long long decay_end, float lr, float beta1, float beta2, float eps,
              float wd, float bc1, float bc2, float max_norm, float skip_threshold, float grad_scale,
              cudaStream_t stream) {
  if (n <= 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd; a.bc1 = bc1; a.bc2 = bc2;
  a.max_norm = max_norm; a.skip_threshold = skip_threshold; a.grad_scale = grad_scale;
  a.n = n; a.decay_end = decay_end;
  const int grid = flat_grid(n, 8);
  if (g_dtype == 0)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)p, (unsigned short*)lo, m, v,
                                                          (const __nv_bfloat16*)g, sumsq, skipped, a);
  else
    adamw_kernel<float><<<grid, 256, 0, stream>>>((__nv_bfloat16*)p, (unsigned short*)lo, m, v,
                                                  (const float*)g, sumsq, skipped, a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_split_master(const float* master, void* p, void* lo, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  split_master_kernel<<<flat_grid(n, 4), 256, 0, stream>>>(master, (__nv_bfloat16*)p, (unsigned short*)lo, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_join_master(const void* p, const void* lo, float* master, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  join_master_kernel<<<flat_grid(n, 4), 256, 0, stream>>>((const __nv_bfloat16*)p, (const unsigned short*)lo,
                                                          master, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
