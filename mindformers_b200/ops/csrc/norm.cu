// RMSNorm forward / backward for sm_100a (bf16 activations, fp32 statistics).
//
// forward : h = x (+ residual);  y = h * rsqrt(mean(h^2) + eps) * w ; saves rstd[T]
//           (the residual add of a pre-LN transformer block is fused: h is written back)
// backward: dx = rstd * (w*dy) - h * rstd^3 * mean(w*dy*h)   (+ dres, the gradient that
//           reaches h through the residual stream);   dw = sum_t dy * h * rstd
// dx and dw come from two kernels: carrying the dw partial sums through the dx loop costs so many registers that
// the loop loses more to low occupancy than the second read of dy and h costs. dw is reduced in two deterministic
// phases through a [parts, H] fp32 scratch buffer.
//
// CTAs of 256 threads walk rows (persistent grid), 16-byte vector accesses, the row kept in registers (H <= 8192) and
// the next row's loads issued before the current row is reduced. A warp-per-row variant serves per-head q/k norms
// (H <= 256, strided rows).
#include <mutex>

#include "common.cuh"
#include "rmsnorm_noalloc.h"

namespace mfb {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 4;  // 4 x 8 bf16 per thread => H <= 8192 stays in registers

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

// NVEC: 16-byte vectors per thread that cover a row (H <= NVEC * 256 * 8). The grid is persistent: a CTA walks rows
// blockIdx.x, blockIdx.x + gridDim.x, ... and issues the loads of its next row before it reduces the current one, so
// that the two block barriers of a row do not leave the memory system idle.
template <bool HAS_RES, int NVEC>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* x, const __nv_bfloat16* res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* h_out, float* __restrict__ rstd_out, int T, int H,
                   float eps) {
  __shared__ float red[32];
  const int nvec = H / 8;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8 wv[NVEC];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) wv[i] = wr[v];
  }
  bf16x8 nx[NVEC], nr[NVEC];
  auto load_row = [&](int row) {
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * H);
    const bf16x8* rr = HAS_RES ? reinterpret_cast<const bf16x8*>(res + (size_t)row * H) : nullptr;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        nx[i] = xr[v];
        if (HAS_RES) nr[i] = rr[v];
      }
    }
  };
  int row = blockIdx.x;
  if (row < T) load_row(row);
  for (; row < T; row += gridDim.x) {
    bf16x8* hr = HAS_RES ? reinterpret_cast<bf16x8*>(h_out + (size_t)row * H) : nullptr;
    float vals[NVEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        bf16x8 a = nx[i];
        if (HAS_RES) {
          bf16x8 o;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 fa = __bfloat1622float2(a.v[j]);
            float2 fb = __bfloat1622float2(nr[i].v[j]);
            o.v[j] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
          }
          hr[v] = o;
          a = o;  // normalise the rounded sum, the value the backward pass will read
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(a.v[j]);
          vals[i][2 * j] = f.x;
          vals[i][2 * j + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    const int next = row + gridDim.x;
    if (next < T) load_row(next);          // in flight during the reduction and the stores below
    const float tot = block_sum(ss, red);
    const float rstd = rsqrtf(tot / (float)H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        bf16x8 o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 fw = __bfloat1622float2(wv[i].v[j]);
          o.v[j] = __floats2bfloat162_rn(vals[i][2 * j] * rstd * fw.x, vals[i][2 * j + 1] * rstd * fw.y);
        }
        yr[v] = o;
      }
    }
  }
}

// Backward over rows [persistent grid]; each CTA keeps its dw partial in registers (columns owned
// by the thread) and writes one row of the scratch buffer at the end.
template <bool HAS_DRES, int NVEC>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int H) {
  __shared__ float red[32];
  const int nvec = H / 8;
  float dw_acc[NVEC][8];
  float wf[NVEC][8];
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw_acc[i][j] = 0.f; wf[i][j] = 0.f; }
    if (v < nvec) {
      const bf16x8 ww = wr[v];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(ww.v[j]);
        wf[i][2 * j] = f.x;
        wf[i][2 * j + 1] = f.y;
      }
    }
  }
  bf16x8 ndy[NVEC], nh[NVEC], ndr[NVEC];
  float nrstd = 0.f;
  auto load_row = [&](int row) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)row * H);
    const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + (size_t)row * H);
    const bf16x8* drr = HAS_DRES ? reinterpret_cast<const bf16x8*>(dres + (size_t)row * H) : nullptr;
    nrstd = rstd[row];
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        ndy[i] = dyr[v];
        nh[i] = hr[v];
        if (HAS_DRES) ndr[i] = drr[v];
      }
    }
  };
  int row = blockIdx.x;
  if (row < T) load_row(row);
  for (; row < T; row += gridDim.x) {
    const float r = nrstd;
    float wdy[NVEC][8], hv[NVEC][8], dr[NVEC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fd = __bfloat1622float2(ndy[i].v[j]);
          const float2 fh = __bfloat1622float2(nh[i].v[j]);
          wdy[i][2 * j] = fd.x * wf[i][2 * j];
          wdy[i][2 * j + 1] = fd.y * wf[i][2 * j + 1];
          hv[i][2 * j] = fh.x;
          hv[i][2 * j + 1] = fh.y;
          dot += wdy[i][2 * j] * fh.x + wdy[i][2 * j + 1] * fh.y;
          dw_acc[i][2 * j] += fd.x * fh.x * r;
          dw_acc[i][2 * j + 1] += fd.y * fh.y * r;
          if (HAS_DRES) {
            const float2 f = __bfloat1622float2(ndr[i].v[j]);
            dr[i][2 * j] = f.x;
            dr[i][2 * j + 1] = f.y;
          }
        }
      }
    }
    const int next = row + gridDim.x;
    if (next < T) load_row(next);          // in flight during the reduction and the stores below
    const float tot = block_sum(dot, red);
    const float c = tot * r * r * r / (float)H;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        bf16x8 o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a0 = wdy[i][2 * j] * r - hv[i][2 * j] * c;
          float a1 = wdy[i][2 * j + 1] * r - hv[i][2 * j + 1] * c;
          if (HAS_DRES) {
            a0 += dr[i][2 * j];
            a1 += dr[i][2 * j + 1];
          }
          o.v[j] = __floats2bfloat162_rn(a0, a1);
        }
        dxr[v] = o;
      }
    }
  }
  float* out = dw_partial + (size_t)blockIdx.x * H;
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) out[v * 8 + j] = dw_acc[i][j];
    }
  }
}

// dx alone (the regular entry point computes dw in a second kernel, which keeps this one light on registers):
// the row and its successor are held as raw bf16 vectors, floats are formed on the fly.
template <bool HAS_DRES, int NVEC>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                      const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                      const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx, int T, int H) {
  __shared__ float red[32];
  const int nvec = H / 8;
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  bf16x8 wv[NVEC];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) wv[i] = wr[v];
  }
  bf16x8 ndy[NVEC], nh[NVEC], ndr[NVEC];
  float nrstd = 0.f;
  auto load_row = [&](int row) {
    const bf16x8* dyr = reinterpret_cast<const bf16x8*>(dy + (size_t)row * H);
    const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + (size_t)row * H);
    const bf16x8* drr = HAS_DRES ? reinterpret_cast<const bf16x8*>(dres + (size_t)row * H) : nullptr;
    nrstd = rstd[row];
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        ndy[i] = dyr[v];
        nh[i] = hr[v];
        if (HAS_DRES) ndr[i] = drr[v];
      }
    }
  };
  int row = blockIdx.x;
  if (row < T) load_row(row);
  for (; row < T; row += gridDim.x) {
    const float r = nrstd;
    bf16x8 cdy[NVEC], ch[NVEC], cdr[NVEC];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      cdy[i] = ndy[i];
      ch[i] = nh[i];
      if (HAS_DRES) cdr[i] = ndr[i];
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fd = __bfloat1622float2(cdy[i].v[j]);
          const float2 fh = __bfloat1622float2(ch[i].v[j]);
          const float2 fw = __bfloat1622float2(wv[i].v[j]);
          dot += fd.x * fw.x * fh.x + fd.y * fw.y * fh.y;
        }
      }
    }
    const int next = row + gridDim.x;
    if (next < T) load_row(next);          // in flight during the reduction and the stores below
    const float tot = block_sum(dot, red);
    const float c = tot * r * r * r / (float)H;
    bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        bf16x8 o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fd = __bfloat1622float2(cdy[i].v[j]);
          const float2 fh = __bfloat1622float2(ch[i].v[j]);
          const float2 fw = __bfloat1622float2(wv[i].v[j]);
          float a0 = fd.x * fw.x * r - fh.x * c;
          float a1 = fd.y * fw.y * r - fh.y * c;
          if (HAS_DRES) {
            const float2 f = __bfloat1622float2(cdr[i].v[j]);
            a0 += f.x;
            a1 += f.y;
          }
          o.v[j] = __floats2bfloat162_rn(a0, a1);
        }
        dxr[v] = o;
      }
    }
  }
}

// dw partial sums: partial[split, c] = sum over the rows of the split of dy * h * rstd. A CTA covers 256 columns
// (a lane owns 8 of them, one 16-byte vector) and its 8 warps walk the rows of the split side by side.
__global__ void __launch_bounds__(256)
rmsnorm_dw_partial_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                          const float* __restrict__ rstd, float* __restrict__ partial, int T, int H,
                          int rows_per_split) {
  __shared__ float sm[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 256 + lane * 8;
  const bool valid = c0 < H;
  const int r_begin = blockIdx.y * rows_per_split;
  const int r_end = (r_begin + rows_per_split < T) ? r_begin + rows_per_split : T;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (valid) {
#pragma unroll 4
    for (int r = r_begin + warp; r < r_end; r += 8) {
      const bf16x8 a = *reinterpret_cast<const bf16x8*>(dy + (size_t)r * H + c0);
      const bf16x8 b = *reinterpret_cast<const bf16x8*>(h + (size_t)r * H + c0);
      const float rs = rstd[r];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __bfloat1622float2(a.v[j]);
        const float2 fb = __bfloat1622float2(b.v[j]);
        acc[2 * j] += fa.x * fb.x * rs;
        acc[2 * j + 1] += fa.y * fb.y * rs;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) sm[warp][lane * 8 + j] = acc[j];
  __syncthreads();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < H) {
    float s = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) s += sm[w8][threadIdx.x];
    partial[(size_t)blockIdx.y * H + c] = s;
  }
}

// dw[c] (+)= sum_p partial[p, c]; output fp32 (accumulate) or bf16. 32 columns per CTA, 8 warps split the parts.
__global__ void __launch_bounds__(256)
colsum_partials_kernel(const float* __restrict__ partial, int parts, int H,
                       float* __restrict__ dw_f32, __nv_bfloat16* __restrict__ dw_bf16,
                       int accumulate) {
  __shared__ float sm[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < H)
    for (int p = warp; p < parts; p += 8) s += partial[(size_t)p * H + c];
  sm[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) t += sm[w8][lane];
    if (dw_f32) dw_f32[c] = accumulate ? dw_f32[c] + t : t;
    if (dw_bf16) dw_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(dw_bf16[c]) + t : t);
  }
}

// ---- warp-per-row variant for per-head q/k norm: rows are (token, head) with strides ----
__global__ void headnorm_fwd_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                    float* __restrict__ rstd_out, int T, int heads, int hd,
                                    long long token_stride, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (row >= (long long)T * heads) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int hh = (int)(row - t * heads);
  __nv_bfloat16* p = x + t * token_stride + (long long)hh * hd;
  float v[8];
  float ss = 0.f;
  const int per = hd / 32;  // elements per lane (hd in {64,128,256})
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (i < per) {
      v[i] = __bfloat162float(p[lane * per + i]);
      ss += v[i] * v[i];
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)hd + eps);
  if (lane == 0 && rstd_out) rstd_out[row] = r;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (i < per) p[lane * per + i] = __float2bfloat16(v[i] * r * __bfloat162float(w[lane * per + i]));
  }
}

}  // namespace mfb

extern "C" {

using namespace mfb;

// y = rmsnorm(x (+res)) * w. `h_out` receives x+res when `res` is given (may alias x or res).
int mfb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                    int T, int H, float eps, cudaStream_t stream) {
  if (H % 8 != 0) {
    mfb_host::set_error("rmsnorm: H=%d must be a multiple of 8", H);
    return 1;
  }
  if (T <= 0) return 0;
  if (H > kNormThreads * kMaxVec * 8) {
    mfb_host::set_error("rmsnorm: H=%d above %d is not supported", H, kNormThreads * kMaxVec * 8);
    return 1;
  }
  const int nv = (H / 8 + kNormThreads - 1) / kNormThreads;      // vectors per thread: 1..4
  const int cap = 148 * (nv <= 2 ? 8 : 4);
  const int grid = T < cap ? T : cap;
#define MFB_RMS_FWD(RES, NV)                                                                              \
  rmsnorm_fwd_kernel<RES, NV><<<grid, kNormThreads, 0, stream>>>(                                          \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,      \
      (__nv_bfloat16*)h_out, rstd, T, H, eps)
  if (res) {
    if (nv == 1) MFB_RMS_FWD(true, 1); else if (nv == 2) MFB_RMS_FWD(true, 2);
    else if (nv == 3) MFB_RMS_FWD(true, 3); else MFB_RMS_FWD(true, 4);
  } else {
    if (nv == 1) MFB_RMS_FWD(false, 1); else if (nv == 2) MFB_RMS_FWD(false, 2);
    else if (nv == 3) MFB_RMS_FWD(false, 3); else MFB_RMS_FWD(false, 4);
  }
#undef MFB_RMS_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Number of scratch rows (of H floats each) that mfb_rmsnorm_bwd needs for a problem of T rows.
int mfb_rmsnorm_bwd_parts(int T) {
  int parts = 148 * 4;
  return T < parts ? T : parts;
}

// dx = d(rmsnorm)/dh (+ dres); dw (fp32 or bf16, one of them non-null) = or += column sums.
// `scratch` must hold mfb_rmsnorm_bwd_parts(T) * H floats. H <= 8192.
int mfb_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                    void* dx, float* dw_f32, void* dw_bf16, int accumulate, float* scratch, int T, int H,
                    cudaStream_t stream) {
  if (H % 8 != 0 || H > kNormThreads * kMaxVec * 8) {
    mfb_host::set_error("rmsnorm_bwd: H=%d must be a multiple of 8 and <= 8192", H);
    return 1;
  }
  if (T <= 0) return 0;
  const int nv = (H / 8 + kNormThreads - 1) / kNormThreads;
  const int cap = 148 * (nv <= 2 ? 6 : 3);
  const int grid = T < cap ? T : cap;
#define MFB_RMS_DX(DRES, NV)                                                                             \
  rmsnorm_bwd_dx_kernel<DRES, NV><<<grid, kNormThreads, 0, stream>>>(                                     \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd,                   \
      (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, T, H)
  if (dres) {
    if (nv == 1) MFB_RMS_DX(true, 1); else if (nv == 2) MFB_RMS_DX(true, 2);
    else if (nv == 3) MFB_RMS_DX(true, 3); else MFB_RMS_DX(true, 4);
  } else {
    if (nv == 1) MFB_RMS_DX(false, 1); else if (nv == 2) MFB_RMS_DX(false, 2);
    else if (nv == 3) MFB_RMS_DX(false, 3); else MFB_RMS_DX(false, 4);
  }
#undef MFB_RMS_DX
  // dw: row splits sized so that (column tiles x splits) fills the GPU a few times over, within the scratch rows
  const int col_tiles = (H + 255) / 256;
  int splits = (148 * 6 + col_tiles - 1) / col_tiles;
  const int max_parts = mfb_rmsnorm_bwd_parts(T);
  if (splits > max_parts) splits = max_parts;
  if (splits > (T + 7) / 8) splits = (T + 7) / 8;
  if (splits < 1) splits = 1;
  const int rows_per_split = (T + splits - 1) / splits;
  const int parts = (T + rows_per_split - 1) / rows_per_split;
  rmsnorm_dw_partial_kernel<<<dim3(col_tiles, parts), 256, 0, stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, rstd, scratch, T, H, rows_per_split);
  colsum_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(scratch, parts, H, dw_f32,
                                                           (__nv_bfloat16*)dw_bf16, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// In-place per-head RMSNorm on x[t, head, :] (rows `token_stride` elements apart).
int mfb_headnorm_fwd(void* x, const void* w, float* rstd, int T, int heads, int hd, long long token_stride,
                     float eps, cudaStream_t stream) {
  if (hd % 32 != 0 || hd > 256) {
    mfb_host::set_error("headnorm: head_dim=%d unsupported", hd);
    return 1;
  }
  const long long rows = (long long)T * heads;
  if (rows <= 0) return 0;
  const int wpb = 8;
  const int grid = (int)((rows + wpb - 1) / wpb);
  headnorm_fwd_kernel<<<grid, wpb * 32, 0, stream>>>((__nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, T,
                                                     heads, hd, token_stride, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"

// =================================================================================================
// RMSNorm backward without any allocation (declaration and user notes: rmsnorm_noalloc.h)
// =================================================================================================
namespace mfb {

// Upper limits of the built-in scratch: one row of partial column sums per resident CTA.
constexpr int kNoAllocMaxParts = 148;
constexpr int kNoAllocMaxH = 8192;

// Lives in the device memory of every GPU that loads this library, from load until the process exits
// (148 * 8192 floats = 4.6 MiB). Host code must not pass this name to a kernel: on the host it is only a
// handle for cudaGetSymbolAddress.
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[kNoAllocMaxParts * kNoAllocMaxH];

}  // namespace mfb

namespace {

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device; looked up once per device.
int noalloc_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    mfb_host::set_error("rmsnorm_bwd_noalloc: cannot identify the current device");
    return 3;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), mfb::g_rmsnorm_bwd_scratch);
    if (e != cudaSuccess || p == nullptr) {
      mfb_host::set_error("rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return 4;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int mfb_rmsnorm_bwd_noalloc(const void* dy, const void* h, const void* w, const float* rstd,
                                       const void* dres, void* dx, float* dw_f32, void* dw_bf16, int accumulate,
                                       int T, int H, cudaStream_t stream) {
  using namespace mfb;
  if (H % 8 != 0 || H <= 0 || H > kNoAllocMaxH) {
    mfb_host::set_error("rmsnorm_bwd_noalloc: H=%d must be a positive multiple of 8 and at most %d", H, kNoAllocMaxH);
    return 1;
  }
  if (T < 0 || (dw_f32 == nullptr && dw_bf16 == nullptr)) {
    mfb_host::set_error("rmsnorm_bwd_noalloc: bad arguments (T=%d, no dw output)", T);
    return 1;
  }
  if (T == 0) return 0;
  float* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  // Every launched CTA overwrites its whole row of partial sums and the reduction reads exactly the rows that
  // were launched, so nothing in the array has to be cleared between calls.
  const int parts = T < kNoAllocMaxParts ? T : kNoAllocMaxParts;
  // the widest register window serves every supported H here (one code path for this entry point)
  if (dres)
    rmsnorm_bwd_kernel<true, kMaxVec><<<parts, kNormThreads, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
        (__nv_bfloat16*)dx, scratch, T, H);
  else
    rmsnorm_bwd_kernel<false, kMaxVec><<<parts, kNormThreads, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd, nullptr, (__nv_bfloat16*)dx,
        scratch, T, H);
  colsum_partials_kernel<<<(H + 31) / 32, 256, 0, stream>>>(scratch, parts, H, dw_f32, (__nv_bfloat16*)dw_bf16,
                                                           accumulate);
  if (cudaGetLastError() != cudaSuccess) {
    mfb_host::set_error("rmsnorm_bwd_noalloc: launch failed");
    return 2;
  }
  return 0;
}
