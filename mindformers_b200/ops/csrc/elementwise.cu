// Memory-bound elementwise kernels for sm_100a: SwiGLU, RoPE, embedding gather / scatter-add,
// bf16<->fp32 casts with scale. All use 16-byte vector accesses and grid-stride loops sized to
// a multiple of the SM count.
#include "common.cuh"

namespace mfb {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

// in: [T, 2F] = [gate | up] ; out: [T, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                  long long T, int F) {
  const int fv = F / 8;
  const long long total = T * fv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i - t * fv);
    const bf16x8 g = reinterpret_cast<const bf16x8*>(in + t * 2 * F)[c];
    const bf16x8 u = reinterpret_cast<const bf16x8*>(in + t * 2 * F + F)[c];
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fg = __bfloat1622float2(g.v[j]);
      float2 fu = __bfloat1622float2(u.v[j]);
      o.v[j] = __floats2bfloat162_rn(silu(fg.x) * fu.x, silu(fg.y) * fu.y);
    }
    reinterpret_cast<bf16x8*>(out + t * F)[c] = o;
  }
}

// din[T,2F] from dout[T,F] and the saved input.
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ din, long long T, int F) {
  const int fv = F / 8;
  const long long total = T * fv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / fv;
    const int c = (int)(i - t * fv);
    const bf16x8 g = reinterpret_cast<const bf16x8*>(in + t * 2 * F)[c];
    const bf16x8 u = reinterpret_cast<const bf16x8*>(in + t * 2 * F + F)[c];
    const bf16x8 d = reinterpret_cast<const bf16x8*>(dout + t * F)[c];
    bf16x8 og, ou;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fg = __bfloat1622float2(g.v[j]);
      float2 fu = __bfloat1622float2(u.v[j]);
      float2 fd = __bfloat1622float2(d.v[j]);
      float s0 = 1.f / (1.f + __expf(-fg.x)), s1 = 1.f / (1.f + __expf(-fg.y));
      float dg0 = fd.x * fu.x * s0 * (1.f + fg.x * (1.f - s0));
      float dg1 = fd.y * fu.y * s1 * (1.f + fg.y * (1.f - s1));
      og.v[j] = __floats2bfloat162_rn(dg0, dg1);
      ou.v[j] = __floats2bfloat162_rn(fd.x * fg.x * s0, fd.y * fg.y * s1);
    }
    reinterpret_cast<bf16x8*>(din + t * 2 * F)[c] = og;
    reinterpret_cast<bf16x8*>(din + t * 2 * F + F)[c] = ou;
  }
}

// Rotary embedding in place on the first `n_heads` heads of x[t, head, hd] (token stride given).
// cos/sin: [max_pos, rot/2] fp32. interleaved=0: pairs (i, i+rot/2); =1: pairs (2i, 2i+1).
// sign=+1 forward, -1 backward (the transpose of a rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cosT,
                            const float* __restrict__ sinT, const int* __restrict__ positions, long long T,
                            int n_heads, int hd, int rot, long long token_stride, int interleaved,
                            float sign, int seq_len) {
  const int half = rot / 2;
  const long long total = T * n_heads * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i % half);
    const long long th = i / half;
    const int h = (int)(th % n_heads);
    const long long t = th / n_heads;
    const int pos = positions ? positions[t] : (int)(t % seq_len);
    const float c = cosT[(long long)pos * half + p];
    const float s = sinT[(long long)pos * half + p] * sign;
    __nv_bfloat16* base = x + t * token_stride + (long long)h * hd;
    const int i0 = interleaved ? 2 * p : p;
    const int i1 = interleaved ? 2 * p + 1 : p + half;
    const float a = __bfloat162float(base[i0]);
    const float b = __bfloat162float(base[i1]);
    base[i0] = __float2bfloat16(a * c - b * s);
    base[i1] = __float2bfloat16(b * c + a * s);
  }
}

// Vector form of rope_kernel: every thread rotates 8 pairs with 16-byte loads and stores.
//   rotate-half  (INTERLEAVED = 0): elements [8c, 8c+8) of the first half pair with the same slice of the second half
//   interleaved  (INTERLEAVED = 1): one 16-byte vector holds 4 pairs (2i, 2i+1); a thread takes two vectors
// Needs rot % 16 == 0, 16-byte aligned rows (hd, token_stride multiples of 8).
template <int INTERLEAVED>
__global__ void __launch_bounds__(256)
rope_vec_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cosT, const float* __restrict__ sinT,
                const int* __restrict__ positions, long long T, int n_heads, int hd, int rot, long long token_stride,
                float sign, int seq_len) {
  const int half = rot / 2;
  const int chunks = half / 8;                      // 8 pairs per thread
  const long long total = T * n_heads * chunks;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % chunks);
    const long long th = i / chunks;
    const int h = (int)(th % n_heads);
    const long long t = th / n_heads;
    const int pos = positions ? positions[t] : (int)(t % seq_len);
    const float4* cp = reinterpret_cast<const float4*>(cosT + (long long)pos * half + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(sinT + (long long)pos * half + c * 8);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x * sign, s0.y * sign, s0.z * sign, s0.w * sign, s1.x * sign, s1.y * sign, s1.z * sign, s1.w * sign};
    __nv_bfloat16* base = x + t * token_stride + (long long)h * hd;
    bf16x8* pa = reinterpret_cast<bf16x8*>(base + (INTERLEAVED ? c * 16 : c * 8));
    bf16x8* pb = reinterpret_cast<bf16x8*>(base + (INTERLEAVED ? c * 16 + 8 : half + c * 8));
    bf16x8 va = *pa, vb = *pb;
    if (INTERLEAVED) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(va.v[j]);
        va.v[j] = __floats2bfloat162_rn(f.x * cs[j] - f.y * sn[j], f.y * cs[j] + f.x * sn[j]);
        float2 g = __bfloat1622float2(vb.v[j]);
        vb.v[j] = __floats2bfloat162_rn(g.x * cs[4 + j] - g.y * sn[4 + j], g.y * cs[4 + j] + g.x * sn[4 + j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = __bfloat1622float2(va.v[j]), b = __bfloat1622float2(vb.v[j]);
        va.v[j] = __floats2bfloat162_rn(a.x * cs[2 * j] - b.x * sn[2 * j], a.y * cs[2 * j + 1] - b.y * sn[2 * j + 1]);
        vb.v[j] = __floats2bfloat162_rn(b.x * cs[2 * j] + a.x * sn[2 * j], b.y * cs[2 * j + 1] + a.y * sn[2 * j + 1]);
      }
    }
    *pa = va;
    *pb = vb;
  }
}

// out[t, :] = table[ids[t] - vocab_start, :] (zero row when the id is outside this rank's shard)
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long T, int H, int vocab_start,
                                     int vocab_rows) {
  const int hv = H / 8;
  const long long total = T * hv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / hv;
    const int c = (int)(i - t * hv);
    const long long id = ids[t] - vocab_start;
    bf16x8 v;
    if (id >= 0 && id < vocab_rows) {
      v = reinterpret_cast<const bf16x8*>(table + id * H)[c];
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v.v[j] = __floats2bfloat162_rn(0.f, 0.f);
    }
    reinterpret_cast<bf16x8*>(out + t * H)[c] = v;
  }
}

// dtable[ids[t]] += dout[t]  (fp32 gradient buffer, vector atomics)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ dtable, long long T, int H, int vocab_start,
                                     int vocab_rows) {
  const int hv = H / 4;
  const long long total = T * hv;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / hv;
    const int c = (int)(i - t * hv);
    const long long id = ids[t] - vocab_start;
    if (id < 0 || id >= vocab_rows) continue;
    const __nv_bfloat162* s = reinterpret_cast<const __nv_bfloat162*>(dout + t * H + c * 4);
    const float2 a = __bfloat1622float2(s[0]);
    const float2 b = __bfloat1622float2(s[1]);
    float* d = dtable + id * H + c * 4;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d), "f"(a.x), "f"(a.y), "f"(b.x),
                 "f"(b.y)
                 : "memory");
  }
}

// dst_f32 = (accumulate ? dst : 0) + scale * src_bf16
__global__ void accum_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst,
                                         long long n, float scale, int accumulate) {
  const long long nv = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const bf16x8 a = reinterpret_cast<const bf16x8*>(src)[i];
    float4* d = reinterpret_cast<float4*>(dst) + 2 * i;
    float4 d0 = accumulate ? d[0] : make_float4(0, 0, 0, 0);
    float4 d1 = accumulate ? d[1] : make_float4(0, 0, 0, 0);
    float2 f0 = __bfloat1622float2(a.v[0]), f1 = __bfloat1622float2(a.v[1]);
    float2 f2 = __bfloat1622float2(a.v[2]), f3 = __bfloat1622float2(a.v[3]);
    d0.x += scale * f0.x; d0.y += scale * f0.y; d0.z += scale * f1.x; d0.w += scale * f1.y;
    d1.x += scale * f2.x; d1.y += scale * f2.y; d1.z += scale * f3.x; d1.w += scale * f3.y;
    d[0] = d0;
    d[1] = d1;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = nv * 8; i < n; ++i)
      dst[i] = (accumulate ? dst[i] : 0.f) + scale * __bfloat162float(src[i]);
  }
}

// out = a + b (bf16), used for residual adds that are not fused into a norm
__global__ void add_bf16_kernel(const __nv_bfloat16* a, const __nv_bfloat16* b, __nv_bfloat16* out,
                                long long n) {
  const long long nv = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
       i += (long long)gridDim.x * blockDim.x) {
    const bf16x8 x = reinterpret_cast<const bf16x8*>(a)[i];
    const bf16x8 y = reinterpret_cast<const bf16x8*>(b)[i];
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 fx = __bfloat1622float2(x.v[j]);
      float2 fy = __bfloat1622float2(y.v[j]);
      o.v[j] = __floats2bfloat162_rn(fx.x + fy.x, fx.y + fy.y);
    }
    reinterpret_cast<bf16x8*>(out)[i] = o;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (long long i = nv * 8; i < n; ++i)
      out[i] = __float2bfloat16(__bfloat162float(a[i]) + __bfloat162float(b[i]));
  }
}

static inline int ew_grid(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = 148 * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace mfb

extern "C" {
using namespace mfb;

int mfb_swiglu_fwd(const void* in, void* out, long long T, int F, cudaStream_t stream) {
  if (F % 8) { mfb_host::set_error("swiglu: F=%d must be a multiple of 8", F); return 1; }
  if (T <= 0) return 0;
  swiglu_fwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, stream>>>((const __nv_bfloat16*)in,
                                                                   (__nv_bfloat16*)out, T, F);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_swiglu_bwd(const void* in, const void* dout, void* din, long long T, int F, cudaStream_t stream) {
  if (F % 8) { mfb_host::set_error("swiglu: F=%d must be a multiple of 8", F); return 1; }
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<ew_grid(T * (F / 8), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)in, (const __nv_bfloat16*)dout, (__nv_bfloat16*)din, T, F);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_rope(void* x, const float* cosT, const float* sinT, const int* positions, long long T, int n_heads,
             int hd, int rot, long long token_stride, int interleaved, int backward, int seq_len,
             cudaStream_t stream) {
  if (rot % 2 || rot > hd) { mfb_host::set_error("rope: rotary dim %d invalid for head dim %d", rot, hd); return 1; }
  if (T <= 0 || n_heads <= 0) return 0;
  if (rot % 16 == 0 && hd % 8 == 0 && token_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(cosT) & 15) == 0 && (reinterpret_cast<uintptr_t>(sinT) & 15) == 0) {
    const long long n = T * n_heads * (rot / 16);
    const float sg = backward ? -1.f : 1.f;
    const int sl = seq_len > 0 ? seq_len : 1;
    if (interleaved)
      rope_vec_kernel<1><<<ew_grid(n, 256), 256, 0, stream>>>((__nv_bfloat16*)x, cosT, sinT, positions, T, n_heads, hd,
                                                             rot, token_stride, sg, sl);
    else
      rope_vec_kernel<0><<<ew_grid(n, 256), 256, 0, stream>>>((__nv_bfloat16*)x, cosT, sinT, positions, T, n_heads, hd,
                                                             rot, token_stride, sg, sl);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  rope_kernel<<<ew_grid(T * n_heads * (rot / 2), 256), 256, 0, stream>>>(
      (__nv_bfloat16*)x, cosT, sinT, positions, T, n_heads, hd, rot, token_stride, interleaved,
      backward ? -1.f : 1.f, seq_len > 0 ? seq_len : 1);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_embedding_fwd(const long long* ids, const void* table, void* out, long long T, int H, int vocab_start,
                      int vocab_rows, cudaStream_t stream) {
  if (H % 8) { mfb_host::set_error("embedding: H=%d must be a multiple of 8", H); return 1; }
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<ew_grid(T * (H / 8), 256), 256, 0, stream>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, T, H, vocab_start, vocab_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_embedding_bwd(const long long* ids, const void* dout, float* dtable, long long T, int H,
                      int vocab_start, int vocab_rows, cudaStream_t stream) {
  if (H % 4) { mfb_host::set_error("embedding: H=%d must be a multiple of 4", H); return 1; }
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<ew_grid(T * (H / 4), 256), 256, 0, stream>>>(ids, (const __nv_bfloat16*)dout, dtable,
                                                                      T, H, vocab_start, vocab_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_accum_bf16_to_f32(const void* src, float* dst, long long n, float scale, int accumulate,
                          cudaStream_t stream) {
  if (n <= 0) return 0;
  accum_bf16_to_f32_kernel<<<ew_grid(n / 8 + 1, 256), 256, 0, stream>>>((const __nv_bfloat16*)src, dst, n,
                                                                        scale, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_add_bf16(const void* a, const void* b, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  add_bf16_kernel<<<ew_grid(n / 8 + 1, 256), 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                               (__nv_bfloat16*)out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
