// Paged KV cache kernels for decoding (sm_100a): cache write by slot mapping, and single-query attention over a
// block table (GQA, head dim 64/128, bf16 cache, fp32 math).
//
// Cache layout (reference generation/text_generator.py:114-160): key_cache / value_cache
// [num_blocks, block_size, kv_heads, head_dim] per layer; slot = block * block_size + offset.
//
// Decode attention: one CTA per (sequence, KV head) handles all query heads of the group, so K and V are read
// from HBM once per group. Keys are processed in tiles of 128: phase 1 computes scores with one warp per key
// (lanes split the head dimension, shuffle reduction), phase 2 accumulates P·V with one thread per output
// dimension so that V rows are read coalesced. Online softmax keeps running (max, sum) per head.
// The kernel is bandwidth-bound: its roofline is KV bytes / HBM bandwidth.
#include "common.cuh"

namespace mfb {

// key/value: [T, kv_heads, hd] (token stride given); slot_mapping[t] < 0 skips the token.
__global__ void reshape_and_cache_kernel(const __nv_bfloat16* __restrict__ key, const __nv_bfloat16* __restrict__ value,
                                         __nv_bfloat16* __restrict__ key_cache, __nv_bfloat16* __restrict__ value_cache,
                                         const int* __restrict__ slot_mapping, long long T, int row_elems,
                                         long long k_stride, long long v_stride) {
  const int vecs = row_elems / 8;
  const long long total = T * vecs;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vecs;
    const int c = (int)(i - t * vecs);
    const int slot = slot_mapping[t];
    if (slot < 0) continue;
    const uint4 kv = *reinterpret_cast<const uint4*>(key + t * k_stride + c * 8);
    *reinterpret_cast<uint4*>(key_cache + (long long)slot * row_elems + c * 8) = kv;
    if (value) {
      const uint4 vv = *reinterpret_cast<const uint4*>(value + t * v_stride + c * 8);
      *reinterpret_cast<uint4*>(value_cache + (long long)slot * row_elems + c * 8) = vv;
    }
  }
}

constexpr int kPaTile = 128;
constexpr int kPaMaxGroup = 16;

template <int HD>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q,        // [B, Hq, HD]
                    const __nv_bfloat16* __restrict__ key_cache, const __nv_bfloat16* __restrict__ value_cache,
                    const int* __restrict__ block_tables,        // [B, max_blocks]
                    const int* __restrict__ context_lens,        // [B] tokens to attend (including the new one)
                    __nv_bfloat16* __restrict__ out,             // [B, Hq, HD]
                    int Hq, int Hkv, int block_size, int max_blocks, float scale) {
  const int b = blockIdx.x, kvh = blockIdx.y;
  const int group = Hq / Hkv;
  const int ctx = context_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int PER_LANE = HD / 32;  // 4 (hd 128) or 2 (hd 64)
  __shared__ float s_q[kPaMaxGroup][HD];
  __shared__ float s_p[kPaMaxGroup][kPaTile];
  __shared__ float s_m[kPaMaxGroup], s_l[kPaMaxGroup], s_alpha[kPaMaxGroup];
  for (int i = threadIdx.x; i < group * HD; i += 128) {
    const int h = i / HD, d = i - h * HD;
    s_q[h][d] = __bfloat162float(q[((size_t)b * Hq + kvh * group + h) * HD + d]) * scale;
  }
  if (threadIdx.x < group) { s_m[threadIdx.x] = -INFINITY; s_l[threadIdx.x] = 0.f; }
  __syncthreads();
  float acc[kPaMaxGroup];
#pragma unroll
  for (int h = 0; h < kPaMaxGroup; ++h) acc[h] = 0.f;
  const int* table = block_tables + (size_t)b * max_blocks;
  const size_t row = (size_t)Hkv * HD;  // elements per cached token
  for (int t0 = 0; t0 < ctx; t0 += kPaTile) {
    const int n = min(kPaTile, ctx - t0);
    // ---- phase 1: scores, one warp per key ----
    for (int k = warp; k < kPaTile; k += 4) {
      if (k < n) {
        const int tok = t0 + k;
        const int blk = table[tok / block_size];
        const __nv_bfloat16* kp = key_cache + ((size_t)blk * block_size + tok % block_size) * row + (size_t)kvh * HD + lane * PER_LANE;
        float kv[PER_LANE];
        if (PER_LANE == 4) {
          const uint2 u = *reinterpret_cast<const uint2*>(kp);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
          const float2 a = __bfloat1622float2(h2[0]), c = __bfloat1622float2(h2[1]);
          kv[0] = a.x; kv[1] = a.y; kv[2 % PER_LANE] = c.x; kv[3 % PER_LANE] = c.y;
        } else {
          const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kp));
          kv[0] = a.x; kv[1] = a.y;
        }
        for (int h = 0; h < group; ++h) {
          float d = 0.f;
#pragma unroll
          for (int i = 0; i < PER_LANE; ++i) d += kv[i] * s_q[h][lane * PER_LANE + i];
          d = warp_sum(d);
          if (lane == 0) s_p[h][k] = d;
        }
      } else if (lane == 0) {
        for (int h = 0; h < group; ++h) s_p[h][k] = -INFINITY;
      }
    }
    __syncthreads();
    // ---- online softmax update: warp w handles heads w, w+4, ... ----
    for (int h = warp; h < group; h += 4) {
      float mx = -INFINITY;
      for (int k = lane; k < kPaTile; k += 32) mx = fmaxf(mx, s_p[h][k]);
      mx = warp_max(mx);
      const float m_old = s_m[h];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      for (int k = lane; k < kPaTile; k += 32) {
        const float p = __expf(s_p[h][k] - m_new);
        s_p[h][k] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float alpha = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
        s_alpha[h] = alpha;
        s_l[h] = s_l[h] * alpha + sum;
        s_m[h] = m_new;
      }
    }
    __syncthreads();
    // ---- phase 2: acc[h] (dimension = thread) = acc*alpha + sum_k p[h][k] V[k][d] ----
    for (int d = threadIdx.x; d < HD; d += 128) {
#pragma unroll
      for (int h = 0; h < kPaMaxGroup; ++h)
        if (h < group) acc[h] *= s_alpha[h];
      for (int k = 0; k < n; ++k) {
        const int tok = t0 + k;
        const int blk = table[tok / block_size];
        const float v = __bfloat162float(value_cache[((size_t)blk * block_size + tok % block_size) * row + (size_t)kvh * HD + d]);
#pragma unroll
        for (int h = 0; h < kPaMaxGroup; ++h)
          if (h < group) acc[h] += s_p[h][k] * v;
      }
    }
    __syncthreads();
  }
  for (int d = threadIdx.x; d < HD; d += 128) {
#pragma unroll
    for (int h = 0; h < kPaMaxGroup; ++h)
      if (h < group) {
        const float l = s_l[h];
        out[((size_t)b * Hq + kvh * group + h) * HD + d] = __float2bfloat16(l > 0.f ? acc[h] / l : 0.f);
      }
  }
}

// out[t, :] = cache[slot(t), :] gathered through the block table: token i of sequence b for i < lens[b],
// written at row cu[b] + i. Used to materialise a contiguous K/V (or MLA latent) for prefill with history.
__global__ void gather_cache_kernel(const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_tables,
                                    const int* __restrict__ cu_lens, __nv_bfloat16* __restrict__ out, int B,
                                    int block_size, int max_blocks, int row_elems) {
  const int b = blockIdx.y;
  const int start = cu_lens[b], n = cu_lens[b + 1] - start;
  const int vecs = row_elems / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n * vecs;
       i += (long long)gridDim.x * blockDim.x) {
    const int tok = (int)(i / vecs), c = (int)(i - (long long)tok * vecs);
    const int blk = block_tables[(size_t)b * max_blocks + tok / block_size];
    const uint4 v = *reinterpret_cast<const uint4*>(cache + ((size_t)blk * block_size + tok % block_size) * row_elems + c * 8);
    *reinterpret_cast<uint4*>(out + (size_t)(start + tok) * row_elems + c * 8) = v;
  }
}

}  // namespace mfb

extern "C" {
using namespace mfb;

int mfb_reshape_and_cache(const void* key, const void* value, void* key_cache, void* value_cache,
                          const int* slot_mapping, long long T, int row_elems, long long k_stride, long long v_stride,
                          cudaStream_t stream) {
  if (row_elems % 8) { mfb_host::set_error("reshape_and_cache: row of %d elements is not a multiple of 8", row_elems); return 1; }
  if (T <= 0) return 0;
  long long blocks = (T * (row_elems / 8) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  reshape_and_cache_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)key, (const __nv_bfloat16*)value,
                                                                (__nv_bfloat16*)key_cache, (__nv_bfloat16*)value_cache,
                                                                slot_mapping, T, row_elems, k_stride, v_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_paged_decode_attention(const void* q, const void* key_cache, const void* value_cache, const int* block_tables,
                               const int* context_lens, void* out, int B, int Hq, int Hkv, int hd, int block_size,
                               int max_blocks, float scale, cudaStream_t stream) {
  if (Hq % Hkv || Hq / Hkv > kPaMaxGroup || (hd != 128 && hd != 64)) {
    mfb_host::set_error("paged_decode_attention: unsupported Hq=%d Hkv=%d hd=%d", Hq, Hkv, hd);
    return 1;
  }
  if (B <= 0) return 0;
  dim3 grid(B, Hkv);
  if (hd == 128)
    paged_decode_kernel<128><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)key_cache,
                                                       (const __nv_bfloat16*)value_cache, block_tables, context_lens,
                                                       (__nv_bfloat16*)out, Hq, Hkv, block_size, max_blocks, scale);
  else
    paged_decode_kernel<64><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)key_cache,
                                                      (const __nv_bfloat16*)value_cache, block_tables, context_lens,
                                                      (__nv_bfloat16*)out, Hq, Hkv, block_size, max_blocks, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_gather_cache(const void* cache, const int* block_tables, const int* cu_lens, void* out, int B, int max_len,
                     int block_size, int max_blocks, int row_elems, cudaStream_t stream) {
  if (row_elems % 8) { mfb_host::set_error("gather_cache: row of %d elements is not a multiple of 8", row_elems); return 1; }
  if (B <= 0 || max_len <= 0) return 0;
  long long per = ((long long)max_len * (row_elems / 8) + 255) / 256;
  if (per > 1024) per = 1024;
  dim3 grid((unsigned)per, B);
  gather_cache_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)cache, block_tables, cu_lens, (__nv_bfloat16*)out, B,
                                                block_size, max_blocks, row_elems);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
