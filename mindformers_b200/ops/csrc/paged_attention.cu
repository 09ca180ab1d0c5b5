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
//
// int8 cache (kv_cache_dtype int8; reference utils/quantization_config.py kv-cache quantisation): rows are stored as
// int8 with one fp32 scale per (token, KV head) in a side array [num_blocks, block_size, kv_heads]; the write kernel
// quantises (absmax / 127), the decode kernel reads 8 bytes per lane instead of 16 and multiplies by the scale, so
// the bytes per cached token halve.
#include <type_traits>

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

// One warp per (token, head): scale = absmax / 127, codes = round(x / scale).
__global__ void reshape_and_cache_int8_kernel(const __nv_bfloat16* __restrict__ key, const __nv_bfloat16* __restrict__ value,
                                              int8_t* __restrict__ key_cache, int8_t* __restrict__ value_cache,
                                              float* __restrict__ key_scale, float* __restrict__ value_scale,
                                              const int* __restrict__ slot_mapping, long long T, int heads, int hd,
                                              long long k_stride, long long v_stride) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * heads) return;
  const long long t = w / heads;
  const int h = (int)(w - t * heads);
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* src = which == 0 ? key + t * k_stride + (long long)h * hd
                                          : (value ? value + t * v_stride + (long long)h * hd : nullptr);
    if (!src) break;
    float m = 0.f;
    for (int d = lane; d < hd; d += 32) m = fmaxf(m, fabsf(__bfloat162float(src[d])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float sc = m > 0.f ? m / 127.f : 1.f;
    const float inv = 1.f / sc;
    int8_t* dst = (which == 0 ? key_cache : value_cache) + ((long long)slot * heads + h) * hd;
    for (int d = lane; d < hd; d += 32) {
      int r = __float2int_rn(__bfloat162float(src[d]) * inv);
      dst[d] = (int8_t)(r > 127 ? 127 : (r < -127 ? -127 : r));
    }
    if (lane == 0) (which == 0 ? key_scale : value_scale)[(long long)slot * heads + h] = sc;
  }
}

constexpr int kPaMaxGroup = 16;
constexpr int kPaWarps = 4;
constexpr int kPaHeadsPerPass = 4;   // query heads kept in registers at a time

// Split-KV decode attention ("flash decoding") on the CUDA cores; the kernel is bandwidth-bound.
//   grid (splits, Hkv, B); CTA = 4 warps. A CTA owns keys [split * chunk, (split + 1) * chunk) of one sequence and
//   one KV head. A key row of HD bf16 is read by HD/8 lanes with one 16-byte load each, so a warp covers
//   32 / (HD/8) keys per instruction (2 for head dim 128, 4 for 64); every lane keeps the query slice, the running
//   (max, sum) and the output slice of its 8 dimensions for up to four query heads. Lane groups never synchronise
//   inside the loop: each keeps its own online softmax and the partial results are merged once, first inside the
//   CTA through shared memory, then across splits by paged_combine_kernel.
template <int HD, bool INT8>
__global__ void __launch_bounds__(kPaWarps * 32)
paged_decode_split_kernel(const __nv_bfloat16* __restrict__ q,        // [B, Hq, HD]
                          const void* __restrict__ key_cache_v, const void* __restrict__ value_cache_v,
                          const float* __restrict__ key_scale, const float* __restrict__ value_scale,   // INT8 only
                          const int* __restrict__ block_tables,        // [B, max_blocks]
                          const int* __restrict__ context_lens,        // [B]
                          float* __restrict__ part_acc,                // [B, Hq, splits, HD]
                          float* __restrict__ part_ml,                 // [B, Hq, splits, 2]  (max, sum)
                          int Hq, int Hkv, int block_size, int max_blocks, int chunk, float scale) {
  constexpr int LPK = HD / 8;          // lanes per key
  constexpr int KPW = 32 / LPK;        // keys per warp instruction
  constexpr int SLOTS = kPaWarps * KPW;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, splits = gridDim.x;
  const int group = Hq / Hkv;
  const int ctx = context_lens[b];
  const int k_begin = split * chunk;
  const int k_end = min(ctx, k_begin + chunk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, dl = lane % LPK;   // key slot within the warp, dimension slice
  const int slot = warp * KPW + sub;
  __shared__ float sh_acc[SLOTS][kPaHeadsPerPass][HD];
  __shared__ float sh_m[SLOTS][kPaHeadsPerPass], sh_l[SLOTS][kPaHeadsPerPass];
  const int* table = block_tables + (size_t)b * max_blocks;
  const size_t row = (size_t)Hkv * HD;
  const float scale_log2 = scale * 1.4426950408889634f;
  for (int h0 = 0; h0 < group; h0 += kPaHeadsPerPass) {
    const int nh = min(kPaHeadsPerPass, group - h0);
    float qr[kPaHeadsPerPass][8], acc[kPaHeadsPerPass][8], m[kPaHeadsPerPass], l[kPaHeadsPerPass];
#pragma unroll
    for (int h = 0; h < kPaHeadsPerPass; ++h) {
      m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[h][i] = 0.f;
      if (h < nh) {
        const uint4 u = *reinterpret_cast<const uint4*>(q + ((size_t)b * Hq + kvh * group + h0 + h) * HD + dl * 8);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          qr[h][2 * i] = f.x * scale_log2; qr[h][2 * i + 1] = f.y * scale_log2;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) qr[h][i] = 0.f;
      }
    }
    // the trip count is the same for every lane of a warp (the shuffles below name all 32 lanes); a lane group
    // whose key lies beyond the end reads the last valid key and discards the result
    // a fetched key / value slice: 16 bytes of bf16, or 8 bytes of int8 codes and the row's scales
    struct SliceBf { uint4 k, v; };
    struct SliceI8 { uint2 k, v; float ks, vs; };
    using Slice = typename std::conditional<INT8, SliceI8, SliceBf>::type;
    auto fetch = [&](int t0, Slice& s_) {
      const int tk = (t0 + sub < k_end) ? t0 + sub : k_end - 1;
      const int blk = table[tk / block_size];
      const size_t tok = (size_t)blk * block_size + tk % block_size;
      const size_t base = tok * row + (size_t)kvh * HD + dl * 8;
      if constexpr (INT8) {
        s_.k = *reinterpret_cast<const uint2*>(reinterpret_cast<const int8_t*>(key_cache_v) + base);
        s_.v = *reinterpret_cast<const uint2*>(reinterpret_cast<const int8_t*>(value_cache_v) + base);
        s_.ks = __ldg(key_scale + tok * Hkv + kvh);
        s_.vs = __ldg(value_scale + tok * Hkv + kvh);
      } else {
        s_.k = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(key_cache_v) + base);
        s_.v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(value_cache_v) + base);
      }
    };
    // key rows in flight per lane group: hides HBM latency at 16 warps per SM. (Six rows for the int8 cache, whose
    // rows are half as long, cost more in occupancy than they gained: 331 us against 284 us at 64 x 2048 tokens.)
    constexpr int DEPTH = 3;
    Slice pipe[DEPTH];
    const int first = k_begin + warp * KPW;
#pragma unroll
    for (int i = 0; i < DEPTH; ++i)
      if (first + i * SLOTS < k_end) fetch(first + i * SLOTS, pipe[i]);
    for (int t0 = first; t0 < k_end; t0 += SLOTS) {
      const bool valid = t0 + sub < k_end;
      const Slice cur = pipe[0];
#pragma unroll
      for (int i = 0; i + 1 < DEPTH; ++i) pipe[i] = pipe[i + 1];
      if (t0 + DEPTH * SLOTS < k_end) fetch(t0 + DEPTH * SLOTS, pipe[DEPTH - 1]);
      float kf[8], vf[8];
      if constexpr (INT8) {
        const int8_t* kb = reinterpret_cast<const int8_t*>(&cur.k);
        const int8_t* vb = reinterpret_cast<const int8_t*>(&cur.v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          kf[i] = static_cast<float>(kb[i]) * cur.ks;
          vf[i] = static_cast<float>(vb[i]) * cur.vs;
        }
      } else {
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&cur.k);
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&cur.v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a = __bfloat1622float2(k2[i]), c = __bfloat1622float2(v2[i]);
          kf[2 * i] = a.x; kf[2 * i + 1] = a.y; vf[2 * i] = c.x; vf[2 * i + 1] = c.y;
        }
      }
#pragma unroll
      for (int h = 0; h < kPaHeadsPerPass; ++h) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(kf[i], qr[h][i], d);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (valid && h < nh) {
          const float m_new = fmaxf(m[h], d);
          const float alpha = exp2f(m[h] - m_new);     // 0 on the first key (m = -inf)
          const float pexp = exp2f(d - m_new);
          l[h] = l[h] * alpha + pexp;
          m[h] = m_new;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(acc[h][i], alpha, pexp * vf[i]);
        }
      }
    }
    // the lanes of a key group hold identical (m, l): merge the SLOTS streams of this CTA through shared memory
    __syncthreads();
#pragma unroll
    for (int h = 0; h < kPaHeadsPerPass; ++h) {
      if (h < nh) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sh_acc[slot][h][dl * 8 + i] = acc[h][i];
        if (dl == 0) { sh_m[slot][h] = m[h]; sh_l[slot][h] = l[h]; }
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nh * HD; idx += kPaWarps * 32) {
      const int h = idx / HD, d = idx - h * HD;
      float mx = -INFINITY;
#pragma unroll
      for (int s2 = 0; s2 < SLOTS; ++s2) mx = fmaxf(mx, sh_m[s2][h]);
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < SLOTS; ++s2) {
        const float w = sh_m[s2][h] == -INFINITY ? 0.f : exp2f(sh_m[s2][h] - mx);
        num += w * sh_acc[s2][h][d];
        den += w * sh_l[s2][h];
      }
      const size_t o = ((size_t)b * Hq + kvh * group + h0 + h) * splits + split;
      part_acc[o * HD + d] = num;
      if (d == 0) { part_ml[o * 2] = mx; part_ml[o * 2 + 1] = den; }
    }
  }
}

// out[b, h, :] = merge over splits of (acc, max, sum)
template <int HD>
__global__ void paged_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                     __nv_bfloat16* __restrict__ out, int splits) {
  const size_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float mx = -INFINITY;
  for (int s2 = 0; s2 < splits; ++s2) mx = fmaxf(mx, part_ml[(bh * splits + s2) * 2]);
  float num = 0.f, den = 0.f;
  for (int s2 = 0; s2 < splits; ++s2) {
    const float ms = part_ml[(bh * splits + s2) * 2];
    const float w = ms == -INFINITY ? 0.f : exp2f(ms - mx);
    num += w * part_acc[(bh * splits + s2) * HD + d];
    den += w * part_ml[(bh * splits + s2) * 2 + 1];
  }
  out[bh * HD + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
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

// The same gather out of an int8 cache, de-quantised to bf16: one warp per (token, head).
__global__ void gather_cache_int8_kernel(const int8_t* __restrict__ cache, const float* __restrict__ scale,
                                         const int* __restrict__ block_tables, const int* __restrict__ cu_lens,
                                         __nv_bfloat16* __restrict__ out, int block_size, int max_blocks, int heads, int hd) {
  const int b = blockIdx.y;
  const int start = cu_lens[b], n = cu_lens[b + 1] - start;
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < (long long)n * heads; w += warps) {
    const int tok = (int)(w / heads), h = (int)(w - (long long)tok * heads);
    const int blk = block_tables[(size_t)b * max_blocks + tok / block_size];
    const size_t slot = (size_t)blk * block_size + tok % block_size;
    const float sc = scale[slot * heads + h];
    const int8_t* src = cache + (slot * heads + h) * hd;
    __nv_bfloat16* dst = out + ((size_t)(start + tok) * heads + h) * hd;
    for (int d = lane; d < hd; d += 32) dst[d] = __float2bfloat16(static_cast<float>(src[d]) * sc);
  }
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// key / value [T, heads, hd] bf16 -> int8 caches [slots, heads, hd] + scales [slots, heads]
int mfb_reshape_and_cache_int8(const void* key, const void* value, void* key_cache, void* value_cache, float* key_scale,
                               float* value_scale, const int* slot_mapping, long long T, int heads, int hd,
                               long long k_stride, long long v_stride, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long blocks = (T * heads * 32 + 255) / 256;
  reshape_and_cache_int8_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
      (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, (int8_t*)key_cache, (int8_t*)value_cache, key_scale,
      value_scale, slot_mapping, T, heads, hd, k_stride, v_stride);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_gather_cache_int8(const void* cache, const float* scale, const int* block_tables, const int* cu_lens, void* out,
                          int B, int max_len, int block_size, int max_blocks, int heads, int hd, cudaStream_t stream) {
  if (B <= 0 || max_len <= 0) return 0;
  long long per = ((long long)max_len * heads * 32 + 255) / 256;
  if (per > 1024) per = 1024;
  dim3 grid((unsigned)per, B);
  gather_cache_int8_kernel<<<grid, 256, 0, stream>>>((const int8_t*)cache, scale, block_tables, cu_lens,
                                                     (__nv_bfloat16*)out, block_size, max_blocks, heads, hd);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

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

// Number of key splits used for a batch of B sequences with at most max_blocks * block_size cached tokens.
int mfb_paged_decode_splits(int B, int Hkv, int block_size, int max_blocks) {
  const long long max_ctx = (long long)max_blocks * block_size;
  const long long ctas = (long long)B * Hkv;
  long long splits = (148 * 8 + ctas - 1) / ctas;           // aim at ~8 CTAs per SM
  const long long by_len = (max_ctx + 255) / 256;           // at least 256 keys per split
  if (splits > by_len) splits = by_len;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  return (int)splits;
}

// fp32 scratch bytes for mfb_paged_decode_attention: partial outputs and (max, sum) per split.
long long mfb_paged_decode_scratch_bytes(int B, int Hq, int hd, int splits) {
  return (long long)B * Hq * splits * (hd + 2) * 4;
}

// key_scale / value_scale non-null: the caches hold int8 codes with one fp32 scale per (slot, KV head).
int mfb_paged_decode_attention_ex(const void* q, const void* key_cache, const void* value_cache, const float* key_scale,
                                  const float* value_scale, const int* block_tables, const int* context_lens, void* out,
                                  void* scratch, int splits, int B, int Hq, int Hkv, int hd, int block_size, int max_blocks,
                                  float scale, cudaStream_t stream) {
  if (Hq % Hkv || Hq / Hkv > kPaMaxGroup || (hd != 128 && hd != 64) || splits < 1) {
    mfb_host::set_error("paged_decode_attention: unsupported Hq=%d Hkv=%d hd=%d splits=%d", Hq, Hkv, hd, splits);
    return 1;
  }
  if (B <= 0) return 0;
  const long long max_ctx = (long long)max_blocks * block_size;
  int chunk = (int)((max_ctx + splits - 1) / splits);
  chunk = (chunk + 63) / 64 * 64;
  float* part_acc = reinterpret_cast<float*>(scratch);
  float* part_ml = part_acc + (size_t)B * Hq * splits * hd;
  dim3 grid(splits, Hkv, B);
  const bool i8 = key_scale != nullptr;
  if (i8 && !value_scale) { mfb_host::set_error("paged_decode_attention: int8 cache needs both scale arrays"); return 1; }
#define MFB_PA_LAUNCH(HD_, I8_)                                                                                       \
  paged_decode_split_kernel<HD_, I8_><<<grid, kPaWarps * 32, 0, stream>>>(                                            \
      (const __nv_bfloat16*)q, key_cache, value_cache, key_scale, value_scale, block_tables, context_lens, part_acc,  \
      part_ml, Hq, Hkv, block_size, max_blocks, chunk, scale)
  if (hd == 128) {
    if (i8) MFB_PA_LAUNCH(128, true); else MFB_PA_LAUNCH(128, false);
    paged_combine_kernel<128><<<B * Hq, 128, 0, stream>>>(part_acc, part_ml, (__nv_bfloat16*)out, splits);
  } else {
    if (i8) MFB_PA_LAUNCH(64, true); else MFB_PA_LAUNCH(64, false);
    paged_combine_kernel<64><<<B * Hq, 64, 0, stream>>>(part_acc, part_ml, (__nv_bfloat16*)out, splits);
  }
#undef MFB_PA_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// out[row, :] = merge of the `splits` partial results of every (sequence, query head) row.
int mfb_paged_combine(const float* part_acc, const float* part_ml, void* out, int splits, int rows, int hd,
                      cudaStream_t stream) {
  if (hd == 128) paged_combine_kernel<128><<<rows, 128, 0, stream>>>(part_acc, part_ml, (__nv_bfloat16*)out, splits);
  else if (hd == 64) paged_combine_kernel<64><<<rows, 64, 0, stream>>>(part_acc, part_ml, (__nv_bfloat16*)out, splits);
  else { mfb_host::set_error("paged_combine: head dim %d", hd); return 1; }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_paged_decode_attention(const void* q, const void* key_cache, const void* value_cache, const int* block_tables,
                               const int* context_lens, void* out, void* scratch, int splits, int B, int Hq, int Hkv,
                               int hd, int block_size, int max_blocks, float scale, cudaStream_t stream) {
  return mfb_paged_decode_attention_ex(q, key_cache, value_cache, nullptr, nullptr, block_tables, context_lens, out,
                                       scratch, splits, B, Hq, Hkv, hd, block_size, max_blocks, scale, stream);
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
