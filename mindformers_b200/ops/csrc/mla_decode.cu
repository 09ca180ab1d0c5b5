// Multi-latent attention decode over a paged latent cache (sm_100a, tcgen05 + TMA).
//
// Every cached token is one row [kv_lora 512 | rope 64] of bf16 shared by all heads. With the up-projections
// absorbed into the query, one decode step is, per sequence and head h:
//     s[t]   = scale * <q[h, 0:576], c[t, 0:576]>          t < len
//     o[h,:] = sum_t softmax(s)[t] * c[t, 0:512]
// A CTA handles (split of the sequence, chunk of 16 heads, sequence). The products are laid out TRANSPOSED so
// that the token dimension, not the (small) head count, fills the 128 rows of the tensor core:
//     S^T [128 tokens x 16 heads]   = C_tile [128 x 576] (A, K-major) . Q^T (B, K-major)          -> TMEM, 16 columns
//     O^T [512 x 16]  (4 x M=128)  += C_tile^T (A, MN-major: the same bytes) . P^T [16 heads x 128 tokens] (B, K-major)
// Softmax threads own one token row each; the per-head maximum over the 128 tokens of a tile is a shuffle
// + shared-memory reduction, per-head sums stay thread-local until the end. O^T is rescaled in TMEM only when
// a head's maximum grew by more than 2^8 (as in the flash-attention kernel).
//
// A tile of 128 tokens is 147 KB, so a second tile cannot be prefetched while one is resident, and the chain
// S^T -> softmax -> O^T of a tile leaves the memory system idle. Instead the cache tile is STREAMED twice through a
// small ring of 32 KB slots (first five units for S^T: four column pairs + the rope columns; then the four pairs
// again for O^T, which hit L2), and the kernel is sized so that TWO CTAs share an SM (88 KB of shared memory and
// 256 TMEM columns each): while one CTA sits in its softmax, the other one streams.
//
// Roles (192 threads): warp 0 = TMA producer (block-table lookups), warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = softmax / rescale / epilogue. Every wait is bounded (see common.cuh). Partial results of the splits
// are merged by mla_combine_kernel.
#include "common.cuh"

namespace mfb {

constexpr int kMlaThreads = 192;
constexpr int kMlaTile = 128;              // tokens per tile
constexpr int kMlaHeads = 16;              // heads per CTA
constexpr int kMlaRank = 512;
constexpr int kMlaRope = 64;
constexpr int kMlaDim = kMlaRank + kMlaRope;
constexpr int kMlaSub = kMlaTile * 128;    // [128 tokens][64 columns] swizzled sub-tile, 16 KB
constexpr int kMlaUnit = 2 * kMlaSub;      // ring slot: a pair of sub-tiles (128 columns)
constexpr int kMlaSlots = 2;
constexpr int kMlaPBytes = 2 * kMlaHeads * 128;   // P^T: two [16 heads][64 tokens] K-major sub-tiles
constexpr int kMlaTmemCols = 256;
constexpr int kMlaQSub = kMlaHeads * 128;  // [16 heads][64 columns], 2 KB
constexpr int kMlaQBytes = 9 * kMlaQSub;
constexpr float kMlaRescale = 8.0f;

struct MlaArgs {
  const int* block_tables;   // [B, max_blocks]
  const int* context_lens;   // [B]
  int max_blocks, block_size, num_heads, splits;
  float scale_log2;
  float* part_o;             // [B, splits, num_heads, 512] unnormalised
  float* part_ml;            // [B, splits, num_heads, 2]: running max (log2 units), sum
  int* status;
};

__device__ __forceinline__ float mla_ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kMlaThreads, 2)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmC, const MlaArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sRing = smem;                               // 2 x 32 KB
  uint8_t* sP = sRing + kMlaSlots * kMlaUnit;          // 4 KB
  uint8_t* sQ = sP + kMlaPBytes;                       // 18 KB
  float* red = reinterpret_cast<float*>(sQ + kMlaQBytes);          // [4 warps][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 4 * kMlaHeads);
  uint64_t* q_full = bars;                  // 1
  uint64_t* full = bars + 1;                // up to 5
  uint64_t* empty = bars + 6;               // up to 5
  uint64_t* s_full = bars + 11;             // 2
  uint64_t* s_empty = bars + 13;            // 2
  uint64_t* p_ready = bars + 15;            // 1
  uint64_t* pv_done = bars + 16;            // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, chunk = blockIdx.y, b = blockIdx.z;
  const int len = args.context_lens[b];
  const int n_tiles_all = (len + kMlaTile - 1) / kMlaTile;
  const int per = (n_tiles_all + args.splits - 1) / args.splits;
  const int t0 = split * per;
  const int t1 = (t0 + per < n_tiles_all) ? t0 + per : n_tiles_all;
  const int n_tiles = t1 > t0 ? t1 - t0 : 0;
  const int head0 = chunk * kMlaHeads;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kMlaSlots; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 128);
    }
    mbar_init(smem_u32(p_ready), 128);
    mbar_init(smem_u32(pv_done), 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), kMlaTmemCols);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_O = tmem_base;              // 4 blocks of 16 columns, 32 apart
  const uint32_t tmem_S = tmem_base + 128;        // 2 buffers of 16 columns, 32 apart

  if (warp == 0) {
    // ------------------------------------ producer ------------------------------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t qb = smem_u32(q_full);
      mbar_expect_tx(qb, kMlaQBytes);
      for (int c = 0; c < 9; ++c)
        tma_load_2d(smem_u32(sQ) + c * kMlaQSub, &tmQ, qb, c * 64, b * args.num_heads + head0);
      const int bs = args.block_size;
      const int pages = kMlaTile / bs;            // pages per tile (block_size divides 128)
      const int* table = args.block_tables + static_cast<size_t>(b) * args.max_blocks;
      uint32_t unit = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int tok0 = (t0 + j) * kMlaTile;
        int page_row[8];
        const int first_page = table[tok0 / bs];
        for (int i = 0; i < pages; ++i) {
          // pages past the end of the sequence may be unallocated: read the tile's first page instead (masked)
          const int pg = (tok0 + i * bs < len) ? table[tok0 / bs + i] : first_page;
          page_row[i] = pg * bs;
        }
        // two passes: [P0 P1 P2 P3 R] for S^T, then [P0 P1 P2 P3] again for O^T
        for (int u = 0; u < 9 && ok; ++u) {
          const int slot = unit % kMlaSlots;
          const uint32_t ph = (unit / kMlaSlots) & 1;
          ok = mbar_wait(smem_u32(&empty[slot]), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full[slot]);
          const uint32_t dst = smem_u32(sRing + slot * kMlaUnit);
          const bool rope = (u == 4);
          const int col0 = rope ? kMlaRank : (u < 4 ? u : u - 5) * 128;
          mbar_expect_tx(fb, rope ? kMlaSub : kMlaUnit);
          for (int i = 0; i < pages; ++i) {
            tma_load_2d(dst + i * bs * 128, &tmC, fb, col0, page_row[i]);
            if (!rope) tma_load_2d(dst + kMlaSub + i * bs * 128, &tmC, fb, col0 + 64, page_row[i]);
          }
          ++unit;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(kMlaTile, kMlaHeads, 0, 0);   // A = cache K-major, B = Q K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(kMlaTile, kMlaHeads, 1, 0);  // A = cache MN-major, B = P^T K-major
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      const uint32_t qa = smem_u32(sQ), pa = smem_u32(sP);
      uint32_t unit = 0;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int sb = j & 1;
        const uint32_t sph = (j >> 1) & 1;
        ok = mbar_wait(smem_u32(&s_empty[sb]), sph ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        // ---- S^T = C . Q^T over the five units of the first pass ----
        for (int u = 0; u < 5 && ok; ++u) {
          const int slot = unit % kMlaSlots;
          const uint32_t ph = (unit / kMlaSlots) & 1;
          ok = mbar_wait(smem_u32(&full[slot]), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t ca = smem_u32(sRing + slot * kMlaUnit);
          const bool rope = (u == 4);
          const int ksteps = rope ? 4 : 8;
          const int qsub0 = rope ? 8 : 2 * u;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (k < ksteps) {
              const uint64_t a_desc = umma_desc_kmajor_sw128(ca + (k >> 2) * kMlaSub + (k & 3) * 32);
              const uint64_t b_desc = umma_desc_kmajor_sw128(qa + (qsub0 + (k >> 2)) * kMlaQSub + (k & 3) * 32);
              umma_f16_ss(tmem_S + sb * 32, a_desc, b_desc, IDESC_S, (u > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&empty[slot]));
          ++unit;
        }
        if (!ok) break;
        umma_commit(smem_u32(&s_full[sb]));
        // ---- O^T += C^T . P^T over the four units of the second pass ----
        ok = mbar_wait(smem_u32(p_ready), j & 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        for (int m = 0; m < 4 && ok; ++m) {
          const int slot = unit % kMlaSlots;
          const uint32_t ph = (unit / kMlaSlots) & 1;
          ok = mbar_wait(smem_u32(&full[slot]), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t ca = smem_u32(sRing + slot * kMlaUnit);
#pragma unroll
          for (int k = 0; k < kMlaTile / 16; ++k) {
            const uint64_t a_desc = umma_desc_mnmajor_sw128(ca + k * 16 * 128, kMlaSub);
            const uint64_t b_desc = umma_desc_kmajor_sw128(pa + (k >> 2) * (kMlaHeads * 128) + (k & 3) * 32);
            umma_f16_ss(tmem_O + m * 32, a_desc, b_desc, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty[slot]));
          ++unit;
        }
        if (!ok) break;
        umma_commit(smem_u32(pv_done));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------ softmax / epilogue ------------------------------------
    const int ew = warp & 3;
    const int row = ew * 32 + lane;                 // token row of S^T, dv row of O^T
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    float m_used[kMlaHeads], l_part[kMlaHeads];
#pragma unroll
    for (int h = 0; h < kMlaHeads; ++h) { m_used[h] = -INFINITY; l_part[h] = 0.f; }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      const uint32_t sph = (j >> 1) & 1;
      ok = mbar_wait(smem_u32(&s_full[sb]), sph, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, 128, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[16];
      tmem_ld_32x32b_x16(tmem_S + sb * 32 + lane_base, sr);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&s_empty[sb]));
      float s[kMlaHeads];
      const bool valid = (t0 + j) * kMlaTile + row < len;
#pragma unroll
      for (int h = 0; h < kMlaHeads; ++h) s[h] = valid ? __uint_as_float(sr[h]) * args.scale_log2 : -INFINITY;
      // per-head maximum over the 128 tokens of the tile
#pragma unroll
      for (int h = 0; h < kMlaHeads; ++h) {
        const float w = warp_max(s[h]);
        if (lane == 0) red[ew * kMlaHeads + h] = w;
      }
      named_bar_sync(1, 128);
      float alpha[kMlaHeads];
      bool any_rescale = false;
#pragma unroll
      for (int h = 0; h < kMlaHeads; ++h) {
        const float mx = fmaxf(fmaxf(red[h], red[kMlaHeads + h]), fmaxf(red[2 * kMlaHeads + h], red[3 * kMlaHeads + h]));
        alpha[h] = 1.f;
        if (m_used[h] == -INFINITY) {
          m_used[h] = mx;                           // first tile with a valid token (nothing accumulated yet)
        } else if (mx > m_used[h] + kMlaRescale) {
          alpha[h] = mla_ex2(m_used[h] - mx);
          m_used[h] = mx;
          any_rescale = true;
        }
      }
#pragma unroll
      for (int h = 0; h < kMlaHeads; ++h) {
        const float neg_m = (m_used[h] == -INFINITY) ? 0.f : -m_used[h];
        s[h] = valid ? mla_ex2(s[h] + neg_m) : 0.f;
        l_part[h] = l_part[h] * alpha[h] + s[h];
      }
      if (j > 0) {
        // the previous O^T update has completed: P^T may be overwritten and O^T touched
        ok = mbar_wait(smem_u32(pv_done), (j - 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
        if (ok && any_rescale) {
          tc_fence_after();
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(tmem_O + lane_base + m * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < kMlaHeads; ++h) r[h] = __float_as_uint(__uint_as_float(r[h]) * alpha[h]);
            tmem_st_32x32b_x16(tmem_O + lane_base + m * 32, r);
          }
          tmem_st_wait();
        }
      }
      ok = named_bar_and(2, 128, ok);               // also orders the reads of `red` before the next tile's writes
      if (!ok) break;
      // P^T[h][token] as a K-major operand: sub-tile of 64 tokens, row h of 128 bytes, 16-byte chunks swizzled by row
      {
        uint8_t* pcol = sP + (row >> 6) * (kMlaHeads * 128) + (row & 7) * 2;
        const int chunk = (row & 63) >> 3;
#pragma unroll
        for (int h = 0; h < kMlaHeads; ++h)
          *reinterpret_cast<__nv_bfloat16*>(pcol + h * 128 + ((chunk ^ (h & 7)) << 4)) = __float2bfloat16_rn(s[h]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(p_ready));
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(smem_u32(pv_done), (n_tiles - 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, 128, ok);
    }
    // per-head sums over the 128 token rows
    float l_tot[kMlaHeads];
#pragma unroll
    for (int h = 0; h < kMlaHeads; ++h) {
      const float w = warp_sum(l_part[h]);
      if (lane == 0) red[ew * kMlaHeads + h] = w;
    }
    named_bar_sync(1, 128);
#pragma unroll
    for (int h = 0; h < kMlaHeads; ++h)
      l_tot[h] = (red[h] + red[kMlaHeads + h]) + (red[2 * kMlaHeads + h] + red[3 * kMlaHeads + h]);
    const size_t ps = static_cast<size_t>(b) * args.splits + split;
    if (row < kMlaHeads && head0 + row < args.num_heads) {
      float mh = -INFINITY, lh = 0.f;
#pragma unroll
      for (int h = 0; h < kMlaHeads; ++h)
        if (h == row) { mh = m_used[h]; lh = l_tot[h]; }
      if (!ok || n_tiles == 0) { mh = -INFINITY; lh = 0.f; }
      float* ml = args.part_ml + (ps * args.num_heads + head0 + row) * 2;
      ml[0] = mh;
      ml[1] = lh;
    }
    if (ok && n_tiles > 0) {
      tc_fence_after();
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(tmem_O + lane_base + m * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < kMlaHeads; ++h) {
          if (head0 + h < args.num_heads)
            args.part_o[(ps * args.num_heads + head0 + h) * kMlaRank + m * 128 + row] = __uint_as_float(r[h]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kMlaTmemCols);
  }
}

// out[b, h, :] = sum_s 2^(m_s - M) o_s / sum_s 2^(m_s - M) l_s
__global__ void __launch_bounds__(128)
mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                   int splits, int num_heads) {
  const int h = blockIdx.x, b = blockIdx.y;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) {
    const float* ml = part_ml + ((static_cast<size_t>(b) * splits + s) * num_heads + h) * 2;
    if (ml[1] > 0.f) M = fmaxf(M, ml[0]);
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float L = 0.f;
  for (int s = 0; s < splits; ++s) {
    const size_t idx = (static_cast<size_t>(b) * splits + s) * num_heads + h;
    const float l = part_ml[idx * 2 + 1];
    if (!(l > 0.f)) continue;
    const float w = exp2f(part_ml[idx * 2] - M);
    L += w * l;
    const float4 v = reinterpret_cast<const float4*>(part_o + idx * kMlaRank)[threadIdx.x];
    acc[0] += w * v.x; acc[1] += w * v.y; acc[2] += w * v.z; acc[3] += w * v.w;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(out + (static_cast<size_t>(b) * num_heads + h) * kMlaRank) + threadIdx.x * 2;
  dst[0] = __floats2bfloat162_rn(acc[0] * inv, acc[1] * inv);
  dst[1] = __floats2bfloat162_rn(acc[2] * inv, acc[3] * inv);
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// Kernel variant: 0 = one CTA per (sequence, split, head chunk), two passes over the cache (this file);
// 1 = a cluster of two CTAs that split the latent columns, one pass (mla_decode_cluster.cu).
static int g_mla_variant = 0;
int mfb_mla_cluster_splits(int B, int num_heads, int max_len);
int mfb_mla_decode_cluster_launch(const void* q, const void* cache, const int* block_tables, const int* context_lens,
                                  float* part_o, float* part_ml, int splits, int B, int num_heads, int num_blocks,
                                  int block_size, int max_blocks, float scale, int* status, cudaStream_t stream);
void mfb_mla_decode_set_variant(int v) { g_mla_variant = v == 1 ? 1 : 0; }
int mfb_mla_decode_get_variant() { return g_mla_variant; }

// Number of sequence splits that fills the GPU for a batch of B sequences of up to max_len tokens.
int mfb_mla_decode_splits(int B, int num_heads, int max_len) {
  if (g_mla_variant == 1) return mfb_mla_cluster_splits(B, num_heads, max_len);
  // cost of a choice = waves of CTAs over the 2 x 148 resident CTAs x (tiles per CTA + about one tile of fixed work per CTA)
  const int chunks = (num_heads + kMlaHeads - 1) / kMlaHeads;
  const int tiles = (max_len + kMlaTile - 1) / kMlaTile;
  int best = 1;
  long long best_cost = -1;
  for (int s = 1; s <= tiles && s <= 32; ++s) {
    const long long ctas = static_cast<long long>(B) * chunks * s;
    const long long waves = (ctas + 295) / 296;          // two CTAs per SM
    const long long cost = waves * ((tiles + s - 1) / s + 1);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
  }
  return best;
}

long long mfb_mla_decode_scratch_bytes(int B, int num_heads, int splits) {
  return static_cast<long long>(B) * splits * num_heads * (kMlaRank + 2) * 4;
}

// q: [B, num_heads, 576] bf16 (absorbed query: latent part then rope part); cache: [num_blocks, block_size, 576] bf16;
// block_tables: [B, max_blocks] int32; context_lens: [B] int32 (tokens in the cache, the new one included);
// out: [B, num_heads, 512] bf16 (latent-space output); scratch: mfb_mla_decode_scratch_bytes.
int mfb_mla_decode_attention(const void* q, const void* cache, const int* block_tables, const int* context_lens, void* out,
                             void* scratch, int splits, int B, int num_heads, int num_blocks, int block_size,
                             int max_blocks, float scale, int* status, cudaStream_t stream) {
  if (B < 1 || num_heads < 1 || splits < 1 || (block_size != 16 && block_size != 32 && block_size != 64 && block_size != 128)) {
    mfb_host::set_error("mla_decode: unsupported B=%d heads=%d splits=%d block_size=%d", B, num_heads, splits, block_size);
    return 1;
  }
  CUtensorMap tQ, tC;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = mfb_host::make_tmap_2d(&tQ, q, 2, BF, (uint64_t)B * num_heads, kMlaDim, kMlaDim, kMlaHeads, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tC, cache, 2, BF, (uint64_t)num_blocks * block_size, kMlaDim, kMlaDim, block_size, 64))) return 30 + rc;
  MlaArgs a;
  a.block_tables = block_tables; a.context_lens = context_lens; a.max_blocks = max_blocks; a.block_size = block_size;
  a.num_heads = num_heads; a.splits = splits; a.scale_log2 = scale * 1.4426950408889634f;
  a.part_o = reinterpret_cast<float*>(scratch);
  a.part_ml = a.part_o + static_cast<size_t>(B) * splits * num_heads * kMlaRank;
  a.status = status;
  if (g_mla_variant == 1) {
    rc = mfb_mla_decode_cluster_launch(q, cache, block_tables, context_lens, a.part_o, a.part_ml, splits, B, num_heads,
                                       num_blocks, block_size, max_blocks, scale, status, stream);
    if (rc) return rc;
    mla_combine_kernel<<<dim3(num_heads, B), 128, 0, stream>>>(a.part_o, a.part_ml, reinterpret_cast<__nv_bfloat16*>(out),
                                                                splits, num_heads);
    return cudaGetLastError() == cudaSuccess ? 0 : 12;
  }
  constexpr int SMEM = kMlaSlots * kMlaUnit + kMlaPBytes + kMlaQBytes + 4 * kMlaHeads * 4 + 18 * 8 + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("mla_decode: cannot raise shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  const int chunks = (num_heads + kMlaHeads - 1) / kMlaHeads;
  dim3 grid(splits, chunks, B);
  mla_decode_kernel<<<grid, kMlaThreads, SMEM, stream>>>(tQ, tC, a);
  if (cudaGetLastError() != cudaSuccess) { mfb_host::set_error("mla_decode: launch failed"); return 11; }
  mla_combine_kernel<<<dim3(num_heads, B), 128, 0, stream>>>(a.part_o, a.part_ml, reinterpret_cast<__nv_bfloat16*>(out), splits,
                                                              num_heads);
  return cudaGetLastError() == cudaSuccess ? 0 : 12;
}

}  // extern "C"
