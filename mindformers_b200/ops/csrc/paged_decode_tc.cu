// Single-query (decode) attention over a paged bf16 KV cache on the tensor cores (sm_100a, tcgen05 + TMA), head
// dim 128, grouped-query attention with up to 16 query heads per KV head.
//
// Cache layout: key_cache / value_cache [num_blocks, block_size, kv_heads, 128]; a sequence's blocks come from its
// block table. A CTA handles (split of the sequence, KV head, sequence) and walks its tokens in tiles of 128. As in
// the latent-cache kernel the products are TRANSPOSED, so that the tokens, not the few query heads, fill the 128
// rows of the tensor core:
//     S^T [128 tokens x 16 heads] = K_tile [128 x 128] (A, K-major) . Q^T (B, K-major)            -> TMEM, 16 columns
//     O^T [128 dims x 16 heads]  += V_tile^T (A, MN-major: the tile as it lies in the cache) . P^T [16 heads x 128 tokens]
// The 16 columns are the query heads of the KV head's group (rows of Q beyond the group belong to the next KV head
// or are zero fill: their columns are computed and never stored). Softmax threads own one token row each; the
// per-head maximum over a tile is a shuffle + shared-memory reduction; O^T is rescaled in tensor memory only when a
// head's maximum grew by more than 2^8.
//
// K and V tiles (32 KB each) stream through a ring of three slots in the order the tensor core consumes them:
// K(0), then K(j + 1), V(j) for every tile j, so S^T of the next tile is computed while the softmax threads work on
// this one. Two CTAs share an SM (105 KB of shared memory and 128 TMEM columns each): while one waits for its
// softmax, the other streams. The kernel is bandwidth-bound: its roofline is the K/V bytes over the HBM bandwidth.
//
// Roles (192 threads): warp 0 TMA producer (block-table lookups), warp 1 MMA issuer + TMEM owner, warps 2..5 softmax
// / rescale / epilogue. Every wait is bounded. Partial results of the splits go to the same scratch layout as the
// CUDA-core kernel's and are merged by its combine kernel.
#include "common.cuh"

namespace mfb {
namespace pdt {

constexpr int kThreads = 192;
constexpr int kTile = 128;                 // tokens per tile
constexpr int kHeads = 16;                 // query-head columns per CTA
constexpr int kHd = 128;
constexpr int kSub = kTile * 128;          // [128 tokens][64 dims] swizzled sub-tile, 16 KB
constexpr int kUnit = 2 * kSub;            // a K or V tile
constexpr int kSlots = 3;
constexpr int kPBytes = 2 * kHeads * 128;  // P^T: two [16 heads][64 tokens] K-major sub-tiles
constexpr int kQBytes = 2 * kHeads * 128;  // Q: two [16 heads][64 dims] sub-tiles
constexpr int kTmemCols = 128;
constexpr float kRescale = 8.0f;
constexpr int kSmem = kSlots * kUnit + kPBytes + kQBytes + 4 * kHeads * 4 + 16 * 8 + 16 + 1024;

struct Args {
  const int* block_tables;   // [B, max_blocks]
  const int* context_lens;   // [B]
  int max_blocks, block_size, num_q_heads, num_kv_heads, group, splits;
  float scale_log2;
  float* part_acc;           // [B, Hq, splits, 128] unnormalised
  float* part_ml;            // [B, Hq, splits, 2]: running max (log2 units), sum
  int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kThreads, 2)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sRing = smem;                               // 3 x 32 KB
  uint8_t* sP = sRing + kSlots * kUnit;                // 4 KB
  uint8_t* sQ = sP + kPBytes;                          // 4 KB
  float* red = reinterpret_cast<float*>(sQ + kQBytes); // [4 warps][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 4 * kHeads);
  uint64_t* q_full = bars;                  // 1
  uint64_t* full = bars + 1;                // 3
  uint64_t* empty = bars + 4;               // 3
  uint64_t* s_full = bars + 7;              // 2
  uint64_t* s_empty = bars + 9;             // 2
  uint64_t* p_ready = bars + 11;            // 1
  uint64_t* pv_done = bars + 12;            // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int len = args.context_lens[b];
  const int n_tiles_all = (len + kTile - 1) / kTile;
  const int per = (n_tiles_all + args.splits - 1) / args.splits;
  const int t0 = split * per;
  const int t1 = (t0 + per < n_tiles_all) ? t0 + per : n_tiles_all;
  const int n_tiles = t1 > t0 ? t1 - t0 : 0;
  const int head0 = kvh * args.group;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kSlots; ++s) {
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
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_O = tmem_base;              // 16 columns
  const uint32_t tmem_S = tmem_base + 32;         // 2 buffers of 16 columns, 32 apart

  if (warp == 0) {
    // ------------------------------------ producer ------------------------------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t qb = smem_u32(q_full);
      mbar_expect_tx(qb, kQBytes);
      for (int c = 0; c < 2; ++c)
        tma_load_2d(smem_u32(sQ) + c * (kHeads * 128), &tmQ, qb, c * 64, b * args.num_q_heads + head0);
      const int bs = args.block_size;
      const int pages = kTile / bs;               // pages per tile (block_size divides 128)
      const int* table = args.block_tables + static_cast<size_t>(b) * args.max_blocks;
      const int col0 = kvh * kHd;
      uint32_t unit = 0;
      bool ok = true;
      // one K or V tile into the next ring slot
      auto load_tile = [&](const CUtensorMap* tm, int j) {
        const int slot = unit % kSlots;
        const uint32_t ph = (unit / kSlots) & 1;
        ok = mbar_wait(smem_u32(&empty[slot]), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) return;
        const int tok0 = (t0 + j) * kTile;
        const int first_page = table[tok0 / bs];
        const uint32_t fb = smem_u32(&full[slot]);
        const uint32_t dst = smem_u32(sRing + slot * kUnit);
        mbar_expect_tx(fb, kUnit);
        for (int i = 0; i < pages; ++i) {
          // pages past the end of the sequence may be unallocated: read the tile's first page instead (masked)
          int pg = (tok0 + i * bs < len) ? table[tok0 / bs + i] : first_page;
          if (pg < 0) pg = first_page;
          tma_load_2d(dst + i * bs * 128, tm, fb, col0, pg * bs);
          tma_load_2d(dst + kSub + i * bs * 128, tm, fb, col0 + 64, pg * bs);
        }
        ++unit;
      };
      load_tile(&tmK, 0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) load_tile(&tmK, j + 1);
        if (ok) load_tile(&tmV, j);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(kTile, kHeads, 0, 0);    // A = K tile K-major, B = Q K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(kHd, kHeads, 1, 0);     // A = V tile MN-major, B = P^T K-major
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      const uint32_t qa = smem_u32(sQ), pa = smem_u32(sP);
      uint32_t unit = 0;
      // S^T(j) = K(j) . Q^T into score buffer j & 1
      auto scores = [&](int j) {
        const int sb = j & 1;
        const uint32_t sph = (j >> 1) & 1;
        ok = mbar_wait(smem_u32(&s_empty[sb]), sph ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) return;
        const int slot = unit % kSlots;
        const uint32_t ph = (unit / kSlots) & 1;
        ok = mbar_wait(smem_u32(&full[slot]), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) return;
        tc_fence_after();
        const uint32_t ka = smem_u32(sRing + slot * kUnit);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t a_desc = umma_desc_kmajor_sw128(ka + (k >> 2) * kSub + (k & 3) * 32);
          const uint64_t b_desc = umma_desc_kmajor_sw128(qa + (k >> 2) * (kHeads * 128) + (k & 3) * 32);
          umma_f16_ss(tmem_S + sb * 32, a_desc, b_desc, IDESC_S, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&empty[slot]));
        umma_commit(smem_u32(&s_full[sb]));
        ++unit;
      };
      if (ok) scores(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) scores(j + 1);
        if (!ok) break;
        // ---- O^T += V(j)^T . P^T(j) ----
        ok = mbar_wait(smem_u32(p_ready), j & 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        const int slot = unit % kSlots;
        const uint32_t ph = (unit / kSlots) & 1;
        ok = mbar_wait(smem_u32(&full[slot]), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t va = smem_u32(sRing + slot * kUnit);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {
          const uint64_t a_desc = umma_desc_mnmajor_sw128(va + k * 16 * 128, kSub);
          const uint64_t b_desc = umma_desc_kmajor_sw128(pa + (k >> 2) * (kHeads * 128) + (k & 3) * 32);
          umma_f16_ss(tmem_O, a_desc, b_desc, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&empty[slot]));
        umma_commit(smem_u32(pv_done));
        ++unit;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------ softmax / epilogue ------------------------------------
    const int ew = warp & 3;
    const int row = ew * 32 + lane;                 // token row of S^T, dim row of O^T
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    float m_used[kHeads], l_part[kHeads];
#pragma unroll
    for (int h = 0; h < kHeads; ++h) { m_used[h] = -INFINITY; l_part[h] = 0.f; }
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
      float s[kHeads];
      const bool valid = (t0 + j) * kTile + row < len;
#pragma unroll
      for (int h = 0; h < kHeads; ++h) s[h] = valid ? __uint_as_float(sr[h]) * args.scale_log2 : -INFINITY;
      // per-head maximum over the 128 tokens of the tile
#pragma unroll
      for (int h = 0; h < kHeads; ++h) {
        const float w = warp_max(s[h]);
        if (lane == 0) red[ew * kHeads + h] = w;
      }
      named_bar_sync(1, 128);
      float alpha[kHeads];
      bool any_rescale = false;
#pragma unroll
      for (int h = 0; h < kHeads; ++h) {
        const float mx = fmaxf(fmaxf(red[h], red[kHeads + h]), fmaxf(red[2 * kHeads + h], red[3 * kHeads + h]));
        alpha[h] = 1.f;
        if (m_used[h] == -INFINITY) {
          m_used[h] = mx;                           // first tile with a valid token (nothing accumulated yet)
        } else if (mx > m_used[h] + kRescale) {
          alpha[h] = ex2(m_used[h] - mx);
          m_used[h] = mx;
          any_rescale = true;
        }
      }
#pragma unroll
      for (int h = 0; h < kHeads; ++h) {
        const float neg_m = (m_used[h] == -INFINITY) ? 0.f : -m_used[h];
        s[h] = valid ? ex2(s[h] + neg_m) : 0.f;
        l_part[h] = l_part[h] * alpha[h] + s[h];
      }
      if (j > 0) {
        // the previous O^T update has completed: P^T may be overwritten and O^T touched
        ok = mbar_wait(smem_u32(pv_done), (j - 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
        if (ok && any_rescale) {
          tc_fence_after();
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_O + lane_base, r);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < kHeads; ++h) r[h] = __float_as_uint(__uint_as_float(r[h]) * alpha[h]);
          tmem_st_32x32b_x16(tmem_O + lane_base, r);
          tmem_st_wait();
        }
      }
      ok = named_bar_and(2, 128, ok);               // also orders the reads of `red` before the next tile's writes
      if (!ok) break;
      // P^T[h][token] as a K-major operand: sub-tile of 64 tokens, row h of 128 bytes, 16-byte chunks swizzled by row
      {
        uint8_t* pcol = sP + (row >> 6) * (kHeads * 128) + (row & 7) * 2;
        const int chunk = (row & 63) >> 3;
#pragma unroll
        for (int h = 0; h < kHeads; ++h)
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
    float l_tot[kHeads];
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
      const float w = warp_sum(l_part[h]);
      if (lane == 0) red[ew * kHeads + h] = w;
    }
    named_bar_sync(1, 128);
#pragma unroll
    for (int h = 0; h < kHeads; ++h)
      l_tot[h] = (red[h] + red[kHeads + h]) + (red[2 * kHeads + h] + red[3 * kHeads + h]);
    const bool have = ok && n_tiles > 0;
    if (row < args.group) {
      float mh = -INFINITY, lh = 0.f;
#pragma unroll
      for (int h = 0; h < kHeads; ++h)
        if (h == row) { mh = m_used[h]; lh = l_tot[h]; }
      if (!have) { mh = -INFINITY; lh = 0.f; }
      float* ml = args.part_ml + ((static_cast<size_t>(b) * args.num_q_heads + head0 + row) * args.splits + split) * 2;
      ml[0] = mh;
      ml[1] = lh;
    }
    uint32_t r[16];
    if (have) {
      tc_fence_after();
      tmem_ld_32x32b_x16(tmem_O + lane_base, r);
      tmem_ld_wait();
    }
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
      if (h < args.group)      // a split without tokens writes zeros: the merge multiplies them by a zero weight
        args.part_acc[((static_cast<size_t>(b) * args.num_q_heads + head0 + h) * args.splits + split) * kHd + row] =
            have ? __uint_as_float(r[h]) : 0.f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace pdt
}  // namespace mfb

extern "C" {
using namespace mfb;

int mfb_paged_combine(const float* part_acc, const float* part_ml, void* out, int splits, int rows, int hd,
                      cudaStream_t stream);      // paged_attention.cu

// 1 when the tensor-core kernel serves these shapes (bf16 cache, head dim 128, at most 16 query heads per KV head,
// block size 16 / 32 / 64 / 128).
int mfb_paged_decode_tc_supported(int Hq, int Hkv, int hd, int block_size) {
  if (hd != 128 || Hkv < 1 || Hq % Hkv || Hq / Hkv > pdt::kHeads) return 0;
  return (block_size == 16 || block_size == 32 || block_size == 64 || block_size == 128) ? 1 : 0;
}

// Number of sequence splits that fills the GPU for B sequences of up to max_len tokens.
int mfb_paged_decode_tc_splits(int B, int Hkv, int max_len) {
  // cost of a choice = waves of CTAs over the 2 x 148 resident CTAs x (tiles per CTA + about one tile of fixed work)
  const int tiles = (max_len + pdt::kTile - 1) / pdt::kTile;
  int best = 1;
  long long best_cost = -1;
  for (int s = 1; s <= tiles && s <= 32; ++s) {
    const long long ctas = static_cast<long long>(B) * Hkv * s;
    const long long waves = (ctas + 295) / 296;
    const long long cost = waves * ((tiles + s - 1) / s + 1);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
  }
  return best;
}

// q [B, Hq, 128] bf16, caches [num_blocks, block_size, Hkv, 128] bf16, out [B, Hq, 128] bf16; scratch as for
// mfb_paged_decode_attention (mfb_paged_decode_scratch_bytes with the same splits).
int mfb_paged_decode_attention_tc(const void* q, const void* key_cache, const void* value_cache, const int* block_tables,
                                  const int* context_lens, void* out, void* scratch, int splits, int B, int Hq, int Hkv,
                                  int num_blocks, int block_size, int max_blocks, float scale, int* status,
                                  cudaStream_t stream) {
  if (!mfb_paged_decode_tc_supported(Hq, Hkv, 128, block_size) || splits < 1 || num_blocks < 1) {
    mfb_host::set_error("paged_decode_tc: unsupported Hq=%d Hkv=%d block_size=%d splits=%d", Hq, Hkv, block_size, splits);
    return 1;
  }
  if (B <= 0) return 0;
  CUtensorMap tQ, tK, tV;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t rows = (uint64_t)num_blocks * block_size, pitch = (uint64_t)Hkv * pdt::kHd;
  if ((rc = mfb_host::make_tmap_2d(&tQ, q, 2, BF, (uint64_t)B * Hq, pdt::kHd, pdt::kHd, pdt::kHeads, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tK, key_cache, 2, BF, rows, pitch, pitch, block_size, 64))) return 30 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tV, value_cache, 2, BF, rows, pitch, pitch, block_size, 64))) return 40 + rc;
  pdt::Args a;
  a.block_tables = block_tables; a.context_lens = context_lens; a.max_blocks = max_blocks; a.block_size = block_size;
  a.num_q_heads = Hq; a.num_kv_heads = Hkv; a.group = Hq / Hkv; a.splits = splits;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.part_acc = reinterpret_cast<float*>(scratch);
  a.part_ml = a.part_acc + static_cast<size_t>(B) * Hq * splits * pdt::kHd;
  a.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(pdt::paged_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pdt::kSmem) != cudaSuccess) {
      mfb_host::set_error("paged_decode_tc: cannot raise the shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  dim3 grid(splits, Hkv, B);
  pdt::paged_decode_tc_kernel<<<grid, pdt::kThreads, pdt::kSmem, stream>>>(tQ, tK, tV, a);
  if (cudaGetLastError() != cudaSuccess) { mfb_host::set_error("paged_decode_tc: launch failed"); return 11; }
  return mfb_paged_combine(a.part_acc, a.part_ml, out, splits, B * Hq, pdt::kHd, stream);
}

}  // extern "C"
