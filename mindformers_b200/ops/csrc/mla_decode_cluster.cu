// Multi-latent attention decode, two-CTA cluster variant (sm_100a, tcgen05 + TMA + distributed shared memory).
//
// Same mathematics and interface as mla_decode.cu; see there for the transposed layout (tokens on the MMA rows, 16
// heads on the columns). The single-CTA kernel has to stream every cache tile twice because a 128-token tile
// (147 KB) leaves no room for its successor; its tensor core then waits for data half of the time. Here a CLUSTER OF
// TWO CTAs (two SMs) shares one (sequence, split, head chunk):
//
//   CTA 0 holds latent columns   0..255 and the 64 rope columns of a tile (80 KB), CTA 1 columns 256..511 (64 KB),
//   so each keeps TWO tiles resident (double buffer) and the cache is read from HBM exactly once;
//   each computes the part of S^T = C . Q^T that its columns contribute (a partial sum over K);
//   the softmax threads exchange the 128 x 16 partials through distributed shared memory (each thread writes its
//   row into the peer's exchange buffer with st.async, which counts the bytes on the peer's mbarrier), add them,
//   and both CTAs run the same softmax on the same numbers;
//   each accumulates O^T for its own 256 latent rows from the columns it already holds.
//
// Per tile and SM that is 36 (CTA 0) or 32 (CTA 1) narrow MMAs instead of 68 and one pass over the cache instead of
// two; the S^T products of tile j + 1 are issued before the O^T products of tile j when their data has arrived.
// Measured slower than the single-CTA kernel (two tile buffers cannot cover the load latency), so it is a selectable
// variant, not the default.
//
// No TMA load here is a cluster-wide broadcast: every CTA loads its own columns into its own shared memory.
// Cross-CTA traffic is the 64-byte st.async rows. Every wait is bounded; both CTAs of a
// cluster see the same tile count, and both always reach the cluster barriers at the start and the end.
#include "common.cuh"

namespace mfb {

constexpr int kMcThreads = 192;
constexpr int kMcTile = 128;               // tokens per tile
constexpr int kMcHeads = 16;               // heads per cluster
constexpr int kMcRank = 512;
constexpr int kMcDim = 576;
constexpr int kMcSub = kMcTile * 128;      // [128 tokens][64 columns] swizzled sub-tile, 16 KB
constexpr int kMcSubsMax = 5;              // CTA 0: 4 latent sub-tiles + rope; CTA 1: 4 latent sub-tiles
constexpr int kMcBuf = kMcSubsMax * kMcSub;          // one tile buffer, 80 KB
constexpr int kMcQSub = kMcHeads * 128;    // [16 heads][64 columns], 2 KB
constexpr int kMcPBytes = 2 * kMcHeads * 128;        // P^T: two [16 heads][64 tokens] K-major sub-tiles
constexpr int kMcXBytes = kMcTile * kMcHeads * 4;    // exchange buffer: 128 rows x 16 fp32, 8 KB
constexpr int kMcTmemCols = 128;
constexpr float kMcRescale = 8.0f;

struct McArgs {
  const int* block_tables;   // [B, max_blocks]
  const int* context_lens;   // [B]
  int max_blocks, block_size, num_heads, splits;
  float scale_log2;
  float* part_o;             // [B, splits, num_heads, 512] unnormalised
  float* part_ml;            // [B, splits, num_heads, 2]
  int* status;
};

__device__ __forceinline__ float mc_ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t mc_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mc_mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// 16-byte store into the peer CTA's shared memory that also counts 16 bytes on the peer's mbarrier: the receiver's
// wait completes when all expected bytes have landed, with no separate arrive from the 128 sending threads
__device__ __forceinline__ void mc_st_async_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                               uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(remote_bar) : "memory");
}
__device__ __forceinline__ uint32_t mc_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// bounded wait with cluster-scope acquire (the barrier is arrived on by the peer CTA)
__device__ __forceinline__ bool mc_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (mc_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!mc_try_wait_cluster(bar, parity)) {
    if (((++it) & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > MFB_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, kStatusWaitTimeoutEpilogue);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void mc_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kMcThreads, 1)
mla_decode_cluster_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmC,
                          const McArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sTile = smem;                               // 2 x 80 KB
  uint8_t* sP = sTile + 2 * kMcBuf;                    // 4 KB
  uint8_t* sQ = sP + kMcPBytes;                        // 10 KB (5 sub-tiles)
  uint8_t* sX = sQ + kMcSubsMax * kMcQSub;             // 2 x 8 KB: the peer's S^T partials
  float* red = reinterpret_cast<float*>(sX + 2 * kMcXBytes);       // [4 warps][16]
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + 4 * kMcHeads);
  uint64_t* q_full = bars;                  // 1
  uint64_t* full = bars + 1;                // 2 tile buffers
  uint64_t* empty = bars + 3;               // 2
  uint64_t* s_full = bars + 5;              // 2
  uint64_t* s_empty = bars + 7;             // 2
  uint64_t* x_full = bars + 9;              // 2: the peer's partial has landed in sX[buf]
  uint64_t* p_ready = bars + 11;            // 1
  uint64_t* pv_done = bars + 12;            // 1
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t crank = mc_cluster_ctarank();          // 0: columns 0..255 + rope, 1: columns 256..511
  const uint32_t peer = crank ^ 1u;
  const int split = blockIdx.x >> 1, chunk = blockIdx.y, b = blockIdx.z;
  const int len = args.context_lens[b];
  const int n_tiles_all = (len + kMcTile - 1) / kMcTile;
  const int per = (n_tiles_all + args.splits - 1) / args.splits;
  const int t0 = split * per;
  const int t1 = (t0 + per < n_tiles_all) ? t0 + per : n_tiles_all;
  const int n_tiles = t1 > t0 ? t1 - t0 : 0;
  const int head0 = chunk * kMcHeads;
  const int n_subs = crank == 0 ? 5 : 4;                 // sub-tiles of this CTA; sub 4 of CTA 0 is the rope block
  const int col_base = crank == 0 ? 0 : 256;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 128);
      mbar_init(smem_u32(&x_full[s]), 1);
    }
    mbar_init(smem_u32(p_ready), 128);
    mbar_init(smem_u32(pv_done), 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), kMcTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  mc_cluster_sync();                    // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_O = tmem_base;              // 2 blocks of 16 columns, 32 apart
  const uint32_t tmem_S = tmem_base + 64;         // 2 buffers of 16 columns, 32 apart

  if (warp == 0) {
    // ------------------------------------ producer ------------------------------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t qb = smem_u32(q_full);
      mbar_expect_tx(qb, n_subs * kMcQSub);
      for (int c = 0; c < n_subs; ++c) {
        const int col = (crank == 0 && c == 4) ? kMcRank : col_base + c * 64;
        tma_load_2d(smem_u32(sQ) + c * kMcQSub, &tmQ, qb, col, b * args.num_heads + head0);
      }
      const int bs = args.block_size;
      const int pages = kMcTile / bs;
      const int* table = args.block_tables + static_cast<size_t>(b) * args.max_blocks;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int buf = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(smem_u32(&empty[buf]), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) break;
        const int tok0 = (t0 + j) * kMcTile;
        int page_row[8];
        const int first_page = table[tok0 / bs];
        for (int i = 0; i < pages; ++i) {
          // pages past the end of the sequence may be unallocated: read the tile's first page instead (masked)
          const int pg = (tok0 + i * bs < len) ? table[tok0 / bs + i] : first_page;
          page_row[i] = pg * bs;
        }
        const uint32_t fb = smem_u32(&full[buf]);
        mbar_expect_tx(fb, n_subs * kMcSub);
        const uint32_t dst0 = smem_u32(sTile + buf * kMcBuf);
        for (int c = 0; c < n_subs; ++c) {
          const int col = (crank == 0 && c == 4) ? kMcRank : col_base + c * 64;
          for (int i = 0; i < pages; ++i)
            tma_load_2d(dst0 + c * kMcSub + i * bs * 128, &tmC, fb, col, page_row[i]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer ------------------------------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t IDESC_S = umma_idesc_bf16(kMcTile, kMcHeads, 0, 0);   // A = cache K-major, B = Q K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(kMcTile, kMcHeads, 1, 0);  // A = cache MN-major, B = P^T K-major
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      const uint32_t qa = smem_u32(sQ), pa = smem_u32(sP);
      // partial S^T of tile j over this CTA's columns, into S buffer j & 1
      auto issue_s = [&](int j) -> bool {
        const int buf = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&s_empty[buf]), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma)) return false;
        if (!mbar_wait(smem_u32(&full[buf]), ph, abort_flag, args.status, kStatusWaitTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t ca = smem_u32(sTile + buf * kMcBuf);
        for (int c = 0; c < n_subs; ++c) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t a_desc = umma_desc_kmajor_sw128(ca + c * kMcSub + k * 32);
            const uint64_t b_desc = umma_desc_kmajor_sw128(qa + c * kMcQSub + k * 32);
            umma_f16_ss(tmem_S + buf * 32, a_desc, b_desc, IDESC_S, (c > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&s_full[buf]));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // S^T of tile j + 1 goes first when its data is already here (it then runs while the softmax threads and the
        // exchange work on tile j); otherwise the O^T update of tile j must not wait for that load, whose buffer is
        // only freed by the O^T update of tile j - 1
        bool next_issued = j + 1 >= n_tiles;
        if (!next_issued && mbar_try_wait(smem_u32(&full[(j + 1) & 1]), ((j + 1) >> 1) & 1)) {
          ok = issue_s(j + 1);
          if (!ok) break;
          next_issued = true;
        }
        ok = mbar_wait(smem_u32(p_ready), j & 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const int buf = j & 1;
        const uint32_t ca = smem_u32(sTile + buf * kMcBuf);
        // O^T blocks of this CTA: latent rows [256 * crank + 128 * m, +128) = its sub-tiles 2m, 2m + 1
#pragma unroll
        for (int m = 0; m < 2; ++m) {
#pragma unroll
          for (int k = 0; k < kMcTile / 16; ++k) {
            const uint64_t a_desc = umma_desc_mnmajor_sw128(ca + 2 * m * kMcSub + k * 16 * 128, kMcSub);
            const uint64_t b_desc = umma_desc_kmajor_sw128(pa + (k >> 2) * (kMcHeads * 128) + (k & 3) * 32);
            umma_f16_ss(tmem_O + m * 32, a_desc, b_desc, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&empty[buf]));
        umma_commit(smem_u32(pv_done));
        if (!next_issued) ok = issue_s(j + 1);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------ softmax / exchange / epilogue ------------------------------------
    const int ew = warp & 3;
    const int row = ew * 32 + lane;                 // token row of S^T, latent row of O^T
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    float m_used[kMcHeads], l_part[kMcHeads];
#pragma unroll
    for (int h = 0; h < kMcHeads; ++h) { m_used[h] = -INFINITY; l_part[h] = 0.f; }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int buf = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ok = mbar_wait(smem_u32(&s_full[buf]), ph, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);             // the tensor-memory load below needs the whole warp
      uint32_t sr[16];
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32b_x16(tmem_S + buf * 32 + lane_base, sr);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(smem_u32(&s_empty[buf]));
      }
      // ---- exchange: my partial row goes into the peer's sX[buf]; the peer's lands in mine (8 KB per tile, counted
      // on x_full[buf]). The peer sends tile j only after it has finished tile j - 1, for which it needed this CTA's
      // rows of tile j - 1, and every thread here sends those only after it has read sX[buf] of tile j - 2 and (for
      // thread 0) seen that phase complete: the slot is free and the barrier is in its next phase. ----
      if (ok) {
        if (row == 0) mbar_expect_tx(smem_u32(&x_full[buf]), kMcXBytes);
        const uint32_t dst = mc_mapa(smem_u32(sX + buf * kMcXBytes + row * (kMcHeads * 4)), peer);
        const uint32_t rbar = mc_mapa(smem_u32(&x_full[buf]), peer);
#pragma unroll
        for (int q = 0; q < 4; ++q)
          mc_st_async_v4(dst + q * 16, sr[4 * q], sr[4 * q + 1], sr[4 * q + 2], sr[4 * q + 3], rbar);
        ok = mc_wait_cluster(smem_u32(&x_full[buf]), ph, abort_flag, args.status);
      }
      float s[kMcHeads];
      const bool valid = (t0 + j) * kMcTile + row < len;
      if (ok) {
        const float4* px = reinterpret_cast<const float4*>(sX + buf * kMcXBytes + row * (kMcHeads * 4));
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 o = px[q];
          s[4 * q] = __uint_as_float(sr[4 * q]) + o.x;
          s[4 * q + 1] = __uint_as_float(sr[4 * q + 1]) + o.y;
          s[4 * q + 2] = __uint_as_float(sr[4 * q + 2]) + o.z;
          s[4 * q + 3] = __uint_as_float(sr[4 * q + 3]) + o.w;
        }
      }
      ok = named_bar_and(2, 128, ok);
      if (!ok) break;
#pragma unroll
      for (int h = 0; h < kMcHeads; ++h) s[h] = valid ? s[h] * args.scale_log2 : -INFINITY;
      // per-head maximum over the 128 tokens of the tile
#pragma unroll
      for (int h = 0; h < kMcHeads; ++h) {
        const float w = warp_max(s[h]);
        if (lane == 0) red[ew * kMcHeads + h] = w;
      }
      named_bar_sync(1, 128);
      float alpha[kMcHeads];
      bool any_rescale = false;
#pragma unroll
      for (int h = 0; h < kMcHeads; ++h) {
        const float mx = fmaxf(fmaxf(red[h], red[kMcHeads + h]), fmaxf(red[2 * kMcHeads + h], red[3 * kMcHeads + h]));
        alpha[h] = 1.f;
        if (m_used[h] == -INFINITY) {
          m_used[h] = mx;
        } else if (mx > m_used[h] + kMcRescale) {
          alpha[h] = mc_ex2(m_used[h] - mx);
          m_used[h] = mx;
          any_rescale = true;
        }
      }
#pragma unroll
      for (int h = 0; h < kMcHeads; ++h) {
        const float neg_m = (m_used[h] == -INFINITY) ? 0.f : -m_used[h];
        s[h] = valid ? mc_ex2(s[h] + neg_m) : 0.f;
        l_part[h] = l_part[h] * alpha[h] + s[h];
      }
      if (j > 0) {
        // the previous O^T update has completed: P^T may be overwritten and O^T touched
        ok = mbar_wait(smem_u32(pv_done), (j - 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
        if (ok && any_rescale) {
          tc_fence_after();
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(tmem_O + lane_base + m * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < kMcHeads; ++h) r[h] = __float_as_uint(__uint_as_float(r[h]) * alpha[h]);
            tmem_st_32x32b_x16(tmem_O + lane_base + m * 32, r);
          }
          tmem_st_wait();
        }
      }
      ok = named_bar_and(2, 128, ok);               // also orders the reads of `red` before the next tile's writes
      if (!ok) break;
      {
        uint8_t* pcol = sP + (row >> 6) * (kMcHeads * 128) + (row & 7) * 2;
        const int chunk8 = (row & 63) >> 3;
#pragma unroll
        for (int h = 0; h < kMcHeads; ++h)
          *reinterpret_cast<__nv_bfloat16*>(pcol + h * 128 + ((chunk8 ^ (h & 7)) << 4)) = __float2bfloat16_rn(s[h]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(p_ready));
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(smem_u32(pv_done), (n_tiles - 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, 128, ok);
    }
    float l_tot[kMcHeads];
#pragma unroll
    for (int h = 0; h < kMcHeads; ++h) {
      const float w = warp_sum(l_part[h]);
      if (lane == 0) red[ew * kMcHeads + h] = w;
    }
    named_bar_sync(1, 128);
#pragma unroll
    for (int h = 0; h < kMcHeads; ++h)
      l_tot[h] = (red[h] + red[kMcHeads + h]) + (red[2 * kMcHeads + h] + red[3 * kMcHeads + h]);
    const size_t ps = static_cast<size_t>(b) * args.splits + split;
    if (crank == 0 && row < kMcHeads && head0 + row < args.num_heads) {
      float mh = -INFINITY, lh = 0.f;
#pragma unroll
      for (int h = 0; h < kMcHeads; ++h)
        if (h == row) { mh = m_used[h]; lh = l_tot[h]; }
      if (!ok || n_tiles == 0) { mh = -INFINITY; lh = 0.f; }
      float* ml = args.part_ml + (ps * args.num_heads + head0 + row) * 2;
      ml[0] = mh;
      ml[1] = lh;
    }
    if (ok && n_tiles > 0) {
      tc_fence_after();
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(tmem_O + lane_base + m * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < kMcHeads; ++h) {
          if (head0 + h < args.num_heads)
            args.part_o[(ps * args.num_heads + head0 + h) * kMcRank + crank * 256 + m * 128 + row] = __uint_as_float(r[h]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  mc_cluster_sync();                    // no CTA leaves while the peer may still arrive on its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kMcTmemCols);
  }
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// Splits for the cluster kernel: a cluster occupies two SMs, so 74 clusters are resident at once.
int mfb_mla_cluster_splits(int B, int num_heads, int max_len) {
  const int chunks = (num_heads + kMcHeads - 1) / kMcHeads;
  const int tiles = (max_len + kMcTile - 1) / kMcTile;
  int best = 1;
  long long best_cost = -1;
  for (int s = 1; s <= tiles && s <= 32; ++s) {
    const long long clusters = static_cast<long long>(B) * chunks * s;
    const long long waves = (clusters + 73) / 74;
    const long long cost = waves * ((tiles + s - 1) / s + 1);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
  }
  return best;
}

// Launch of the cluster kernel; arguments as mfb_mla_decode_attention (mla_decode.cu). The combine kernel of that
// file merges the splits afterwards. block_size must divide 128.
int mfb_mla_decode_cluster_launch(const void* q, const void* cache, const int* block_tables, const int* context_lens,
                                  float* part_o, float* part_ml, int splits, int B, int num_heads, int num_blocks,
                                  int block_size, int max_blocks, float scale, int* status, cudaStream_t stream) {
  CUtensorMap tQ, tC;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = mfb_host::make_tmap_2d(&tQ, q, 2, BF, (uint64_t)B * num_heads, kMcDim, kMcDim, kMcHeads, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tC, cache, 2, BF, (uint64_t)num_blocks * block_size, kMcDim, kMcDim, block_size, 64))) return 30 + rc;
  McArgs a;
  a.block_tables = block_tables; a.context_lens = context_lens; a.max_blocks = max_blocks; a.block_size = block_size;
  a.num_heads = num_heads; a.splits = splits; a.scale_log2 = scale * 1.4426950408889634f;
  a.part_o = part_o; a.part_ml = part_ml; a.status = status;
  constexpr int SMEM = 2 * kMcBuf + kMcPBytes + kMcSubsMax * kMcQSub + 2 * kMcXBytes + 4 * kMcHeads * 4 + 14 * 8 + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(mla_decode_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("mla_decode (cluster): cannot raise shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  const int chunks = (num_heads + kMcHeads - 1) / kMcHeads;
  dim3 grid(2 * splits, chunks, B);
  mla_decode_cluster_kernel<<<grid, kMcThreads, SMEM, stream>>>(tQ, tC, a);
  if (cudaGetLastError() != cudaSuccess) { mfb_host::set_error("mla_decode (cluster): launch failed"); return 11; }
  return 0;
}

}  // extern "C"
