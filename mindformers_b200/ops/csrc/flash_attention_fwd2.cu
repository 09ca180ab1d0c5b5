// Flash attention forward for sm_100a, head dim 128 (bf16, GQA, causal or full): two query tiles per CTA.
//
// One CTA owns 256 query rows of one head as two 128-row tiles, A and B, and walks over the key/value tiles once
// for both. Each tile has its own softmax warpgroup (128 threads, one query row each), so the tensor core works on
// one tile's products while the other tile's exponentials run:
//
//   MMA warp, per key tile j:   O_A += P_A(j) V_j ;  S_A = Q_A K_{j+1}^T ;  O_B += P_B(j) V_j ;  S_B = Q_B K_{j+1}^T
//   softmax warpgroup X:        S_X(j) (tensor memory) -> row max, exp2 -> P_X(j) as bf16 back into tensor memory
//
// P never touches shared memory: the softmax threads write it with tcgen05.st over the first 64 columns of the S
// buffer it came from, and the P V product reads it as the tensor-memory A operand. The tensor core executes the
// MMAs of one issuing thread in order, so S_X(j+1), which overwrites those columns, is issued right behind
// the P_X(j) V product that reads them. Tensor memory: S_A, S_B, O_A, O_B, 128 fp32 columns each (all 512).
// Shared memory: Q_A, Q_B, two stages of K, two stages of V (192 KB); the Q buffers stage the output at the end.
//
// The running maximum is lazy as in the single-tile kernel: O is rescaled only when a row maximum grows by more
// than 2^8. A fraction of the exponentials (template POLY, in quarters) is evaluated by a polynomial on the FMA pipe
// instead of the 16-per-clock MUFU unit (the loop is bound by instruction issue: scores are scaled, summed and
// converted two at a time with the packed fp32 instructions of sm_100, row maxima use the three-input maximum).
//
// Roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 softmax of tile A,
// warps 6..9 softmax of tile B. Every wait is bounded (common.cuh).
#include "common.cuh"

namespace mfb {
namespace fa2 {

constexpr int kThreads = 320;
constexpr int kTile = 128;
constexpr int kHd = 128;
constexpr int kSubBytes = kTile * 128;     // [128 rows][128 B] swizzled sub-tile (64 bf16 columns)
constexpr int kTileBytes = 2 * kSubBytes;  // 128 x 128 bf16
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct Args {
  int seq_q, seq_k;
  int q_off_tiles;         // causal: query row i sits at key position q_off_tiles * 128 + i
  int num_q_heads, group;
  int causal;
  float scale_log2;
  float* lse;              // [B, Hq, Sq] natural-log LSE (may be null)
  const int* doc_start;    // [B, Sq] packed sequences: position at which the document of each token starts
                           // (null: every sequence is one document). Needs Sq == Sk and no query offset.
  int* status;
};

__device__ __forceinline__ float ex2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed fp32 pairs (one instruction for two lanes of work) and the three-input maximum of sm_100: the softmax
// loop is bound by instruction issue, not by a single pipe, so halving the instruction count is what pays.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x for x <= 0 on the FMA pipe: x = n + f with f in [-0.5, 0.5], cubic for 2^f (max relative error 7.5e-5,
// below the bf16 rounding of P), n added to the exponent field.
__device__ __forceinline__ float ex2_fma(float x) {
  x = fmaxf(x, -125.f);
  const float xr = x + 12582912.f;
  const float f = x - (xr - 12582912.f);
  float p = fmaf(0.05517165f, f, 0.24261112f);
  p = fmaf(p, f, 0.69326099f);
  p = fmaf(p, f, 0.99992807f);
  return __uint_as_float(__float_as_uint(p) + (__float_as_uint(xr) << 23));
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16,"
      " %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// Warps are given registers in groups of four, so 320 threads are budgeted like 384: 168 registers per thread.
// The softmax therefore reads its S row from tensor memory twice (once for the maximum, once, in halves, for the
// exponentials) instead of holding all 128 scores across both passes.
template <int POLY>
__global__ void __launch_bounds__(kThreads, 1)
flash_attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                       const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                         // 2 tiles (A, B)
  uint8_t* sK = sQ + 2 * kTileBytes;          // 2 stages
  uint8_t* sV = sK + 2 * kTileBytes;          // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * kTileBytes);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2: S of tile A / B complete
  uint64_t* p_ready = bars + 11;    // 2: P of tile A / B written (128 arrivals)
  uint64_t* pv_done = bars + 13;    // 2: P V of tile A / B complete
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one-dimensional grid, heaviest work first over ALL heads and sequences: the late (long) query tiles of every
  // head are scheduled before any early (short) one, so the last wave is made of short CTAs
  const int n_q_tiles = args.seq_q / kTile;
  const int n_pairs = (n_q_tiles + 1) / 2;
  const int per_pair = gridDim.x / n_pairs;          // heads x sequences
  const int pair = n_pairs - 1 - static_cast<int>(blockIdx.x) / per_pair;
  const int hb = static_cast<int>(blockIdx.x) % per_pair;
  const int head = hb % args.num_q_heads, batch = hb / args.num_q_heads;
  const int kv_head = head / args.group;
  const int n_kv_all = args.seq_k / kTile;
  const int tile_of[2] = {2 * pair, 2 * pair + 1};
  int n_kv_x[2], lo_x[2];   // tile x works on key tiles lo_x[x] .. n_kv_x[x] - 1
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int diag = args.q_off_tiles + tile_of[x];
    int n = args.causal ? (diag + 1 < n_kv_all ? diag + 1 : n_kv_all) : n_kv_all;
    if (tile_of[x] >= n_q_tiles) n = 0;              // odd number of query tiles: the last CTA has tile A only
    n_kv_x[x] = n;
    lo_x[x] = 0;
    if (args.doc_start && n > 0) {
      // documents are contiguous, so no row of the tile starts earlier than its first row's document
      lo_x[x] = args.doc_start[static_cast<size_t>(batch) * args.seq_q + tile_of[x] * kTile] / kTile;
    }
  }
  const int n_kv = n_kv_x[0] > n_kv_x[1] ? n_kv_x[0] : n_kv_x[1];
  const int lo = (n_kv_x[1] > 0 && lo_x[1] < lo_x[0]) ? lo_x[1] : lo_x[0];   // first key tile this CTA loads
  const int k_row0 = batch * args.seq_k;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&p_ready[s]), 128);
      mbar_init(smem_u32(&pv_done[s]), 1);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // S_A +0, S_B +128, O_A +256, O_B +384; P_X lives in the first 64 columns of S_X
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      const uint32_t qb = smem_u32(q_full);
      const int n_tiles_here = (n_kv_x[1] > 0) ? 2 : 1;
      mbar_expect_tx(qb, n_tiles_here * kTileBytes);
      for (int x = 0; x < n_tiles_here; ++x) {
        const int q_row = batch * args.seq_q + tile_of[x] * kTile;
        tma_load_2d(smem_u32(sQ) + x * kTileBytes, &tmQ, qb, head * kHd, q_row);
        tma_load_2d(smem_u32(sQ) + x * kTileBytes + kSubBytes, &tmQ, qb, head * kHd + 64, q_row);
      }
      bool ok = true;
      for (int j = lo; j < n_kv && ok; ++j) {
        const int st = (j - lo) & 1;
        const uint32_t ph = ((j - lo) >> 1) & 1;
        ok = mbar_wait(smem_u32(&k_empty[st]), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) break;
        const uint32_t kb = smem_u32(&k_full[st]);
        mbar_expect_tx(kb, kTileBytes);
        const uint32_t kd = smem_u32(sK + st * kTileBytes);
        tma_load_2d(kd, &tmK, kb, kv_head * kHd, k_row0 + j * kTile);
        tma_load_2d(kd + kSubBytes, &tmK, kb, kv_head * kHd + 64, k_row0 + j * kTile);
        ok = mbar_wait(smem_u32(&v_empty[st]), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) break;
        const uint32_t vb = smem_u32(&v_full[st]);
        mbar_expect_tx(vb, kTileBytes);
        const uint32_t vd = smem_u32(sV + st * kTileBytes);
        tma_load_2d(vd, &tmV, vb, kv_head * kHd, k_row0 + j * kTile);
        tma_load_2d(vd + kSubBytes, &tmV, vb, kv_head * kHd + 64, k_row0 + j * kTile);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = umma_idesc_bf16(kTile, kTile, 0, 0);  // A = Q K-major (smem), B = K K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(kTile, kHd, 0, 1);    // A = P (tensor memory), B = V MN-major
      auto issue_qk = [&](int x, int j) {
        const uint32_t qa = smem_u32(sQ) + x * kTileBytes;
        const uint32_t ka = smem_u32(sK) + ((j - lo) & 1) * kTileBytes;
#pragma unroll
        for (int k = 0; k < kHd / 16; ++k) {
          const uint32_t off = (k >> 2) * kSubBytes + (k & 3) * 32;
          umma_f16_ss(tmem_base + x * kTile, umma_desc_kmajor_sw128(qa + off), umma_desc_kmajor_sw128(ka + off),
                      IDESC_QK, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_full[x]));
      };
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      auto active = [&](int x, int j) { return j >= lo_x[x] && j < n_kv_x[x]; };
      if (ok && n_kv > lo) {
        ok = mbar_wait(smem_u32(&k_full[0]), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (ok) {
          tc_fence_after();
          if (active(0, lo)) issue_qk(0, lo);
          if (active(1, lo)) issue_qk(1, lo);
          umma_commit(smem_u32(&k_empty[0]));
        }
      }
      for (int j = lo; j < n_kv && ok; ++j) {
        const int st = (j - lo) & 1;
        const uint32_t ph = ((j - lo) >> 1) & 1;
        ok = mbar_wait(smem_u32(&v_full[st]), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        bool k_next_waited = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const bool pv_now = active(x, j), qk_next = active(x, j + 1);
          if (pv_now) {
          ok = mbar_wait(smem_u32(&p_ready[x]), (j - lo_x[x]) & 1, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t va = smem_u32(sV) + st * kTileBytes;
          const uint32_t p_tmem = tmem_base + x * kTile;          // bf16 pairs: 8 columns per 16 keys
          const uint32_t o_tmem = tmem_base + 256 + x * kTile;
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k) {
            const uint64_t b_desc = umma_desc_mnmajor_sw128(va + k * 16 * 128, kSubBytes);
            umma_f16_ts(o_tmem, p_tmem + k * 8, b_desc, IDESC_PV, (j > lo_x[x] || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&pv_done[x]));
          }
          if (qk_next) {
            if (!k_next_waited) {
              ok = mbar_wait(smem_u32(&k_full[(j + 1 - lo) & 1]), ((j + 1 - lo) >> 1) & 1, abort_flag, args.status,
                             kStatusWaitTimeoutMma);
              if (!ok) break;
              tc_fence_after();
              k_next_waited = true;
            }
            issue_qk(x, j + 1);   // overwrites S_X / P_X: executes behind the P V product issued just above
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&v_empty[st]));
        if (k_next_waited) umma_commit(smem_u32(&k_empty[(j + 1 - lo) & 1]));
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ softmax warpgroups ------------------------------
    const int x = (warp - 2) >> 2;                 // 0 = tile A, 1 = tile B
    const int ew = warp & 3;                       // TMEM lane quarter of this warp
    const int row = ew * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    const uint32_t s_tmem = tmem_base + x * kTile + lane_base;
    const uint32_t o_tmem = tmem_base + 256 + x * kTile + lane_base;
    const uint32_t bar_and = 2 + x, bar_sync = 4 + x;
    const int my_n = n_kv_x[x], my_lo = lo_x[x];
    const int diag_tile = args.q_off_tiles + tile_of[x];
    // first key this row may see (its document's start); 0 without packed sequences
    const int my_doc = (args.doc_start && my_n > 0)
                           ? args.doc_start[static_cast<size_t>(batch) * args.seq_q + tile_of[x] * kTile + row] : 0;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    const uint64_t scale2 = pack2(args.scale_log2, args.scale_log2);
    for (int j = my_lo; j < my_n; ++j) {
      ok = mbar_wait(smem_u32(&s_full[x]), (j - my_lo) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      if (!ok) break;
      tc_fence_after();
      // columns [col_lo, col_hi] of this key tile are visible to the row; the tile is masked only where some row
      // of the warp needs it (the diagonal tile, and tiles that hold the start of a row's document)
      const int col_lo = my_doc - j * kTile;
      const int col_hi = (args.causal && j == diag_tile) ? row : kTile - 1;
      const bool on_diag = __any_sync(0xffffffffu, col_lo > 0 || col_hi < kTile - 1);
      // pass 1: row maximum (four independent chains of three-input maxima); the scores are not kept
      float mxs[4];
      {
        uint32_t sr[kTile];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t (&r)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sr[c * 32]);
          tmem_ld_32x32b_x32(s_tmem + c * 32, r);
        }
        tmem_ld_wait();
        float* s = reinterpret_cast<float*>(sr);
        if (on_diag) {
#pragma unroll
          for (int i = 0; i < kTile; ++i)
            if (i > col_hi || i < col_lo) s[i] = -INFINITY;
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          float m = s[a * 32];
#pragma unroll
          for (int i = 1; i + 1 < 32; i += 2) m = fmax3(m, s[a * 32 + i], s[a * 32 + i + 1]);
          mxs[a] = fmaxf(m, s[a * 32 + 31]);
        }
      }
      float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
      mx *= args.scale_log2;
      float alpha = 1.f;
      if (j == my_lo) {
        m_used = mx;
      } else if (mx > m_used + kRescaleThreshold) {
        alpha = ex2_mufu(m_used - mx);
        m_used = mx;
      }
      if (j > my_lo && __any_sync(0xffffffffu, alpha != 1.f)) {
        // S(j) is complete, so every earlier P V product has finished; the next one waits for p_ready below:
        // nobody else touches O now
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(o_tmem + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x16(o_tmem + c * 16, r);
        }
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      const uint64_t negm2 = pack2(neg_m, neg_m);
      uint64_t rs2[4] = {0, 0, 0, 0};
      // exp2 of the scaled, shifted scores two at a time; P goes back as bf16 pairs, 64 score columns (32 packed
      // registers) per store, into the first 64 columns of this tile's S buffer
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // pass 2: 64 scores at a time; the second half is read before the first half's P overwrites columns 0..31
        uint32_t sr[64];
        {
          uint32_t (&ra)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sr[0]);
          uint32_t (&rb)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sr[32]);
          tmem_ld_32x32b_x32(s_tmem + h * 64, ra);
          tmem_ld_32x32b_x32(s_tmem + h * 64 + 32, rb);
          tmem_ld_wait();
        }
        float* s = reinterpret_cast<float*>(sr);
        if (on_diag) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (h * 64 + i > col_hi || h * 64 + i < col_lo) s[i] = -INFINITY;
        }
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float t0, t1;
          unpack2(fma2(pack2(s[2 * i], s[2 * i + 1]), scale2, negm2), t0, t1);
          const bool poly = (i & 3) < POLY;
          const float e0 = poly ? ex2_fma(t0) : ex2_mufu(t0);
          const float e1 = poly ? ex2_fma(t1) : ex2_mufu(t1);
          rs2[i & 3] = add2(rs2[i & 3], pack2(e0, e1));
          pk[i] = pack_bf16x2(e0, e1);
        }
        if (h == 0) {
          // P of scores 0..63 goes to columns 0..31, which still hold scores 0..31 only: already consumed
          tmem_st_32x32b_x32(s_tmem, pk);
        } else {
          tmem_st_32x32b_x32(s_tmem + 32, pk);
        }
      }
      float r0, r1, r2, r3;
      unpack2(add2(rs2[0], rs2[1]), r0, r1);
      unpack2(add2(rs2[2], rs2[3]), r2, r3);
      l_sum = l_sum * alpha + ((r0 + r1) + (r2 + r3));
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&p_ready[x]));
    }
    if (my_n > 0) {
      if (ok) ok = mbar_wait(smem_u32(&pv_done[x]), (my_n - 1 - my_lo) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      // one decision for the whole warpgroup (a thread that gave up above still arrives here)
      ok = named_bar_and(bar_and, 128, ok);
      if (ok) {
        tc_fence_after();
        // every MMA that read Q_X has completed: its shared-memory tile now stages the output
        const float inv_l = 1.f / l_sum;
        uint8_t* stage = sQ + x * kTileBytes;
        uint8_t* orow = stage + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(o_tmem + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int chunk = c * 4 + q;
            uint4 v = make_uint4(
                pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * inv_l, __uint_as_float(r[q * 8 + 1]) * inv_l),
                pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * inv_l, __uint_as_float(r[q * 8 + 3]) * inv_l),
                pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * inv_l, __uint_as_float(r[q * 8 + 5]) * inv_l),
                pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * inv_l, __uint_as_float(r[q * 8 + 7]) * inv_l));
            *reinterpret_cast<uint4*>(orow + (chunk >> 3) * kSubBytes + (((chunk & 7) ^ (row & 7)) << 4)) = v;
          }
        }
        if (args.lse) {
          const size_t idx = (static_cast<size_t>(batch) * args.num_q_heads + head) * args.seq_q +
                             tile_of[x] * kTile + row;
          args.lse[idx] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
        }
        fence_proxy_async_smem();
        named_bar_sync(bar_sync, 128);
        if ((threadIdx.x & 127) == 64) {   // one thread of each warpgroup (threads 64 and 192)
          const int q_row = batch * args.seq_q + tile_of[x] * kTile;
          tma_store_2d(&tmO, smem_u32(stage), head * kHd, q_row);
          tma_store_2d(&tmO, smem_u32(stage) + kSubBytes, head * kHd + 64, q_row);
          tma_commit_group();
          tma_wait_group<0>();
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace fa2
}  // namespace mfb

namespace {
using namespace mfb;
int g_fa2_poly = 0;   // quarters of the exponentials evaluated on the FMA pipe

template <int POLY>
int fa2_launch_poly(const CUtensorMap& tQ, const CUtensorMap& tK, const CUtensorMap& tV, const CUtensorMap& tO,
                    const fa2::Args& a, dim3 grid, cudaStream_t stream) {
  constexpr int SMEM = 6 * fa2::kTileBytes + 16 * 8 + 16 + 1024;
  static_assert(SMEM <= 232448, "shared memory budget exceeded");
  auto kern = fa2::flash_attn_fwd2_kernel<POLY>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("flash_attn_fwd2: cannot raise shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  kern<<<grid, fa2::kThreads, SMEM, stream>>>(tQ, tK, tV, tO, a);
  if (cudaGetLastError() != cudaSuccess) {
    mfb_host::set_error("flash_attn_fwd2: launch failed");
    return 11;
  }
  return 0;
}
}  // namespace

extern "C" {

// Fraction (in quarters, 0..2) of the exponentials that the two-tile forward evaluates on the FMA pipe.
void mfb_flash_attn_fwd2_set_poly(int quarters) { g_fa2_poly = quarters < 0 ? 0 : (quarters > 2 ? 2 : quarters); }

int mfb_flash_attn_fwd2_varlen(const void* q, const void* k, const void* v, void* o, float* lse, const int* doc_start,
                               int B, int Sq, int Sk, int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld,
                               long long o_ld, int causal, int q_offset, float scale, int* status, cudaStream_t stream);

// Two-tile forward, head dim 128. Arguments as mfb_flash_attn_fwd_ex.
int mfb_flash_attn_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                        int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld, long long o_ld, int causal,
                        int q_offset, float scale, int* status, cudaStream_t stream) {
  return mfb_flash_attn_fwd2_varlen(q, k, v, o, lse, nullptr, B, Sq, Sk, Hq, Hkv, q_ld, k_ld, v_ld, o_ld, causal, q_offset,
                                    scale, status, stream);
}

// The same with packed sequences: `doc_start` [B, Sq] int32 (device) gives, for every token, the position inside its
// row at which its document starts; a token attends to the keys of its own document only (and, with `causal`, not to
// later ones). Needs Sq == Sk and q_offset == 0. Null `doc_start` = one document per row.
int mfb_flash_attn_fwd2_varlen(const void* q, const void* k, const void* v, void* o, float* lse, const int* doc_start,
                               int B, int Sq, int Sk, int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld,
                               long long o_ld, int causal, int q_offset, float scale, int* status, cudaStream_t stream) {
  using namespace mfb;
  constexpr int T = fa2::kTile, HD = fa2::kHd;
  if (doc_start && (Sq != Sk || q_offset != 0)) {
    mfb_host::set_error("flash_attn_fwd2: packed sequences need Sq == Sk and no query offset");
    return 1;
  }
  if (Sq % T || Sk % T || Hq % Hkv || B <= 0 || q_offset % T || q_offset < 0 || (causal && q_offset + Sq > Sk)) {
    mfb_host::set_error("flash_attn_fwd2: unsupported shape B=%d Sq=%d Sk=%d Hq=%d Hkv=%d causal=%d q_offset=%d", B,
                        Sq, Sk, Hq, Hkv, causal, q_offset);
    return 1;
  }
  CUtensorMap tQ, tK, tV, tO;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = mfb_host::make_tmap_2d(&tQ, q, 2, BF, (uint64_t)B * Sq, (uint64_t)Hq * HD, q_ld, T, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tK, k, 2, BF, (uint64_t)B * Sk, (uint64_t)Hkv * HD, k_ld, T, 64))) return 30 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tV, v, 2, BF, (uint64_t)B * Sk, (uint64_t)Hkv * HD, v_ld, T, 64))) return 40 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tO, o, 2, BF, (uint64_t)B * Sq, (uint64_t)Hq * HD, o_ld, T, 64))) return 50 + rc;
  fa2::Args a;
  a.seq_q = Sq; a.seq_k = Sk; a.q_off_tiles = q_offset / T; a.num_q_heads = Hq; a.group = Hq / Hkv;
  a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.lse = lse; a.status = status; a.doc_start = doc_start;
  dim3 grid(((Sq / T + 1) / 2) * Hq * B);
  switch (g_fa2_poly) {
    case 0: return fa2_launch_poly<0>(tQ, tK, tV, tO, a, grid, stream);
    case 1: return fa2_launch_poly<1>(tQ, tK, tV, tO, a, grid, stream);
    default: return fa2_launch_poly<2>(tQ, tK, tV, tO, a, grid, stream);
  }
}

}  // extern "C"
