// Flash attention backward for sm_100a, head dim 128 (bf16, GQA, causal or full): pipelined, keys on the lanes.
//
// One CTA owns a tile of 128 keys of one KV head and loops over (query head of its share of the group, query
// tile that sees the key tile). The scores are computed TRANSPOSED, keys on the tensor-memory lanes:
//
//   S^T  = K Q^T                 dP^T = V dO^T                                   (tensor memory, 128 columns each)
//   P^T  = exp2(S^T scale - lse)            -> bf16 back into the S^T columns    (A operand of dV += P^T dO)
//   dS^T = P^T (dP^T - delta) scale         -> bf16 back into the dP^T columns   (A operand of dK += dS^T Q)
//                                           -> and as a [key][query] image in shared memory
//   dQ_part = dS K   (A = that image, MN-major)  -> the dP^T columns, drained by a warpgroup of its own into the
//                                                   fp32 dQ accumulator with TMA reduce-add
//
// so neither P nor dS^T crosses shared memory on its way to the dV / dK products, the per-query statistics (lse,
// delta) are per COLUMN and sit in a small shared-memory table, and Q is double-buffered. The MMA warp issues in the
// order  dV(i), S^T(i+1), dK(i), dQ(i), dP^T(i+1):  the tensor core runs the next tile's scores while this tile's
// dS is computed, and the drain of dQ(i) overlaps S^T / P of tile i+1. Products issued by one thread execute in
// order, which is what allows an MMA that overwrites columns (S^T(i+1) over P^T(i), dQ(i) over dS^T(i)) to be issued
// right behind the MMA that reads them.
//
// A KV head's query-head group can be split over `split` CTAs (more, shorter CTAs when there are few KV heads, as
// under tensor parallelism); dK / dV are then reduced in fp32 with TMA reduce-add and converted afterwards.
//
// Roles (448 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..5 and 6..9 the two compute
// warpgroups (query columns 0..63 / 64..127 of every key row), warps 10..13 dQ drain. Every wait is bounded.
#include "common.cuh"

namespace mfb {
namespace fb2 {

constexpr int kThreads = 448;
constexpr int kTile = 128;
constexpr int kHd = 128;
constexpr int kSubBytes = kTile * 128;
constexpr int kTileBytes = 2 * kSubBytes;
constexpr int kBarStats = 6, kBarDrain = 7, kBarEpi0 = 8;   // named barrier ids (0 is __syncthreads)

struct Args {
  int seq_q, seq_k;
  int q_off_tiles;
  int num_q_heads, num_kv_heads, group;
  int split;               // CTAs per (key tile, KV head): each takes group / split query heads
  int causal;
  float scale, scale_log2;
  const float* lse;        // [B, Hq, Sq]
  const float* delta;      // [B, Hq, Sq]
  const int* doc_start;    // [B, Sq] packed sequences: start of each token's document (null: one document per row)
  const int* doc_end;      // [B, Sq] one past the last position of each token's document
  int* status;
  int probe;               // timing probes (results are wrong): bit 0 the drain drops its staging and reduce-add,
                           // bit 1 the compute warpgroups drop the exponentials and the dS arithmetic
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
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
__device__ __forceinline__ float bf16lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// Warps are given registers in groups of four, so 448 threads are budgeted like 512: 128 registers per thread.
// The compute threads therefore work through their 64 queries in chunks of 32, and the drain in halves.
__global__ void __launch_bounds__(kThreads, 1)
flash_attn_bwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                       const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                       const __grid_constant__ CUtensorMap tmdQ, const __grid_constant__ CUtensorMap tmdK32,
                       const __grid_constant__ CUtensorMap tmdV32, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQ = sV + kTileBytes;            // 2 stages
  uint8_t* sdO = sQ + 2 * kTileBytes;
  uint8_t* sdS = sdO + kTileBytes;          // [key][query] image of dS
  uint8_t* sdQ = sdS + kTileBytes;          // 16 KB: one [128 rows][32 floats] image of a dQ quarter
  float* s_lse = reinterpret_cast<float*>(sdQ + kSubBytes);   // [2][128], log2 units
  float* s_dlt = s_lse + 2 * kTile;                           // [2][128]
  int* s_doc = reinterpret_cast<int*>(s_dlt + 2 * kTile);     // [2][128] document start of the query columns
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_doc + 2 * kTile);
  uint64_t* kv_full = bars;         // 1
  uint64_t* q_full = bars + 1;      // 2
  uint64_t* q_empty = bars + 3;     // 2
  uint64_t* do_full = bars + 5;
  uint64_t* do_empty = bars + 6;
  uint64_t* s_full = bars + 7;      // S^T complete
  uint64_t* p_ready = bars + 8;     // P^T written (256 arrivals)
  uint64_t* dp_full = bars + 9;     // dP^T complete
  uint64_t* ds_ready = bars + 10;   // dS^T (tensor memory) and dS (shared memory) written (256 arrivals)
  uint64_t* dq_full = bars + 11;    // dQ_part complete
  uint64_t* dq_free = bars + 12;    // dQ_part loaded out of tensor memory (128 arrivals)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one-dimensional grid, early key tiles (which every later query tile sees) first
  const int per_tile = args.num_kv_heads * args.split * (gridDim.x / ((args.seq_k / kTile) * args.num_kv_heads * args.split));
  const int kv_tile = static_cast<int>(blockIdx.x) / per_tile;
  int rest = static_cast<int>(blockIdx.x) % per_tile;
  const int part = rest % args.split;  rest /= args.split;
  const int kv_head = rest % args.num_kv_heads;
  const int batch = rest / args.num_kv_heads;
  const int heads_here = args.group / args.split;
  const int head0 = kv_head * args.group + part * heads_here;
  const int n_q_tiles = args.seq_q / kTile;
  int first_q = args.causal ? kv_tile - args.q_off_tiles : 0;
  int end_q = n_q_tiles;                      // one past the last query tile that sees this key tile
  if (args.doc_start) {
    // packed sequences (Sq == Sk, no offset): the queries that see a key are those of the key's document
    const size_t k0 = static_cast<size_t>(batch) * args.seq_q + kv_tile * kTile;
    if (!args.causal) first_q = args.doc_start[k0] / kTile;
    end_q = (args.doc_end[k0 + kTile - 1] - 1) / kTile + 1;
    if (end_q > n_q_tiles) end_q = n_q_tiles;
  }
  if (first_q < 0) first_q = 0;
  if (first_q > end_q) first_q = end_q;
  const int iters_per_head = end_q - first_q;
  const int n_iter = iters_per_head * heads_here;
  const int row_base = batch * args.seq_q;
  const int krow = batch * args.seq_k + kv_tile * kTile;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(kv_full), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&q_full[s]), 1);
      mbar_init(smem_u32(&q_empty[s]), 1);
    }
    mbar_init(smem_u32(do_full), 1);
    mbar_init(smem_u32(do_empty), 1);
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(p_ready), 256);
    mbar_init(smem_u32(dp_full), 1);
    mbar_init(smem_u32(ds_ready), 256);
    mbar_init(smem_u32(dq_full), 1);
    mbar_init(smem_u32(dq_free), 128);
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmdQ);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dV = tmem_base + 256, tmem_dK = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && n_iter > 0) {
      const uint32_t kvb = smem_u32(kv_full);
      mbar_expect_tx(kvb, 2 * kTileBytes);
      tma_load_2d(smem_u32(sK), &tmK, kvb, kv_head * kHd, krow);
      tma_load_2d(smem_u32(sK) + kSubBytes, &tmK, kvb, kv_head * kHd + 64, krow);
      tma_load_2d(smem_u32(sV), &tmV, kvb, kv_head * kHd, krow);
      tma_load_2d(smem_u32(sV) + kSubBytes, &tmV, kvb, kv_head * kHd + 64, krow);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int hq = head0 + it / iters_per_head;
        const int qrow = row_base + (first_q + it % iters_per_head) * kTile;
        const int st = it & 1;
        ok = mbar_wait(smem_u32(&q_empty[st]), ((it >> 1) & 1) ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) break;
        const uint32_t qb = smem_u32(&q_full[st]);
        mbar_expect_tx(qb, kTileBytes);
        tma_load_2d(smem_u32(sQ) + st * kTileBytes, &tmQ, qb, hq * kHd, qrow);
        tma_load_2d(smem_u32(sQ) + st * kTileBytes + kSubBytes, &tmQ, qb, hq * kHd + 64, qrow);
        ok = mbar_wait(smem_u32(do_empty), (it & 1) ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) break;
        const uint32_t db = smem_u32(do_full);
        mbar_expect_tx(db, kTileBytes);
        tma_load_2d(smem_u32(sdO), &tmdO, db, hq * kHd, qrow);
        tma_load_2d(smem_u32(sdO) + kSubBytes, &tmdO, db, hq * kHd + 64, qrow);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t IDESC_KK = umma_idesc_bf16(kTile, kTile, 0, 0);   // smem K-major x smem K-major
      constexpr uint32_t IDESC_TM = umma_idesc_bf16(kTile, kHd, 0, 1);     // tensor-memory A x smem MN-major
      constexpr uint32_t IDESC_MM = umma_idesc_bf16(kTile, kHd, 1, 1);     // smem MN-major x smem MN-major
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV), doa = smem_u32(sdO), dsa = smem_u32(sdS);
      auto issue_s = [&](int it) {        // S^T = K Q^T
        const uint32_t qa = smem_u32(sQ) + (it & 1) * kTileBytes;
#pragma unroll
        for (int k = 0; k < kHd / 16; ++k) {
          const uint32_t off = (k >> 2) * kSubBytes + (k & 3) * 32;
          umma_f16_ss(tmem_S, umma_desc_kmajor_sw128(ka + off), umma_desc_kmajor_sw128(qa + off), IDESC_KK,
                      k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(s_full));
      };
      auto issue_dp = [&]() {             // dP^T = V dO^T
#pragma unroll
        for (int k = 0; k < kHd / 16; ++k) {
          const uint32_t off = (k >> 2) * kSubBytes + (k & 3) * 32;
          umma_f16_ss(tmem_dP, umma_desc_kmajor_sw128(va + off), umma_desc_kmajor_sw128(doa + off), IDESC_KK,
                      k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(dp_full));
      };
      bool ok = mbar_wait(smem_u32(kv_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      if (ok) ok = mbar_wait(smem_u32(&q_full[0]), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        ok = mbar_wait(smem_u32(do_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      }
      if (ok) {
        tc_fence_after();
        issue_dp();
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        const uint32_t qa = smem_u32(sQ) + (it & 1) * kTileBytes;
        ok = mbar_wait(smem_u32(p_ready), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {   // dV += P^T dO, reduction over the 128 queries
          const uint32_t a_tmem = tmem_S + (k >> 2) * 64 + (k & 3) * 8;     // bf16 pairs of queries 16k .. 16k+15
          umma_f16_ts(tmem_dV, a_tmem, umma_desc_mnmajor_sw128(doa + k * 16 * 128, kSubBytes), IDESC_TM,
                      (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(do_empty));
        if (it + 1 < n_iter) {
          ok = mbar_wait(smem_u32(&q_full[(it + 1) & 1]), ((it + 1) >> 1) & 1, abort_flag, args.status,
                         kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          issue_s(it + 1);   // overwrites P^T(it): executes behind the dV product above
        }
        ok = mbar_wait(smem_u32(ds_ready), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {   // dK += dS^T Q
          const uint32_t a_tmem = tmem_dP + (k >> 2) * 64 + (k & 3) * 8;
          umma_f16_ts(tmem_dK, a_tmem, umma_desc_mnmajor_sw128(qa + k * 16 * 128, kSubBytes), IDESC_TM,
                      (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&q_empty[it & 1]));
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {   // dQ_part = dS K, reduction over the 128 keys; overwrites dS^T
          umma_f16_ss(tmem_dP, umma_desc_mnmajor_sw128(dsa + k * 16 * 128, kSubBytes),
                      umma_desc_mnmajor_sw128(ka + k * 16 * 128, kSubBytes), IDESC_MM, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(dq_full));
        if (it + 1 < n_iter) {
          ok = mbar_wait(smem_u32(do_full), (it + 1) & 1, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          ok = mbar_wait(smem_u32(dq_free), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          issue_dp();
        }
      }
    }
    __syncwarp();
  } else if (warp < 10) {
    // ------------------------------ compute warpgroups ------------------------------
    const int h = (warp - 2) >> 2;                    // query columns h*64 .. h*64+63
    const int ew = warp & 3;
    const int row = ew * 32 + lane;                   // key row of the tile
    const int tid = threadIdx.x - 64 - h * 128;       // 0..127 inside the warpgroup
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const uint32_t ph = it & 1;
      const int hq = head0 + it / iters_per_head;
      const int qi = first_q + it % iters_per_head;
      {
        const size_t idx = (static_cast<size_t>(batch) * args.num_q_heads + hq) * args.seq_q + qi * kTile + tid;
        if (h == 0) {
          s_lse[ph * kTile + tid] = args.lse[idx] * 1.4426950408889634f;
        } else {
          s_dlt[ph * kTile + tid] = args.delta[idx];
          if (args.doc_start)
            s_doc[ph * kTile + tid] = args.doc_start[static_cast<size_t>(batch) * args.seq_q + qi * kTile + tid];
        }
      }
      ok = named_bar_and(kBarStats, 256, ok);          // the table is complete; one decision for both warpgroups
      if (!ok) break;
      const bool diag = args.causal && (qi + args.q_off_tiles == kv_tile);
      // some query of the tile belongs to a document that starts after the first key of this key tile
      const int kpos = kv_tile * kTile + row;
      const bool doc_mask = args.doc_start && (s_doc[ph * kTile + kTile - 1] > kv_tile * kTile);
      uint32_t pk[32];                                 // P^T of this thread's 64 queries as bf16 pairs
      // ---- P^T ----
      if (ok) ok = mbar_wait(smem_u32(s_full), ph, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_S + lane_base + h * 64 + c * 32, r);
          tmem_ld_wait();
          const float4* l4 = reinterpret_cast<const float4*>(s_lse + ph * kTile + h * 64 + c * 32);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 l = l4[g];
            const int q0 = h * 64 + c * 32 + g * 4;
            float p0, p1, p2, p3;
            if (args.probe & 2) {
              p0 = __uint_as_float(r[g * 4 + 0]); p1 = __uint_as_float(r[g * 4 + 1]);
              p2 = __uint_as_float(r[g * 4 + 2]); p3 = __uint_as_float(r[g * 4 + 3]);
            } else {
              p0 = ex2f(fmaf(__uint_as_float(r[g * 4 + 0]), args.scale_log2, -l.x));
              p1 = ex2f(fmaf(__uint_as_float(r[g * 4 + 1]), args.scale_log2, -l.y));
              p2 = ex2f(fmaf(__uint_as_float(r[g * 4 + 2]), args.scale_log2, -l.z));
              p3 = ex2f(fmaf(__uint_as_float(r[g * 4 + 3]), args.scale_log2, -l.w));
            }
            if (diag) {                                // a query sees keys up to its own position
              if (q0 + 0 < row) p0 = 0.f;
              if (q0 + 1 < row) p1 = 0.f;
              if (q0 + 2 < row) p2 = 0.f;
              if (q0 + 3 < row) p3 = 0.f;
            }
            if (doc_mask) {                            // and none before the start of its document
              const int4 d = *reinterpret_cast<const int4*>(s_doc + ph * kTile + q0);
              if (d.x > kpos) p0 = 0.f;
              if (d.y > kpos) p1 = 0.f;
              if (d.z > kpos) p2 = 0.f;
              if (d.w > kpos) p3 = 0.f;
            }
            pk[c * 16 + g * 2] = pack_bf16x2(p0, p1);
            pk[c * 16 + g * 2 + 1] = pack_bf16x2(p2, p3);
          }
          // 32 queries = 16 packed columns, inside the 32 columns of chunk 0, which this thread has read already
          uint32_t (&pc)[16] = *reinterpret_cast<uint32_t(*)[16]>(&pk[c * 16]);
          tmem_st_32x32b_x16(tmem_S + lane_base + h * 64 + c * 16, pc);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(smem_u32(p_ready));
      }
      // ---- dS^T ----
      if (ok) ok = mbar_wait(smem_u32(dp_full), ph, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      // the dS image in shared memory was last read by the dQ product of the previous iteration
      if (ok && it > 0)
        ok = mbar_wait(smem_u32(dq_full), (it - 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      if (ok) {
        tc_fence_after();
        uint8_t* drow = sdS + h * kSubBytes + row * 128;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_dP + lane_base + h * 64 + c * 32, r);
          tmem_ld_wait();
          const float4* d4 = reinterpret_cast<const float4*>(s_dlt + ph * kTile + h * 64 + c * 32);
          uint32_t dsk[16];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 d = d4[g];
            const uint32_t pa = pk[c * 16 + g * 2], pb = pk[c * 16 + g * 2 + 1];
            const float s0 = bf16lo(pa) * (__uint_as_float(r[g * 4 + 0]) - d.x) * args.scale;
            const float s1 = bf16hi(pa) * (__uint_as_float(r[g * 4 + 1]) - d.y) * args.scale;
            const float s2 = bf16lo(pb) * (__uint_as_float(r[g * 4 + 2]) - d.z) * args.scale;
            const float s3 = bf16hi(pb) * (__uint_as_float(r[g * 4 + 3]) - d.w) * args.scale;
            dsk[g * 2] = pack_bf16x2(s0, s1);
            dsk[g * 2 + 1] = pack_bf16x2(s2, s3);
          }
          tmem_st_32x32b_x16(tmem_dP + lane_base + h * 64 + c * 16, dsk);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int chunk = c * 4 + j;               // 16-byte chunk (8 queries) of this row's 128-byte half
            *reinterpret_cast<uint4*>(drow + ((chunk ^ (row & 7)) << 4)) =
                make_uint4(dsk[4 * j], dsk[4 * j + 1], dsk[4 * j + 2], dsk[4 * j + 3]);
          }
        }
        fence_proxy_async_smem();
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(smem_u32(ds_ready));
      }
    }
    // ---- dK (warpgroup 0) and dV (warpgroup 1) of this key tile ----
    if (ok && n_iter > 0)
      ok = mbar_wait(smem_u32(dq_full), (n_iter - 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
    ok = named_bar_and(kBarEpi0 + h, 128, ok);
    if (ok) {
      tc_fence_after();
      const uint32_t src = (h == 0 ? tmem_dK : tmem_dV) + lane_base;
      uint8_t* stage = sQ + h * kTileBytes;             // every product that read Q has completed
      const bool issuer = (tid == 0);
      const CUtensorMap* tm16 = h == 0 ? &tmdK : &tmdV;
      const CUtensorMap* tm32 = h == 0 ? &tmdK32 : &tmdV32;
      if (args.split == 1) {
        uint8_t* orow = stage + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          if (n_iter > 0) {
            tmem_ld_32x32b_x32(src + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0;      // no query sees this key tile: zero gradients
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int chunk = c * 4 + q;
            *reinterpret_cast<uint4*>(orow + (chunk >> 3) * kSubBytes + (((chunk & 7) ^ (row & 7)) << 4)) =
                make_uint4(pack_bf16x2(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1])),
                           pack_bf16x2(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3])),
                           pack_bf16x2(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5])),
                           pack_bf16x2(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7])));
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(kBarEpi0 + h, 128);
        if (issuer) {
          tma_store_2d(tm16, smem_u32(stage), kv_head * kHd, krow);
          tma_store_2d(tm16, smem_u32(stage) + kSubBytes, kv_head * kHd + 64, krow);
          tma_commit_group();
          tma_wait_group<0>();
        }
      } else if (n_iter > 0) {
        // partial sums of a split group: fp32 reduce-add, 32 columns (one 16 KB image) at a time, two images in flight
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(src + c * 32, r);
          tmem_ld_wait();
          if (issuer) tma_wait_group_read<1>();
          named_bar_sync(kBarEpi0 + h, 128);
          uint8_t* irow = stage + (c & 1) * kSubBytes + row * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(irow + ((ch ^ (row & 7)) << 4)) =
                make_uint4(r[ch * 4], r[ch * 4 + 1], r[ch * 4 + 2], r[ch * 4 + 3]);
          fence_proxy_async_smem();
          named_bar_sync(kBarEpi0 + h, 128);
          if (issuer) {
            tma_reduce_add_2d(tm32, smem_u32(stage) + (c & 1) * kSubBytes, kv_head * kHd + c * 32, krow);
            tma_commit_group();
          }
        }
        if (issuer) tma_wait_group<0>();
      }
    }
  } else {
    // ------------------------------ dQ drain warpgroup ------------------------------
    const int ew = warp & 3;
    const int row = ew * 32 + lane;                   // query row of the tile
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    const bool issuer = (threadIdx.x == 320);
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int hq = head0 + it / iters_per_head;
      const int qrow = row_base + (first_q + it % iters_per_head) * kTile;
      if (ok) ok = mbar_wait(smem_u32(dq_full), it & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(kBarDrain, 128, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[64];
        {
          uint32_t (&ra)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[0]);
          uint32_t (&rb)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[32]);
          tmem_ld_32x32b_x32(tmem_dP + lane_base + half * 64, ra);
          tmem_ld_32x32b_x32(tmem_dP + lane_base + half * 64 + 32, rb);
          tmem_ld_wait();
        }
        if (half == 1) {
          tc_fence_before();
          mbar_arrive(smem_u32(dq_free));              // the columns can take dP^T of the next tile
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (args.probe & 1) continue;
          if (issuer) tma_wait_group_read<0>();         // the previous reduction has read the staging image
          named_bar_sync(kBarDrain, 128);
          uint8_t* irow = sdQ + row * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(irow + ((ch ^ (row & 7)) << 4)) =
                make_uint4(r[c * 32 + ch * 4], r[c * 32 + ch * 4 + 1], r[c * 32 + ch * 4 + 2], r[c * 32 + ch * 4 + 3]);
          fence_proxy_async_smem();
          named_bar_sync(kBarDrain, 128);
          if (issuer) {
            tma_reduce_add_2d(&tmdQ, smem_u32(sdQ), hq * kHd + half * 64 + c * 32, qrow);
            tma_commit_group();
          }
        }
      }
    }
    if (issuer) tma_wait_group<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// out (bf16, row pitch ld) = acc (fp32, contiguous [T, width])
__global__ void fb2_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, long long T,
                                   int width, long long ld) {
  const int wv = width / 4;
  const long long total = T * wv;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / wv;
    const int c = static_cast<int>(i - t * wv);
    const float4 v = reinterpret_cast<const float4*>(acc + t * width)[c];
    *reinterpret_cast<uint2*>(out + t * ld + c * 4) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (token, head)
__global__ void fb2_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                 float* __restrict__ delta, int B, int S, int H, long long do_ld, long long o_ld) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(B) * S * H) return;
  const int h = static_cast<int>(w % H);
  const long long tok = w / H;
  const uint2 a = *reinterpret_cast<const uint2*>(dO + tok * do_ld + h * kHd + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(O + tok * o_ld + h * kHd + lane * 4);
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float2 x = __bfloat1622float2(pa[i]), y = __bfloat1622float2(pb[i]);
    acc += x.x * y.x + x.y * y.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const int b_idx = static_cast<int>(tok / S), s = static_cast<int>(tok % S);
    delta[(static_cast<size_t>(b_idx) * H + h) * S + s] = acc;
  }
}

}  // namespace fb2
}  // namespace mfb

namespace {
int g_fb2_split = 0;   // 0 = choose from the problem size
int g_fb2_probe = 0;
}

extern "C" {
using namespace mfb;

// Split of a KV head's query-head group over CTAs: 0 lets the launcher choose, 1 / 2 / 4 force it.
void mfb_flash_attn_bwd2_set_split(int split) { g_fb2_split = split; }
// Timing probes for benchmarks (the results are wrong while one is set); see Args::probe.
void mfb_flash_attn_bwd2_set_probe(int bits) { g_fb2_probe = bits; }

static int fb2_choose_split(int B, int Sk, int Hq, int Hkv) {
  const int group = Hq / Hkv;
  if (g_fb2_split > 0 && group % g_fb2_split == 0) return g_fb2_split;
  // aim for at least about three CTAs per SM so that the longest CTA does not set the run time
  int split = 1;
  const long long ctas = static_cast<long long>(B) * (Sk / fb2::kTile) * Hkv;
  while (split * 2 <= group && group % (split * 2) == 0 && ctas * split < 3 * 148) split *= 2;
  return split;
}

// Scratch of mfb_flash_attn_bwd2: fp32 dQ accumulator, delta, and the fp32 dK / dV accumulators of a split group.
long long mfb_flash_attn_bwd2_scratch_bytes(int B, int Sq, int Sk, int Hq, int Hkv) {
  const long long dq = static_cast<long long>(B) * Sq * Hq * fb2::kHd * 4;
  const long long dl = static_cast<long long>(B) * Sq * Hq * 4;
  const long long dkv = 2ll * B * Sk * Hkv * fb2::kHd * 4;
  return dq + dl + dkv;
}

int mfb_flash_attn_bwd2_varlen(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                               const float* lse, const int* doc_start, const int* doc_end, void* dq, void* dk, void* dv,
                               void* scratch, int B, int S, int Sk, int Hq, int Hkv, long long q_ld, long long k_ld,
                               long long v_ld, long long o_ld, long long do_ld, long long dq_ld, long long dk_ld,
                               long long dv_ld, int causal, int q_offset, float scale, int* status, cudaStream_t stream);

// Arguments as mfb_flash_attn_bwd_ex; `scratch` holds mfb_flash_attn_bwd2_scratch_bytes(B, Sq, Sk, Hq, Hkv) bytes.
int mfb_flash_attn_bwd2(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                        void* dq, void* dk, void* dv, void* scratch, int B, int S, int Sk, int Hq, int Hkv,
                        long long q_ld, long long k_ld, long long v_ld, long long o_ld, long long do_ld,
                        long long dq_ld, long long dk_ld, long long dv_ld, int causal, int q_offset, float scale,
                        int* status, cudaStream_t stream) {
  return mfb_flash_attn_bwd2_varlen(q, k, v, o, d_o, lse, nullptr, nullptr, dq, dk, dv, scratch, B, S, Sk, Hq, Hkv, q_ld,
                                    k_ld, v_ld, o_ld, do_ld, dq_ld, dk_ld, dv_ld, causal, q_offset, scale, status, stream);
}

// The same with packed sequences: `doc_start` / `doc_end` [B, S] int32 (device) give for every token the first position
// of its document and one past its last. Needs S == Sk and q_offset == 0. Both null = one document per row.
int mfb_flash_attn_bwd2_varlen(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                               const float* lse, const int* doc_start, const int* doc_end, void* dq, void* dk, void* dv,
                               void* scratch, int B, int S, int Sk, int Hq, int Hkv, long long q_ld, long long k_ld,
                               long long v_ld, long long o_ld, long long do_ld, long long dq_ld, long long dk_ld,
                               long long dv_ld, int causal, int q_offset, float scale, int* status, cudaStream_t stream) {
  constexpr int T128 = fb2::kTile, HD = fb2::kHd;
  if ((doc_start != nullptr) != (doc_end != nullptr) || (doc_start && (S != Sk || q_offset != 0))) {
    mfb_host::set_error("flash_attn_bwd2: packed sequences need both document tables, Sq == Sk and no query offset");
    return 1;
  }
  if (S % T128 || Sk % T128 || Hq % Hkv || B <= 0 || q_offset % T128 || q_offset < 0 || (causal && q_offset + S > Sk)) {
    mfb_host::set_error("flash_attn_bwd2: unsupported shape B=%d Sq=%d Sk=%d Hq=%d Hkv=%d q_offset=%d", B, S, Sk, Hq, Hkv,
                        q_offset);
    return 1;
  }
  const long long T = static_cast<long long>(B) * S;
  const long long Tk = static_cast<long long>(B) * Sk;
  const int split = fb2_choose_split(B, Sk, Hq, Hkv);
  float* dq_accum = reinterpret_cast<float*>(scratch);
  float* delta = dq_accum + T * Hq * HD;
  float* dk_accum = delta + T * Hq;
  float* dv_accum = dk_accum + Tk * Hkv * HD;
  cudaMemsetAsync(dq_accum, 0, T * Hq * HD * sizeof(float), stream);
  if (split > 1) cudaMemsetAsync(dk_accum, 0, 2 * Tk * Hkv * HD * sizeof(float), stream);
  {
    const long long warps = T * Hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    fb2::fb2_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>((const __nv_bfloat16*)d_o, (const __nv_bfloat16*)o,
                                                                   delta, B, S, Hq, do_ld, o_ld);
  }
  CUtensorMap tQ, tK, tV, tdO, tdK, tdV, tdQ, tdK32, tdV32;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, F32 = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if ((rc = mfb_host::make_tmap_2d(&tdQ, dq_accum, 4, F32, T, (uint64_t)Hq * HD, (uint64_t)Hq * HD, T128, 32))) return 80 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdK32, dk_accum, 4, F32, Tk, (uint64_t)Hkv * HD, (uint64_t)Hkv * HD, T128, 32))) return 90 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdV32, dv_accum, 4, F32, Tk, (uint64_t)Hkv * HD, (uint64_t)Hkv * HD, T128, 32))) return 100 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tQ, q, 2, BF, T, (uint64_t)Hq * HD, q_ld, T128, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tK, k, 2, BF, Tk, (uint64_t)Hkv * HD, k_ld, T128, 64))) return 30 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tV, v, 2, BF, Tk, (uint64_t)Hkv * HD, v_ld, T128, 64))) return 40 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdO, d_o, 2, BF, T, (uint64_t)Hq * HD, do_ld, T128, 64))) return 50 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdK, dk, 2, BF, Tk, (uint64_t)Hkv * HD, dk_ld, T128, 64))) return 60 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdV, dv, 2, BF, Tk, (uint64_t)Hkv * HD, dv_ld, T128, 64))) return 70 + rc;
  fb2::Args a;
  a.seq_q = S; a.seq_k = Sk; a.q_off_tiles = q_offset / T128; a.num_q_heads = Hq; a.num_kv_heads = Hkv;
  a.group = Hq / Hkv; a.split = split; a.causal = causal;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f;
  a.lse = lse; a.delta = delta; a.status = status; a.doc_start = doc_start; a.doc_end = doc_end; a.probe = g_fb2_probe;
  constexpr int SMEM = 6 * fb2::kTileBytes + fb2::kSubBytes + 6 * T128 * 4 + 14 * 8 + 16 + 1024;
  static_assert(SMEM <= 232448, "shared memory budget exceeded");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(fb2::flash_attn_bwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("flash_attn_bwd2: cannot raise shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  const unsigned grid = static_cast<unsigned>((Sk / T128) * Hkv * split * B);
  fb2::flash_attn_bwd2_kernel<<<grid, fb2::kThreads, SMEM, stream>>>(tQ, tK, tV, tdO, tdK, tdV, tdQ, tdK32, tdV32, a);
  auto convert = [&](const float* acc, void* out, long long rows, int width, long long ld) {
    const long long total = rows * (width / 4);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fb2::fb2_convert_kernel<<<(unsigned)blocks, 256, 0, stream>>>(acc, (__nv_bfloat16*)out, rows, width, ld);
  };
  convert(dq_accum, dq, T, Hq * HD, dq_ld);
  if (split > 1) {
    convert(dk_accum, dk, Tk, Hkv * HD, dk_ld);
    convert(dv_accum, dv, Tk, Hkv * HD, dv_ld);
  }
  if (cudaGetLastError() != cudaSuccess) {
    mfb_host::set_error("flash_attn_bwd2: launch failed");
    return 11;
  }
  return 0;
}

}  // extern "C"
