// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
//   COMM = 1  all-gather -> GEMM   D[T, N] = gather_rows(A_r)[T, K] x B
//       Each rank contributes a chunk of T/tp rows of A that lives in peer-mapped ("symmetric")
//       memory. Four extra warps per CTA pull the remote chunks into a local [T, K] buffer with plain
//       peer loads (16-byte vectors), publishing a counter per 128-row block; the TMA producer of the
//       GEMM waits on that counter before it loads tiles of the block. Tiles of the rank's own rows
//       run first, so the NVLink transfer hides behind them. The gathered A is left complete in the
//       local buffer for the weight-gradient GEMM of the backward pass.
//   COMM = 2  GEMM -> reduce-scatter   D_r[T/tp, N] = sum_p (A_p x B_p)[rows of rank r]
//       Every rank computes all T rows of its partial product, remote-owned row chunks first. The
//       epilogue of a remote-owned tile stores the bf16 tile straight into the owner's receive buffer
//       (peer stores) and releases a per-tile flag; the epilogue of an own tile acquires the flags of
//       all peers, adds their tiles to the accumulator in fp32 and writes the final rows. No separate
//       reduction pass and no host synchronisation.
//
//   COMM = 3  GEMM -> all-reduce (one shot)   D[M, N] = sum_p (A_p x B_p), the same bits on every rank
//       For tensor-parallel inference, where M is a decode batch or a prefill chunk and no rank owns a row
//       range. The epilogue of every tile rounds the partial tile to bf16, stores it into the receive slot
//       [rank] of every peer (coalesced peer stores) and releases the tile's flag there; then it acquires the
//       flags of all peers for the same tile, adds the tp bf16 partials in rank order (its own rounded one
//       included, so that all ranks produce identical bits) and writes the tile with a TMA store. All ranks
//       walk the tiles in the same order, so the wait is for a store that the peer issues before it waits
//       itself. M needs no alignment: TMA zero-fills rows past M on load and clips them on store.
//
// Cross-rank flags carry a monotonically increasing epoch (the call counter, identical on all ranks),
// so they never need a reset; receive buffers are double-buffered on the epoch parity. A rank can be at
// most one call ahead of a peer, because each call waits for data that the peer only produces in the
// same call. Every wait is bounded and reports through the status word.
//
// PAIR = true runs COMM 1 / 2 on CTA pairs (`cta_group::2`, 256 x 256 MMA tiles, see gemm_tcgen05_2cta.cu):
// the two CTAs of a cluster take the row blocks 2i and 2i+1 of one tile column, each loads its own A block
// and its own half of the B tile, the even CTA issues the MMA for both. Everything that crosses ranks
// (copy warps, block counters, tile flags, receive slots) stays per 128-row block, i.e. per CTA.
//
// No TMA load in this file uses cluster multicast, and no TMA load reads peer memory.
#include "common.cuh"

namespace mfb {

constexpr int kTpBM = 128;
constexpr int kTpBK = 64;
constexpr int kTpStaging = 128 * 128;
constexpr int kTpMaxRanks = 8;
constexpr int kCopySlices = 8;  // a 128-row block is copied as 8 slices of 16 rows

struct TpArgs {
  int M, N, K;          // D is [M, N] for COMM 1; the partial product is [M, N] for COMM 2
  int num_m_blocks, num_n_blocks;
  int tp, rank, epoch;
  int rows_per_chunk;   // M / tp, multiple of 128
  int ksplit;           // COMM 3: CTAs that share the K range of one tile (1 = no split); otherwise 1
  int probe;            // timing probes (results are wrong): bit 0 drops the peer stores and their fence, bit 1 the
                        // owner's wait for and reads of the peers' partial tiles
  int rs_lag;           // COMM 2: > 0 interleaves own and remote tiles after this many remote tiles (see rs_order)
  int band;             // raster band of the CTA-pair walk, in pairs of row blocks
  int* status;
  // ---- COMM 1 ----
  const __nv_bfloat16* peer_a[kTpMaxRanks];  // chunk [rows_per_chunk, K] of every rank (row pitch lda)
  long long lda;
  __nv_bfloat16* a_full;                     // local [M, K], contiguous
  int* block_flags;                          // [num_m_blocks] local counters, zero before launch
  int* ready_local;                          // [tp]: entry p is written by rank p
  int* ready_peer[kTpMaxRanks];              // the same array on every rank
  // ---- COMM 2 ----
  __nv_bfloat16* recv_local;                 // [2][tp][rows_per_chunk, N] receive slots of this rank
  __nv_bfloat16* recv_peer[kTpMaxRanks];
  int* tile_flags_local;                     // [2][tp][blocks_per_chunk * num_n_blocks]
  int* tile_flags_peer[kTpMaxRanks];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Bounded spin until *flag >= want (system or gpu scope acquire).
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int want, volatile int* abort_flag, int* status) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    const int v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if (v >= want) return true;
    if (((++it) & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > MFB_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, kStatusPeerFlagTimeout);
        return false;
      }
    }
    __nanosleep(64);
  }
}

struct TpTile {
  int m_blk, n_blk;
};

// Banded rasterisation with the row blocks rotated so that the chunk order starts at `first_chunk`.
__device__ __forceinline__ TpTile tp_tile(const TpArgs& a, int tile, int first_chunk) {
  constexpr int kBand = 16;
  const int tiles_per_band = kBand * a.num_n_blocks;
  const int band = tile / tiles_per_band;
  const int first_m = band * kBand;
  const int band_h = (a.num_m_blocks - first_m) < kBand ? (a.num_m_blocks - first_m) : kBand;
  const int r = tile - band * tiles_per_band;
  int m = first_m + r % band_h;
  const int bpc = a.rows_per_chunk / kTpBM;
  m = (m + first_chunk * bpc) % a.num_m_blocks;
  TpTile t;
  t.m_blk = m;
  t.n_blk = r / band_h;
  return t;
}

// The same walk over pairs of row blocks: tile -> (pair of row blocks, column block); CTA `cta` of the cluster
// takes row block 2 * pair + cta. Chunks hold an even number of row blocks, so a pair never straddles two ranks.
__device__ __forceinline__ TpTile tp_tile_pair(const TpArgs& a, int tile, int first_chunk, int cta) {
  const int kBand = a.band;     // pairs of row blocks per raster band: 16 for K <= 4096, else 8 (see gemm_tcgen05_2cta.cu)
  const int num_pairs = a.num_m_blocks >> 1;
  const int tiles_per_band = kBand * a.num_n_blocks;
  const int band = tile / tiles_per_band;
  const int first_m = band * kBand;
  const int band_h = (num_pairs - first_m) < kBand ? (num_pairs - first_m) : kBand;
  const int r = tile - band * tiles_per_band;
  int m = first_m + r % band_h;
  const int ppc = (a.rows_per_chunk / kTpBM) >> 1;
  m = (m + first_chunk * ppc) % num_pairs;
  TpTile t;
  t.m_blk = 2 * m + cta;
  t.n_blk = r / band_h;
  return t;
}

// Work order of the GEMM -> reduce-scatter kernel. In chunk order the tiles of the other ranks' rows (whose
// epilogues store over NVLink) come first and the rank's own tiles last, which packs all link traffic into the first
// (tp-1)/tp of the run; with a short reduction dimension that phase is bound by the link, not by the tensor core.
// This order starts with `lag` remote tiles (so that every partial tile is on its way well before its owner needs
// it) and then takes one own tile after every tp-1 remote ones, spreading the stores over the whole run. All ranks
// use the same order, so the rank that produces a partial tile stays `lag` positions ahead of its consumer.
__device__ __forceinline__ int rs_order(int i, int n_tiles, int tp, int lag) {
  const int n_o = n_tiles / tp, n_r = n_tiles - n_o;
  const int L = lag < n_r ? lag : n_r;
  if (i < L) return i;
  const int j = i - L;
  const int rm1 = tp - 1;
  int n_cyc = (n_r - L) / rm1;
  if (n_cyc > n_o) n_cyc = n_o;
  const int cyc = j / tp, pos = j - cyc * tp;
  if (cyc < n_cyc) return pos == 0 ? n_r + cyc : L + cyc * rm1 + (pos - 1);
  const int k = j - n_cyc * tp;
  const int rem_left = (n_r - L) - n_cyc * rm1;
  return k < rem_left ? L + n_cyc * rm1 + k : n_r + n_cyc + (k - rem_left);
}

template <int BN, int STAGES, bool B_MN, int COMM, bool PAIR>
__global__ void __launch_bounds__(COMM == 1 ? 320 : 192, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA,      // COMM 1: own chunk; COMM 2: A [M, K]
               const __grid_constant__ CUtensorMap tmAfull,  // COMM 1: gathered A [M, K]
               const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmD,      // COMM 1: D [M, N]; COMM 2: D_r [M/tp, N]
               const TpArgs args) {
  static_assert(!PAIR || (COMM != 3 && BN == 256), "CTA pairs serve the 256-wide training tiles only");
  constexpr int A_BYTES = kTpBM * kTpBK * 2;
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;   // rows of B this CTA stages (a pair splits the tile's N)
  constexpr int B_BYTES = B_ROWS * kTpBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;
  constexpr int NUM_CHUNKS = BN / 64;
  constexpr uint32_t IDESC = umma_idesc_bf16(PAIR ? 2 * kTpBM : kTpBM, BN, 0, B_MN ? 1 : 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * kTpStaging);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bpc = args.rows_per_chunk / kTpBM;  // row blocks per chunk
  const int k_blocks = (args.K + kTpBK - 1) / kTpBK;
  const int cta = PAIR ? static_cast<int>(cluster_ctarank()) : 0;
  const int wid = PAIR ? (blockIdx.x >> 1) : blockIdx.x;        // work-item walker: one per CTA or per pair
  const int wstride = PAIR ? (gridDim.x >> 1) : gridDim.x;
  const int n_tiles = (PAIR ? (args.num_m_blocks >> 1) : args.num_m_blocks) * args.num_n_blocks;
  const int ksplit = (COMM == 3 && args.ksplit > 1) ? args.ksplit : 1;
  const int k_per_split = (k_blocks + ksplit - 1) / ksplit;
  const int n_items = n_tiles * ksplit;
  // COMM 1 starts with the rank's own rows, COMM 2 with the rows of the next rank (own rows last)
  const int first_chunk = (COMM == 1) ? args.rank : (COMM == 2 ? (args.rank + 1) % args.tp : 0);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tfull_bar[s]), 1);
      mbar_init(smem_u32(&tempty_bar[s]), PAIR ? 8 : 4);   // the epilogue warps of both CTAs of a pair
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
    if (COMM == 1) {
      tma_prefetch_desc(&tmAfull);
      if (blockIdx.x == 0) {
        // this rank's chunk was written by earlier work on the stream: tell every peer it may read it
        for (int p = 0; p < args.tp; ++p)
          if (p != args.rank) st_release_sys(args.ready_peer[p] + args.rank, args.epoch);
      }
    }
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_holder), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer CTA's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = wid; item < n_items && ok; item += wstride) {
        const int tile = (COMM == 2 && args.rs_lag > 0) ? rs_order(item, n_tiles, args.tp, args.rs_lag) : item / ksplit;
        const int kb0 = (item - (item / ksplit) * ksplit) * k_per_split;
        const int kb1 = (kb0 + k_per_split < k_blocks) ? kb0 + k_per_split : k_blocks;
        const TpTile t = PAIR ? tp_tile_pair(args, tile, first_chunk, cta) : tp_tile(args, tile, first_chunk);
        const int chunk = t.m_blk / bpc;
        const bool own = (COMM == 1) && (chunk == args.rank);
        if (COMM == 1 && !own) {
          ok = wait_flag_ge<false>(args.block_flags + t.m_blk, kCopySlices, abort_flag, args.status);
          if (!ok) break;
          // the copy was made with generic-proxy stores; order it before the async-proxy (TMA) reads
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, args.status,
                         kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb_local = smem_u32(&full_bar[stage]);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_BYTES;
          if (PAIR) {
            // both CTAs' loads count on the even CTA's barrier, which expects the bytes of both
            const uint32_t fb = mapa_shared(fb_local, 0);
            if (cta == 0) mbar_expect_tx(fb_local, 2 * STAGE_BYTES);
            const int b_n0 = t.n_blk * BN + cta * B_ROWS;
            if (own) tma_load_2d_pair(a_dst, &tmA, fb, kb * kTpBK, (t.m_blk - args.rank * bpc) * kTpBM);
            else if (COMM == 1) tma_load_2d_pair(a_dst, &tmAfull, fb, kb * kTpBK, t.m_blk * kTpBM);
            else tma_load_2d_pair(a_dst, &tmA, fb, kb * kTpBK, t.m_blk * kTpBM);
            if (B_MN) {
#pragma unroll
              for (int at = 0; at < B_ROWS / 64; ++at)
                tma_load_2d_pair(b_dst + at * (kTpBK * 128), &tmB, fb, b_n0 + at * 64, kb * kTpBK);
            } else {
              tma_load_2d_pair(b_dst, &tmB, fb, kb * kTpBK, b_n0);
            }
          } else {
            const uint32_t fb = fb_local;
            mbar_expect_tx(fb, STAGE_BYTES);
            if (own) tma_load_2d(a_dst, &tmA, fb, kb * kTpBK, (t.m_blk - args.rank * bpc) * kTpBM);
            else if (COMM == 1) tma_load_2d(a_dst, &tmAfull, fb, kb * kTpBK, t.m_blk * kTpBM);
            else tma_load_2d(a_dst, &tmA, fb, kb * kTpBK, t.m_blk * kTpBM);
            if (B_MN) {
#pragma unroll
              for (int at = 0; at < BN / 64; ++at)
                tma_load_2d(b_dst + at * (kTpBK * 128), &tmB, fb, t.n_blk * BN + at * 64, kb * kTpBK);
            } else {
              tma_load_2d(b_dst, &tmB, fb, kb * kTpBK, t.n_blk * BN);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && cta == 0) {   // in a pair the even CTA issues the MMAs of both
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int item = wid; item < n_items && ok; item += wstride) {
        const int kb0 = (item % ksplit) * k_per_split;
        const int kb1 = (kb0 + k_per_split < k_blocks) ? kb0 + k_per_split : k_blocks;
        ok = mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
          for (int k = 0; k < kTpBK / 16; ++k) {
            const uint64_t a_desc = umma_desc_kmajor_sw128(a_base + k * 32);
            const uint64_t b_desc = B_MN ? umma_desc_mnmajor_sw128(b_base + k * 16 * 128, kTpBK * 128)
                                         : umma_desc_kmajor_sw128(b_base + k * 32);
            if (PAIR) umma_f16_ss_pair(d_tmem, a_desc, b_desc, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
            else umma_f16_ss(d_tmem, a_desc, b_desc, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          if (PAIR) umma_commit_pair(smem_u32(&empty_bar[stage]));
          else umma_commit(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) umma_commit_pair(smem_u32(&tfull_bar[acc]));
        else umma_commit(smem_u32(&tfull_bar[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    const int ew = warp & 3;
    const int row = ew * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    int acc = 0;
    uint32_t acc_phase = 0, chunk_counter = 0;
    bool ok = true;
    const int parity = args.epoch & 1;
    const size_t slot_elems = static_cast<size_t>(args.rows_per_chunk) * args.N;
    const int tiles_per_chunk = bpc * args.num_n_blocks;
    // accumulator-drained arrivals go to the even CTA of a pair (its own barrier otherwise)
    const uint32_t tempty0 = PAIR ? mapa_shared(smem_u32(&tempty_bar[0]), 0) : smem_u32(&tempty_bar[0]);
    const uint32_t tempty1 = PAIR ? mapa_shared(smem_u32(&tempty_bar[1]), 0) : smem_u32(&tempty_bar[1]);
    for (int item = wid; item < n_items && ok; item += wstride) {
      const int tile = (COMM == 2 && args.rs_lag > 0) ? rs_order(item, n_tiles, args.tp, args.rs_lag) : item / ksplit;
      const int ks = item - (item / ksplit) * ksplit;
      const TpTile t = PAIR ? tp_tile_pair(args, tile, first_chunk, cta) : tp_tile(args, tile, first_chunk);
      const int owner = t.m_blk / bpc;
      const int mb_local = t.m_blk - owner * bpc;
      const int tile_in_chunk = mb_local * args.num_n_blocks + t.n_blk;
      ok = mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      if (COMM == 2 && ok && owner == args.rank && !(args.probe & 2)) {
        // the peers' partial tiles must have landed in this rank's receive slots
        if (issuer) {
          for (int p = 0; p < args.tp && ok; ++p) {
            if (p == args.rank) continue;
            const int* f = args.tile_flags_local + (static_cast<size_t>(parity) * args.tp + p) * tiles_per_chunk + tile_in_chunk;
            ok = wait_flag_ge<true>(f, args.epoch, abort_flag, args.status);
          }
        }
      }
      ok = named_bar_and(2, 128, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * BN;
      const int local_row = mb_local * kTpBM + row;   // row inside the owner's chunk
      if (COMM == 3) {
        // slot (rank, K-split) of every partial; the sum runs over slots in index order on every rank
        const int n_slots = args.tp * ksplit;
        const int my_slot = args.rank * ksplit + ks;
        // ---- push the bf16 partial tile to every peer (a K-split helper also to its own rank) ----
        const int et = threadIdx.x - 64;   // 0..127
        const int cj = et & 7;             // 16-byte chunk inside a 128-byte staging row
        if (issuer) tma_wait_group_read<0>();   // the stores of the previous tile have read the staging buffers
#pragma unroll 1
        for (int c = 0; c < NUM_CHUNKS; ++c) {
          uint32_t v0[32], v1[32], packed[32];
          tmem_ld_32x32b_x32(t_addr + c * 64, v0);
          tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            packed[i] = pack_bf16x2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1]));
            packed[16 + i] = pack_bf16x2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1]));
          }
          const int col0 = t.n_blk * BN + c * 64;
          const int buf = chunk_counter & 1;
          named_bar_sync(1, 128);
          uint8_t* sbase = staging + buf * kTpStaging;
          uint8_t* srow = sbase + row * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          named_bar_sync(1, 128);
          if (col0 < args.N) {
            uint4 vals[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 16 + (et >> 3);
              vals[i] = *reinterpret_cast<const uint4*>(sbase + r * 128 + ((cj ^ (r & 7)) << 4));
            }
            for (int p = 0; p < args.tp; ++p) {
              if (p == args.rank && ks == 0) continue;     // the reducing CTA keeps its own partial in registers
              __nv_bfloat16* dst0 = args.recv_peer[p] + (static_cast<size_t>(parity) * n_slots + my_slot) * slot_elems +
                                    static_cast<size_t>(t.m_blk * kTpBM) * args.N + col0 + cj * 8;
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int r = i * 16 + (et >> 3);
                *reinterpret_cast<uint4*>(dst0 + static_cast<size_t>(r) * args.N) = vals[i];
              }
            }
          }
          ++chunk_counter;
        }
        __threadfence_system();
        named_bar_sync(1, 128);
        if (issuer) {
          for (int p = 0; p < args.tp; ++p) {
            if (p == args.rank && ks == 0) continue;
            st_release_sys(args.tile_flags_peer[p] + (static_cast<size_t>(parity) * n_slots + my_slot) * tiles_per_chunk + tile_in_chunk,
                           args.epoch);
          }
        }
        if (ks != 0) {
          // a K-split helper is done once its partial is published; the CTA with ks == 0 reduces the tile
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          continue;
        }
        if (warp == 2) {
          // ---- the other partial tiles: every rank's K-splits; the lanes of one warp poll the flags side by side ----
          bool okl = ok;
          for (int sl = lane; sl < n_slots && okl; sl += 32) {
            if (sl == my_slot) continue;
            okl = wait_flag_ge<true>(args.tile_flags_local + (static_cast<size_t>(parity) * n_slots + sl) * tiles_per_chunk + tile_in_chunk,
                                     args.epoch, abort_flag, args.status);
          }
          ok = __all_sync(0xffffffffu, okl);
        }
        ok = named_bar_and(2, 128, ok);
        if (!ok) break;
        // ---- sum in slot order and store ----
#pragma unroll 1
        for (int c = 0; c < NUM_CHUNKS; ++c) {
          uint32_t packed[32];
          const int col0 = t.n_blk * BN + c * 64;
          const bool in_range = col0 < args.N;
#pragma unroll 1
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t v[32];
            float sum[32];
            tmem_ld_32x32b_x32(t_addr + c * 64 + hf * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) sum[i] = 0.f;
            const __nv_bfloat16* src0 = args.recv_local + static_cast<size_t>(parity) * n_slots * slot_elems +
                                        static_cast<size_t>(t.m_blk * kTpBM + row) * args.N + col0 + hf * 32;
            // the loads of up to four slots are in flight together; the additions keep the slot order
#pragma unroll 1
            for (int base = 0; base < n_slots; base += 4) {
              uint4 buf[4][4];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int sl = base + u;
                if (sl < n_slots && sl != my_slot && in_range) {
                  const __nv_bfloat16* src = src0 + static_cast<size_t>(sl) * slot_elems;
#pragma unroll
                  for (int j = 0; j < 4; ++j) buf[u][j] = ld_cg_v4(src + j * 8);
                }
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int sl = base + u;
                if (sl >= n_slots) continue;
                if (sl == my_slot) {
#pragma unroll
                  for (int i = 0; i < 32; ++i) sum[i] += __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[i])));
                } else if (in_range) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&buf[u][j]);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                      const float2 f = __bfloat1622float2(h[q]);
                      sum[j * 8 + q * 2] += f.x;
                      sum[j * 8 + q * 2 + 1] += f.y;
                    }
                  }
                }
              }
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) packed[hf * 16 + i] = pack_bf16x2(sum[2 * i], sum[2 * i + 1]);
          }
          const int buf = chunk_counter & 1;
          if (issuer) tma_wait_group_read<1>();
          named_bar_sync(1, 128);
          uint8_t* srow = staging + buf * kTpStaging + row * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          fence_proxy_async_smem();
          named_bar_sync(1, 128);
          if (issuer) {
            if (col0 < args.N) tma_store_2d(&tmD, smem_u32(staging + buf * kTpStaging), col0, t.m_blk * kTpBM);
            tma_commit_group();
          }
          ++chunk_counter;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
      // Own tiles add the peers' partial tiles. The 128 bytes a thread needs from the first peer for chunk c + 1 are
      // requested while chunk c is converted and stored, so their latency (the data was written over NVLink into this
      // GPU's memory) is not paid once per chunk in sequence.
      const bool add_partials = (COMM == 2 && owner == args.rank && !(args.probe & 2));
      const int p_first = (args.rank == 0) ? 1 : 0;
      uint4 pre[8];
      auto partial_src = [&](int p, int c) -> const __nv_bfloat16* {
        return args.recv_local + (static_cast<size_t>(parity) * args.tp + p) * slot_elems +
               static_cast<size_t>(local_row) * args.N + t.n_blk * BN + c * 64;
      };
      if (add_partials && t.n_blk * BN < args.N) {
        const __nv_bfloat16* src = partial_src(p_first, 0);
#pragma unroll
        for (int j = 0; j < 8; ++j) pre[j] = ld_cg_v4(src + j * 8);
      }
#pragma unroll 1
      for (int c = 0; c < NUM_CHUNKS; ++c) {
        uint32_t v0[32], v1[32], packed[32];
        tmem_ld_32x32b_x32(t_addr + c * 64, v0);
        tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
        tmem_ld_wait();
        const int col0 = t.n_blk * BN + c * 64;
        if (add_partials && col0 < args.N) {
          for (int p = 0; p < args.tp; ++p) {
            if (p == args.rank) continue;
            const __nv_bfloat16* src = partial_src(p, c);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint4 u = (p == p_first) ? pre[j] : ld_cg_v4(src + j * 8);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 f = __bfloat1622float2(h[q]);
                const int idx = j * 8 + q * 2;
                if (idx < 32) {
                  v0[idx] = __float_as_uint(__uint_as_float(v0[idx]) + f.x);
                  v0[idx + 1] = __float_as_uint(__uint_as_float(v0[idx + 1]) + f.y);
                } else {
                  v1[idx - 32] = __float_as_uint(__uint_as_float(v1[idx - 32]) + f.x);
                  v1[idx - 31] = __float_as_uint(__uint_as_float(v1[idx - 31]) + f.y);
                }
              }
            }
          }
          if (c + 1 < NUM_CHUNKS && col0 + 64 < args.N) {
            const __nv_bfloat16* src = partial_src(p_first, c + 1);
#pragma unroll
            for (int j = 0; j < 8; ++j) pre[j] = ld_cg_v4(src + j * 8);
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          packed[i] = pack_bf16x2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1]));
          packed[16 + i] = pack_bf16x2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1]));
        }
        if (COMM == 2 && owner != args.rank) {
          // stage the chunk in shared memory, then store it to the owner with coalesced 128-byte rows
          // (a warp writes four full rows per instruction; row-per-thread stores would fill only half of
          // every 32-byte sector on the link)
          const int buf = chunk_counter & 1;
          if (issuer) tma_wait_group_read<1>();
          named_bar_sync(1, 128);
          uint8_t* sbase = staging + buf * kTpStaging;
          uint8_t* srow = sbase + row * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          named_bar_sync(1, 128);
          if (col0 < args.N && !(args.probe & 1)) {
            const int et = threadIdx.x - 64;   // 0..127
            const int cj = et & 7;             // 16-byte chunk inside the row
            __nv_bfloat16* dst0 = args.recv_peer[owner] + (static_cast<size_t>(parity) * args.tp + args.rank) * slot_elems +
                                  static_cast<size_t>(mb_local * kTpBM) * args.N + col0 + cj * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 16 + (et >> 3);
              const uint4 v = *reinterpret_cast<const uint4*>(sbase + r * 128 + ((cj ^ (r & 7)) << 4));
              *reinterpret_cast<uint4*>(dst0 + static_cast<size_t>(r) * args.N) = v;
            }
          }
          ++chunk_counter;
        } else {
          const int buf = chunk_counter & 1;
          if (issuer) tma_wait_group_read<1>();
          named_bar_sync(1, 128);
          uint8_t* srow = staging + buf * kTpStaging + row * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          fence_proxy_async_smem();
          named_bar_sync(1, 128);
          if (issuer) {
            if (col0 < args.N) {
              const int d_row = (COMM == 2) ? mb_local * kTpBM : t.m_blk * kTpBM;
              tma_store_2d(&tmD, smem_u32(staging + buf * kTpStaging), col0, d_row);
            }
            tma_commit_group();
          }
          ++chunk_counter;
        }
      }
      // the accumulator has been read out: hand it back to the MMA warp BEFORE the tile is published, so that the
      // system-scope fence below (a round trip over NVLink) is not on the path of the next tile's main loop
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(acc == 0 ? tempty0 : tempty1);
        else mbar_arrive(smem_u32(&tempty_bar[acc]));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      if (COMM == 2 && owner != args.rank) {
        // all 128 threads have issued their peer stores: publish the tile. The barrier orders every thread's stores
        // before the issuer's release store, whose system scope is cumulative over them; one thread pays the round
        // trip over the link, not 128
        named_bar_sync(1, 128);
        if (issuer) {
          int* f = args.tile_flags_peer[owner] + (static_cast<size_t>(parity) * args.tp + args.rank) * tiles_per_chunk + tile_in_chunk;
          st_release_sys(f, args.epoch);
        }
      }
    }
    if (issuer) tma_wait_group<0>();
  } else {
    // ------------------------------ COMM 1: gather warps ------------------------------
    if (COMM == 1) {
      const int ct = threadIdx.x - 192;  // 0..127
      const int rows_per_item = kTpBM / kCopySlices;  // 16
      const int vec_per_row = args.K / 8;             // 16-byte vectors per row
      bool ok = true;
      // remote chunks in the order the GEMM consumes them, then the own chunk (only needed afterwards)
      for (int step = 1; step <= args.tp && ok; ++step) {
        const int p = (args.rank + step) % args.tp;
        if (p != args.rank) {
          if (ct == 0) ok = wait_flag_ge<true>(args.ready_local + p, args.epoch, abort_flag, args.status);
          ok = named_bar_and(3, 128, ok);
          if (!ok) break;
        }
        const __nv_bfloat16* src = args.peer_a[p];
        const int items = bpc * kCopySlices;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
          const int rb = item / kCopySlices, sl = item - rb * kCopySlices;
          const int row0 = rb * kTpBM + sl * rows_per_item;          // row inside the chunk
          const int total = rows_per_item * vec_per_row;
          // A load over NVLink takes a few microseconds to come back; with one load in flight per thread the link
          // idles (about 150 GB/s for the whole GPU). Eight independent loads per thread before the first store keep
          // 2.4 MB in flight over the 148 CTAs, which covers the round trip at the link's rate.
          constexpr int kInFlight = 8;
          const __nv_bfloat16* src_rows = src + static_cast<size_t>(row0) * args.lda;
          __nv_bfloat16* dst_rows = args.a_full + (static_cast<size_t>(p) * args.rows_per_chunk + row0) * args.K;
          for (int base = ct; base < total; base += 128 * kInFlight) {
            uint4 v[kInFlight];
#pragma unroll
            for (int j = 0; j < kInFlight; ++j) {
              const int i = base + j * 128;
              if (i < total) {
                const int r = i / vec_per_row, cv = i - r * vec_per_row;
                v[j] = ld_cg_v4(src_rows + static_cast<size_t>(r) * args.lda + cv * 8);
              }
            }
#pragma unroll
            for (int j = 0; j < kInFlight; ++j) {
              const int i = base + j * 128;
              if (i < total) {
                const int r = i / vec_per_row, cv = i - r * vec_per_row;
                *reinterpret_cast<uint4*>(dst_rows + static_cast<size_t>(r) * args.K + cv * 8) = v[j];
              }
            }
          }
          if (p != args.rank) {
            __threadfence();
            named_bar_sync(3, 128);
            if (ct == 0) red_release_gpu_add(args.block_flags + p * bpc + rb, 1);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA of a pair leaves while the other may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace mfb

namespace {
using namespace mfb;

bool g_tp_pair_enabled = true;
bool g_tp_rs_interleave = true;
int g_tp_probe = 0;

// Raster band of the CTA-pair walk (pairs of row blocks): 16 for K <= 4096, else 8, cut down to a divisor of the pairs
// per chunk so that a band never straddles two ranks' rows (the chunk order of the walk is what makes the waits safe).
int g_tp_band = 0;   // > 0: fixed band (benchmarks)

int tp_pair_band(int K, int rows_per_chunk) {
  const int ppc = rows_per_chunk / (2 * mfb::kTpBM);
  int band = (K <= 4096) ? 16 : 8;
  if (g_tp_band > 0) band = g_tp_band;
  while (band > 1 && (ppc < band || ppc % band)) band >>= 1;
  return band;
}

template <int BN, int STAGES, bool B_MN, int COMM, bool PAIR = false>
int tp_launch(const CUtensorMap& tA, const CUtensorMap& tAf, const CUtensorMap& tB, const CUtensorMap& tD,
              const TpArgs& a, cudaStream_t stream) {
  constexpr int STAGE_BYTES = kTpBM * kTpBK * 2 + (PAIR ? BN / 2 : BN) * kTpBK * 2;
  constexpr int SMEM = STAGES * STAGE_BYTES + 2 * kTpStaging + (2 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(SMEM <= 232448, "shared memory budget exceeded");
  auto kern = tp_gemm_kernel<BN, STAGES, B_MN, COMM, PAIR>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("tp gemm: cannot raise shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = a.num_m_blocks * a.num_n_blocks * (COMM == 3 && a.ksplit > 1 ? a.ksplit : 1);
  // COMM 1 needs the gather warps of every CTA to be resident, whatever the tile count
  int grid = (COMM == 1) ? sms : (tiles < sms ? tiles : sms);
  if (PAIR) {
    grid &= ~1;   // whole pairs; `tiles` counts 128-row blocks, i.e. one CTA each
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(COMM == 1 ? 320 : 192);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tA, tAf, tB, tD, a);
    if (e != cudaSuccess) {
      mfb_host::set_error("tp gemm (pairs): launch failed: %s", cudaGetErrorString(e));
      return 11;
    }
    return 0;
  }
  kern<<<grid, COMM == 1 ? 320 : 192, SMEM, stream>>>(tA, tAf, tB, tD, a);
  if (cudaGetLastError() != cudaSuccess) {
    mfb_host::set_error("tp gemm: launch failed");
    return 11;
  }
  return 0;
}

}  // namespace

extern "C" {

// All-gather -> GEMM. `peer_a[p]`: chunk [M/tp, K] (row pitch lda) of rank p, peer-mapped; `a_full`: local
// contiguous [M, K] buffer that holds the gathered A when the kernel ends; `block_flags`: M/128 ints, zeroed
// by this call; `ready_local` / `ready_peer[p]`: tp ints per rank in peer-mapped memory, persistent across
// calls; `epoch`: call counter (>= 1, increasing, identical on all ranks). B: [N, K] (or [K, N] when
// b_mn_major), row pitch ldb. D: [M, N] bf16, row pitch ldd.
int mfb_tp_allgather_gemm(const void* const* peer_a, long long lda, void* a_full, const void* B, void* D, int M,
                          int N, int K, int ldb, int ldd, int b_mn_major, int tp, int rank, int epoch,
                          int* block_flags, int* ready_local, int* const* ready_peer, int* status,
                          cudaStream_t stream) {
  if (tp < 2 || tp > kTpMaxRanks || M % (tp * kTpBM) || K % 8 || N < 128) {
    mfb_host::set_error("tp_allgather_gemm: unsupported M=%d N=%d K=%d tp=%d", M, N, K, tp);
    return 1;
  }
  TpArgs a = {};
  a.M = M; a.N = N; a.K = K; a.tp = tp; a.rank = rank; a.epoch = epoch; a.rows_per_chunk = M / tp;
  a.num_m_blocks = M / kTpBM; a.status = status;
  a.lda = lda; a.a_full = (__nv_bfloat16*)a_full; a.block_flags = block_flags; a.ready_local = ready_local;
  for (int p = 0; p < tp; ++p) { a.peer_a[p] = (const __nv_bfloat16*)peer_a[p]; a.ready_peer[p] = ready_peer[p]; }
  const bool bn256 = N >= 256;
  const int BN = bn256 ? 256 : 128;
  // CTA pairs: 256-wide tiles and an even number of 128-row blocks per rank
  const bool pair = g_tp_pair_enabled && bn256 && (a.rows_per_chunk % (2 * kTpBM) == 0);
  a.num_n_blocks = (N + BN - 1) / BN;
  a.band = tp_pair_band(K, a.rows_per_chunk);
  cudaMemsetAsync(block_flags, 0, sizeof(int) * a.num_m_blocks, stream);
  CUtensorMap tA, tAf, tB, tD;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = mfb_host::make_tmap_2d(&tA, peer_a[rank], 2, BF, a.rows_per_chunk, K, lda, kTpBM, kTpBK))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tAf, a_full, 2, BF, M, K, K, kTpBM, kTpBK))) return 30 + rc;
  if (b_mn_major) rc = mfb_host::make_tmap_2d(&tB, B, 2, BF, K, N, ldb, kTpBK, 64);
  else rc = mfb_host::make_tmap_2d(&tB, B, 2, BF, N, K, ldb, pair ? BN / 2 : BN, kTpBK);
  if (rc) return 40 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tD, D, 2, BF, M, N, ldd, kTpBM, 64))) return 50 + rc;
  if (pair) return b_mn_major ? tp_launch<256, 6, true, 1, true>(tA, tAf, tB, tD, a, stream)
                              : tp_launch<256, 6, false, 1, true>(tA, tAf, tB, tD, a, stream);
  if (bn256) return b_mn_major ? tp_launch<256, 4, true, 1>(tA, tAf, tB, tD, a, stream)
                               : tp_launch<256, 4, false, 1>(tA, tAf, tB, tD, a, stream);
  return b_mn_major ? tp_launch<128, 6, true, 1>(tA, tAf, tB, tD, a, stream)
                    : tp_launch<128, 6, false, 1>(tA, tAf, tB, tD, a, stream);
}

// GEMM -> reduce-scatter. A: [M, K] local (row pitch lda); B: [N, K] or [K, N]; D: this rank's [M/tp, N] bf16.
// `recv_local` / `recv_peer[p]`: peer-mapped receive buffers of 2 * tp * (M/tp) * N bf16; `tile_flags_*`:
// peer-mapped 2 * tp * (M/tp/128) * ceil(N/BN) ints, persistent across calls, zero at start of the job.
int mfb_tp_gemm_reduce_scatter(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd,
                               int b_mn_major, int tp, int rank, int epoch, void* recv_local,
                               void* const* recv_peer, int* tile_flags_local, int* const* tile_flags_peer,
                               int* status, cudaStream_t stream) {
  if (tp < 2 || tp > kTpMaxRanks || M % (tp * kTpBM) || K % 8 || N < 128 || N % 64) {
    mfb_host::set_error("tp_gemm_reduce_scatter: unsupported M=%d N=%d K=%d tp=%d", M, N, K, tp);
    return 1;
  }
  TpArgs a = {};
  a.M = M; a.N = N; a.K = K; a.tp = tp; a.rank = rank; a.epoch = epoch; a.rows_per_chunk = M / tp;
  a.num_m_blocks = M / kTpBM; a.status = status;
  a.recv_local = (__nv_bfloat16*)recv_local; a.tile_flags_local = tile_flags_local;
  for (int p = 0; p < tp; ++p) { a.recv_peer[p] = (__nv_bfloat16*)recv_peer[p]; a.tile_flags_peer[p] = tile_flags_peer[p]; }
  const bool bn256 = N >= 256;
  const int BN = bn256 ? 256 : 128;
  const bool pair = g_tp_pair_enabled && bn256 && (a.rows_per_chunk % (2 * kTpBM) == 0);
  a.num_n_blocks = (N + BN - 1) / BN;
  a.band = tp_pair_band(K, a.rows_per_chunk);
  CUtensorMap tA, tB, tD;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = mfb_host::make_tmap_2d(&tA, A, 2, BF, M, K, lda, kTpBM, kTpBK))) return 20 + rc;
  if (b_mn_major) rc = mfb_host::make_tmap_2d(&tB, B, 2, BF, K, N, ldb, kTpBK, 64);
  else rc = mfb_host::make_tmap_2d(&tB, B, 2, BF, N, K, ldb, pair ? BN / 2 : BN, kTpBK);
  if (rc) return 40 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tD, D, 2, BF, a.rows_per_chunk, N, ldd, kTpBM, 64))) return 50 + rc;
  a.probe = g_tp_probe;
  if (g_tp_rs_interleave && tp == 2) {
    // With two ranks the producer of every partial tile is 2 * lag - 1 positions ahead of its consumer, so the tile
    // at the smallest unfinished position never waits on a later one and the order cannot deadlock; with more ranks
    // the last remote chunk would come after the own tiles that need it, so chunk order is kept there.
    // two waves of remote tiles first. The tile walk goes band by band (8 pairs or 16 row blocks): a chunk must be
    // whole bands for "the first (tp-1)/tp of the tiles" to be exactly the remote ones; otherwise chunk order is kept
    const int units = pair ? (a.num_m_blocks / 2) : a.num_m_blocks;
    const int band = pair ? a.band : 16;
    if ((units / tp) % band == 0) a.rs_lag = 2 * (148 / (pair ? 2 : 1));
  }
  if (pair) return b_mn_major ? tp_launch<256, 6, true, 2, true>(tA, tA, tB, tD, a, stream)
                              : tp_launch<256, 6, false, 2, true>(tA, tA, tB, tD, a, stream);
  if (bn256) return b_mn_major ? tp_launch<256, 4, true, 2>(tA, tA, tB, tD, a, stream)
                               : tp_launch<256, 4, false, 2>(tA, tA, tB, tD, a, stream);
  return b_mn_major ? tp_launch<128, 6, true, 2>(tA, tA, tB, tD, a, stream)
                    : tp_launch<128, 6, false, 2>(tA, tA, tB, tD, a, stream);
}

// GEMM -> all-reduce (one shot). A: [M, K] local (row pitch lda); B: [N, K] or [K, N]; D: [M, N] bf16, the full sum
// on every rank. `recv_local` / `recv_peer[p]`: peer-mapped 2 * tp * ksplit * ceil(M/128)*128 * N bf16 with
// ksplit = mfb_tp_allreduce_ksplit(M, N, K); `tile_flags_*`: peer-mapped 2 * tp * 8 * flag_tiles ints, persistent
// across calls, zero at the start of the job. Any M >= 1.
// K-split used for a problem: more than 1 only with a single row block (decode), when all tile x split CTAs are
// resident at once (the reducing CTA of a tile waits for its helpers) and every split keeps at least 8 K blocks.
int mfb_tp_allreduce_ksplit(int M, int N, int K) {
  if (M > kTpBM) return 1;
  const int tiles = (N + 127) / 128;
  const int k_blocks = (K + kTpBK - 1) / kTpBK;
  int ks = 148 / tiles;
  if (ks > 8) ks = 8;
  while (ks > 1 && (k_blocks / ks < 8 || ((k_blocks + ks - 1) / ks) * (ks - 1) >= k_blocks)) --ks;
  return ks < 1 ? 1 : ks;
}

int mfb_tp_gemm_allreduce(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd,
                          int b_mn_major, int tp, int rank, int epoch, void* recv_local, void* const* recv_peer,
                          int* tile_flags_local, int* const* tile_flags_peer, int flag_tiles, int* status,
                          cudaStream_t stream) {
  if (tp < 2 || tp > kTpMaxRanks || M < 1 || K % 8 || N < 128 || N % 64 || lda % 8 || ldd % 8) {
    mfb_host::set_error("tp_gemm_allreduce: unsupported M=%d N=%d K=%d tp=%d", M, N, K, tp);
    return 1;
  }
  TpArgs a = {};
  a.M = M; a.N = N; a.K = K; a.tp = tp; a.rank = rank; a.epoch = epoch;
  a.num_m_blocks = (M + kTpBM - 1) / kTpBM; a.rows_per_chunk = a.num_m_blocks * kTpBM; a.status = status;
  a.recv_local = (__nv_bfloat16*)recv_local; a.tile_flags_local = tile_flags_local;
  for (int p = 0; p < tp; ++p) {
    a.recv_peer[p] = (__nv_bfloat16*)recv_peer[p]; a.tile_flags_peer[p] = tile_flags_peer[p];
    if ((reinterpret_cast<uintptr_t>(recv_peer[p]) & 15) || (reinterpret_cast<uintptr_t>(tile_flags_peer[p]) & 3)) {
      mfb_host::set_error("tp_gemm_allreduce: receive buffers must be 16-byte aligned");
      return 1;
    }
  }
  a.ksplit = mfb_tp_allreduce_ksplit(M, N, K);
  // few row blocks (decode): narrower tiles put more SMs to work
  const bool bn256 = a.ksplit == 1 && N >= 256 && a.num_m_blocks * ((N + 255) / 256) >= 96;
  const int BN = bn256 ? 256 : 128;
  a.num_n_blocks = (N + BN - 1) / BN;
  if (a.num_m_blocks * a.num_n_blocks > flag_tiles) {
    mfb_host::set_error("tp_gemm_allreduce: %d tiles exceed the %d flags provided", a.num_m_blocks * a.num_n_blocks, flag_tiles);
    return 1;
  }
  CUtensorMap tA, tB, tD;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = mfb_host::make_tmap_2d(&tA, A, 2, BF, M, K, lda, kTpBM, kTpBK))) return 20 + rc;
  if (b_mn_major) rc = mfb_host::make_tmap_2d(&tB, B, 2, BF, K, N, ldb, kTpBK, 64);
  else rc = mfb_host::make_tmap_2d(&tB, B, 2, BF, N, K, ldb, BN, kTpBK);
  if (rc) return 40 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tD, D, 2, BF, M, N, ldd, kTpBM, 64))) return 50 + rc;
  if (bn256) return b_mn_major ? tp_launch<256, 4, true, 3>(tA, tA, tB, tD, a, stream)
                               : tp_launch<256, 4, false, 3>(tA, tA, tB, tD, a, stream);
  return b_mn_major ? tp_launch<128, 6, true, 3>(tA, tA, tB, tD, a, stream)
                    : tp_launch<128, 6, false, 3>(tA, tA, tB, tD, a, stream);
}

// Fix the raster band of the CTA-pair walk (0 = choose from K) for A/B measurements.
void mfb_tp_set_band(int band) { g_tp_band = band; }
// Timing probes of the reduce-scatter GEMM (see TpArgs::probe); results are wrong while a probe is set.
void mfb_tp_set_probe(int bits) { g_tp_probe = bits; }

// Switch the interleaved work order of the reduce-scatter GEMM (on by default) for A/B measurements.
void mfb_tp_set_rs_interleave(int enabled) { g_tp_rs_interleave = enabled != 0; }

// Switch the CTA-pair variant of the all-gather and reduce-scatter GEMMs (on by default) for A/B measurements.
void mfb_tp_set_pair(int enabled) { g_tp_pair_enabled = enabled != 0; }

// Upper bound of ceil(N / BN) that the flag arrays must provide room for.
int mfb_tp_num_n_blocks(int N) { return N >= 256 ? (N + 255) / 256 : (N + 127) / 128; }

}  // extern "C"
