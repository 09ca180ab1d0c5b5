// bf16 GEMM for sm_100a: persistent, warp-specialised, TMA-fed, tcgen05.mma with the
// accumulator in tensor memory (double-buffered so the epilogue of tile i overlaps the
// main loop of tile i+1), TMA-store epilogue.
//
//   D[M,N] = sum_k A(m,k) * B(n,k)        fp32 accumulation
//
// Operand storage ("major-ness") is a template switch so that forward, dgrad and wgrad
// of a linear layer all run without a transpose pass:
//   A K-major : A is [M,K] row-major      A MN-major : A is [K,M] row-major
//   B K-major : B is [N,K] row-major      B MN-major : B is [K,N] row-major
// forward  y  = x  W^T : A=x  (K-major),  B=W  (K-major)
// dgrad    dx = dy W   : A=dy (K-major),  B=W  (MN-major)
// wgrad    dW = dy^T x : A=dy (MN-major), B=x  (MN-major)   (optionally D += via TMA reduce)
//
// Grouped (MoE) modes reuse the same pipeline:
//   mode 1 "ragged M": rows of A/D are expert segments padded to 128; a device table maps each
//          128-row block to its expert, B holds one matrix per expert.
//   mode 2 "ragged K": per-expert wgrad; the reduction runs over that expert's row segment.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (TMEM -> registers -> swizzled smem -> TMA store).
#include "common.cuh"

namespace mfb {

constexpr int kBM = 128;
constexpr int kBK = 64;  // 128 bytes of bf16: one swizzle row
constexpr int kEpiThreads = 128;
constexpr int kThreads = 192;
constexpr int kStagingBytes = 128 * 128;  // one epilogue chunk: 128 rows x 128 bytes

struct GemmArgs {
  int M, N, K;         // logical problem (per group in mode 2)
  int num_m_blocks;    // upper bound in mode 1
  int num_n_blocks;
  int mode;            // 0 dense, 1 ragged-M grouped, 2 ragged-K grouped (wgrad)
  int num_groups;
  int group_b_stride;  // rows of B per group (mode 1); rows of D per group (mode 2)
  const int* m_block_group;     // mode 1: [num_m_blocks] expert of each 128-row block
  const int* num_m_blocks_dev;  // mode 1: actual number of row blocks (device scalar)
  const int* group_offsets;     // mode 2: [G+1] padded row offsets (multiples of 128)
  int* status;
};

struct Tile {
  int a_mn0, b_mn0;  // first row (M / N index) of the tile in A / B
  int a_k0, b_k0;    // first reduction index in A / B
  int k_blocks;
  int d_row, d_col;
};

__device__ __forceinline__ int total_tiles(const GemmArgs& g) {
  if (g.mode == 1) {
    int mb = g.num_m_blocks_dev ? *g.num_m_blocks_dev : g.num_m_blocks;
    mb = mb < g.num_m_blocks ? mb : g.num_m_blocks;
    return mb * g.num_n_blocks;
  }
  if (g.mode == 2) return g.num_groups * g.num_m_blocks * g.num_n_blocks;
  return g.num_m_blocks * g.num_n_blocks;
}

template <int BN, bool B_MN>
__device__ __forceinline__ Tile get_tile(const GemmArgs& g, int tile, int mb_total) {
  Tile t;
  if (g.mode == 2) {
    const int per_group = g.num_m_blocks * g.num_n_blocks;
    const int grp = tile / per_group;
    const int r = tile - grp * per_group;
    const int m_blk = r % g.num_m_blocks;
    const int n_blk = r / g.num_m_blocks;
    const int k0 = g.group_offsets[grp];
    const int k1 = g.group_offsets[grp + 1];
    t.a_mn0 = m_blk * kBM;
    t.b_mn0 = n_blk * BN;
    t.a_k0 = k0;
    t.b_k0 = k0;
    t.k_blocks = (k1 - k0 + kBK - 1) / kBK;
    t.d_row = grp * g.group_b_stride + m_blk * kBM;
    t.d_col = n_blk * BN;
    return t;
  }
  // banded rasterisation: 16 row blocks share their B tiles through L2
  constexpr int kBand = 16;
  const int tiles_per_band = kBand * g.num_n_blocks;
  const int band = tile / tiles_per_band;
  const int first_m = band * kBand;
  const int band_h = (mb_total - first_m) < kBand ? (mb_total - first_m) : kBand;
  const int r = tile - band * tiles_per_band;
  const int m_blk = first_m + r % band_h;
  const int n_blk = r / band_h;
  t.a_mn0 = m_blk * kBM;
  t.a_k0 = 0;
  t.b_mn0 = n_blk * BN;
  t.b_k0 = 0;
  t.k_blocks = (g.K + kBK - 1) / kBK;
  t.d_row = m_blk * kBM;
  t.d_col = n_blk * BN;
  if (g.mode == 1) {
    const int grp = g.m_block_group[m_blk];
    if (B_MN) t.b_k0 = grp * g.group_b_stride;
    else t.b_mn0 += grp * g.group_b_stride;
  }
  return t;
}

// OUT_MODE: 0 bf16 store, 1 f32 store, 2 f32 reduce-add, 3 bf16 reduce-add
template <int BN, int STAGES, bool A_MN, bool B_MN, int OUT_MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const GemmArgs args) {
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BN * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;  // two accumulators of BN fp32 columns
  constexpr bool OUT_F32 = (OUT_MODE == 1 || OUT_MODE == 2);
  constexpr int CHUNK_COLS = OUT_F32 ? 32 : 64;  // 128 bytes per row per chunk
  constexpr int NUM_CHUNKS = BN / CHUNK_COLS;
  constexpr uint32_t IDESC = umma_idesc_bf16(kBM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tfull_bar[s]), 1);
      mbar_init(smem_u32(&tempty_bar[s]), 4);  // one arrival per epilogue warp
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int n_tiles = total_tiles(args);
  const int mb_total = (args.mode == 1) ? n_tiles / args.num_n_blocks : args.num_m_blocks;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const Tile t = get_tile<BN, B_MN>(args, tile, mb_total);
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, args.status,
                         kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, STAGE_BYTES);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_BYTES;
          if (A_MN) {
#pragma unroll
            for (int at = 0; at < kBM / 64; ++at)
              tma_load_2d(a_dst + at * (kBK * 128), &tmA, fb, t.a_mn0 + at * 64, t.a_k0 + kb * kBK);
          } else {
            tma_load_2d(a_dst, &tmA, fb, t.a_k0 + kb * kBK, t.a_mn0);
          }
          if (B_MN) {
#pragma unroll
            for (int at = 0; at < BN / 64; ++at)
              tma_load_2d(b_dst + at * (kBK * 128), &tmB, fb, t.b_mn0 + at * 64, t.b_k0 + kb * kBK);
          } else {
            tma_load_2d(b_dst, &tmB, fb, t.b_k0 + kb * kBK, t.b_mn0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const Tile t = get_tile<BN, B_MN>(args, tile, mb_total);
        if (t.k_blocks == 0) continue;  // empty expert: the epilogue writes zeros by itself
        ok = mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, args.status,
                       kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, args.status,
                         kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_base = a_base + A_BYTES;
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t a_desc = A_MN ? umma_desc_mnmajor_sw128(a_base + k * 16 * 128, kBK * 128)
                                         : umma_desc_kmajor_sw128(a_base + k * 32);
            const uint64_t b_desc = B_MN ? umma_desc_mnmajor_sw128(b_base + k * 16 * 128, kBK * 128)
                                         : umma_desc_kmajor_sw128(b_base + k * 32);
            umma_f16_ss(d_tmem, a_desc, b_desc, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));  // smem stage free once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&tfull_bar[acc]));  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ------------------------------
    const int ew = warp & 3;           // TMEM lane quarter this warp may read
    const int row = ew * 32 + lane;    // row of the 128-row tile
    const bool issuer = (threadIdx.x == 64);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t chunk_counter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const Tile t = get_tile<BN, B_MN>(args, tile, mb_total);
      if (t.k_blocks > 0) {
        ok = mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, args.status,
                       kStatusWaitTimeoutEpilogue);
      }
      // one decision for all 128 epilogue threads, so nobody is left alone at a named barrier
      ok = named_bar_and(2, kEpiThreads, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < NUM_CHUNKS; ++c) {
        uint32_t packed[32];
        if (OUT_F32) {
          if (t.k_blocks > 0) {
            tmem_ld_32x32b_x32(t_addr + c * 32, packed);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) packed[i] = 0;
          }
        } else {
          uint32_t v0[32], v1[32];
          if (t.k_blocks > 0) {
            tmem_ld_32x32b_x32(t_addr + c * 64, v0);
            tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) { v0[i] = 0; v1[i] = 0; }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            packed[i] = pack_bf16x2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1]));
            packed[16 + i] = pack_bf16x2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1]));
          }
        }
        const int buf = chunk_counter & 1;
        // the TMA store that last read this staging buffer must have finished reading it
        if (issuer) tma_wait_group_read<1>();
        named_bar_sync(1, kEpiThreads);
        uint8_t* srow = staging + buf * kStagingBytes + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint4 v = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) = v;
        }
        fence_proxy_async_smem();
        named_bar_sync(1, kEpiThreads);
        if (issuer) {
          const int x = t.d_col + c * CHUNK_COLS;
          if (x < args.N) {
            const uint32_t src = smem_u32(staging + buf * kStagingBytes);
            if (OUT_MODE >= 2) tma_reduce_add_2d(&tmD, src, x, t.d_row);
            else tma_store_2d(&tmD, src, x, t.d_row);
          }
          tma_commit_group();
        }
        ++chunk_counter;
      }
      if (t.k_blocks > 0) {
        // every tcgen05.ld of this accumulator has completed (wait::ld above)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    if (issuer) tma_wait_group<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace mfb

// ---------------------------------------------------------------------------------------
// host launcher
// ---------------------------------------------------------------------------------------
namespace {

using namespace mfb;

int g_num_sms = 0;

int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int OUT_MODE>
int launch(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, const GemmArgs& args,
           int max_tiles, int sm_limit, cudaStream_t stream) {
  constexpr int STAGE_BYTES = kBM * kBK * 2 + BN * kBK * 2;
  constexpr int SMEM = STAGES * STAGE_BYTES + 2 * kStagingBytes + (2 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(SMEM <= 232448, "shared memory budget exceeded");
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN, OUT_MODE>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) {
      mfb_host::set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 10;
    }
    attr_set = true;
  }
  int sms = num_sms();
  if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
  int grid = max_tiles < sms ? max_tiles : sms;
  if (grid < 1) grid = 1;
  kern<<<grid, kThreads, SMEM, stream>>>(tA, tB, tD, args);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    mfb_host::set_error("gemm launch: %s", cudaGetErrorString(e));
    return 11;
  }
  return 0;
}

template <int BN, int STAGES>
int dispatch(int a_mn, int b_mn, int out_mode, const CUtensorMap& tA, const CUtensorMap& tB,
             const CUtensorMap& tD, const GemmArgs& args, int max_tiles, int sm_limit,
             cudaStream_t stream) {
#define MFB_CASE(AM, BMJ, OM)                                                                   \
  if (a_mn == AM && b_mn == BMJ && out_mode == OM)                                              \
    return launch<BN, STAGES, AM != 0, BMJ != 0, OM>(tA, tB, tD, args, max_tiles, sm_limit, stream);
  MFB_CASE(0, 0, 0)
  MFB_CASE(0, 0, 1)
  MFB_CASE(0, 1, 0)
  MFB_CASE(0, 1, 1)
  MFB_CASE(1, 1, 0)
  MFB_CASE(1, 1, 1)
  MFB_CASE(1, 1, 2)
  MFB_CASE(1, 1, 3)
  MFB_CASE(0, 0, 2)
  MFB_CASE(1, 0, 0)
#undef MFB_CASE
  mfb_host::set_error("gemm: unsupported combination a_mn=%d b_mn=%d out_mode=%d", a_mn, b_mn, out_mode);
  return 12;
}

}  // namespace

extern "C" {

// Dense or grouped bf16 GEMM. See the file header for operand conventions.
//   mode 0: D[M,N] (ldd) = A x B.
//   mode 1: A/D rows are expert segments padded to 128 rows; `m_block_group[b]` is the expert of
//           row block b and `num_m_blocks_dev` the device-side count of valid row blocks
//           (`M` is the allocated upper bound of rows). B holds `num_groups` matrices stacked on its
//           row axis: [G*N, K] when K-major, [G*K, N] when MN-major.
//   mode 2: per-expert wgrad: D[g] [M,N] = A[rows_g, M]^T B[rows_g, N] with
//           rows_g = [group_offsets[g], group_offsets[g+1]); A and B MN-major; D is [G*M, N].
// out_mode: 0 bf16 store, 1 f32 store, 2 f32 reduce-add into D, 3 bf16 reduce-add into D.
// `status` is a device int that receives a non-zero code if a bounded wait ran out (may be null).
// `sm_limit` > 0 restricts the persistent grid (used to leave SMs to a concurrent kernel).
int mfb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd,
                  int a_mn_major, int b_mn_major, int out_mode, int mode, int num_groups,
                  const int* m_block_group, const int* num_m_blocks_dev, const int* group_offsets,
                  int total_rows, int* status, int sm_limit, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K < 0) {
    mfb_host::set_error("gemm: bad shape M=%d N=%d K=%d", M, N, K);
    return 1;
  }
  const bool bn256 = (N >= 256);
  const int BN = bn256 ? 256 : 128;
  const bool out_f32 = (out_mode == 1 || out_mode == 2);

  CUtensorMap tA, tB, tD;
  int rc = 0;
  // extents of the stored operands
  uint64_t a_rows, a_cols, b_rows, b_cols, d_rows;
  if (mode == 0) {
    a_rows = a_mn_major ? K : M;  a_cols = a_mn_major ? M : K;
    b_rows = b_mn_major ? K : N;  b_cols = b_mn_major ? N : K;
    d_rows = M;
  } else if (mode == 1) {
    if (a_mn_major) { mfb_host::set_error("gemm mode 1 needs K-major A"); return 2; }
    a_rows = M;  a_cols = K;
    b_rows = b_mn_major ? (uint64_t)num_groups * K : (uint64_t)num_groups * N;
    b_cols = b_mn_major ? N : K;
    d_rows = M;
    if (b_mn_major && (K % kBK) != 0) { mfb_host::set_error("gemm mode 1 dgrad needs K %% 64 == 0"); return 2; }
  } else {
    if (!a_mn_major || !b_mn_major) { mfb_host::set_error("gemm mode 2 needs MN-major A and B"); return 2; }
    if (M % kBM != 0) { mfb_host::set_error("gemm mode 2 needs M %% 128 == 0"); return 2; }
    a_rows = total_rows;  a_cols = M;
    b_rows = total_rows;  b_cols = N;
    d_rows = (uint64_t)num_groups * M;
  }
  if (a_mn_major) rc = mfb_host::make_tmap_2d(&tA, A, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a_rows, a_cols, lda, kBK, 64);
  else            rc = mfb_host::make_tmap_2d(&tA, A, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a_rows, a_cols, lda, kBM, kBK);
  if (rc) return 20 + rc;
  if (b_mn_major) rc = mfb_host::make_tmap_2d(&tB, B, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b_rows, b_cols, ldb, kBK, 64);
  else            rc = mfb_host::make_tmap_2d(&tB, B, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b_rows, b_cols, ldb, BN, kBK);
  if (rc) return 30 + rc;
  if (out_f32) rc = mfb_host::make_tmap_2d(&tD, D, 4, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, d_rows, N, ldd, kBM, 32);
  else         rc = mfb_host::make_tmap_2d(&tD, D, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, d_rows, N, ldd, kBM, 64);
  if (rc) return 40 + rc;

  GemmArgs args;
  args.M = M; args.N = N; args.K = K;
  args.num_m_blocks = (M + kBM - 1) / kBM;
  args.num_n_blocks = (N + BN - 1) / BN;
  args.mode = mode;
  args.num_groups = num_groups;
  args.group_b_stride = (mode == 1) ? (b_mn_major ? K : N) : M;
  args.m_block_group = m_block_group;
  args.num_m_blocks_dev = num_m_blocks_dev;
  args.group_offsets = group_offsets;
  args.status = status;
  int max_tiles = args.num_m_blocks * args.num_n_blocks * (mode == 2 ? num_groups : 1);

  if (bn256) return dispatch<256, 4>(a_mn_major, b_mn_major, out_mode, tA, tB, tD, args, max_tiles, sm_limit, stream);
  return dispatch<128, 6>(a_mn_major, b_mn_major, out_mode, tA, tB, tD, args, max_tiles, sm_limit, stream);
}

}  // extern "C"
