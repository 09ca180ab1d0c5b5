// Block-scaled fp8 (e4m3) GEMM for sm_100a: DeepSeek-V3 style scales, tcgen05 kind::f8f6f4, TMEM partials.
//
//   D[m, n] = sum_kb  sa[kb, m] * sb[g, n / 128, kb] * sum_{k in block kb} A[m, k] * B[g * N + n, k]
//
//   A   [M, K]   e4m3, K-major; one fp32 scale per row and per block of 128 k   -> sa [K/128, M]
//   B   [G*N, K] e4m3, K-major; one fp32 scale per 128 x 128 block              -> sb [G, N/128, K/128]
//   D   [M, N]   bf16
//
// The scale changes every 128 k, so a tile cannot accumulate in the tensor core across the whole reduction:
// each K block (4 MMAs of k = 32) goes into a fresh TMEM partial (double-buffered), the four epilogue warps read the
// partial, multiply by sa * sb and add it to per-thread fp32 accumulators (one output row of 128 columns per
// thread) while the tensor core already works on the next block. Tiles are 128 x 128, the grid is persistent,
// operands arrive by TMA through a 5-stage ring, the bf16 result leaves through swizzled staging and TMA stores.
//
// Small M (one row block, few column tiles; the decode regime, where the job is to stream the weights once at HBM
// speed): the K range of a tile is split over the KS = 2, 4 or 8 CTAs of a thread-block cluster, so KS times as many
// SMs pull weights. Each CTA accumulates its K slice as above, then the cluster reduce-scatters the 128 x 128 fp32
// partials through distributed shared memory: CTA c receives columns [c * 128 / KS, (c + 1) * 128 / KS) of every
// partial into its (now idle) operand ring, adds them in rank order (the same bits on every run) and stores its
// slice of the bf16 result.
//
// mode 0: dense. mode 1: ragged-M grouped (MoE experts): rows of A / D are expert segments padded to 128 rows,
// `m_block_group[b]` gives the expert of row block b and `num_m_blocks_dev` the number of row blocks in use.
//
// The reference only de-quantises such checkpoints to bf16 on the host
// (toolkit/weight_convert/deepseekv3/convert_deepseekv3_hf_weight.py:67-114); keeping the weights in fp8 on the
// device halves their HBM traffic and doubles the tensor-core rate.
#include <cuda_fp8.h>

#include "common.cuh"

namespace mfb {

constexpr int kF8BM = 128, kF8BN = 128, kF8BK = 128;   // 128 fp8 = one 128-byte swizzle row
constexpr int kF8Stages = 5;
constexpr int kF8Threads = 192;
constexpr int kF8TileBytes = 128 * 128;                 // one operand tile per stage

struct F8Args {
  int M, N, K, kblocks;
  int num_m_blocks, num_n_blocks;
  int mode, num_groups;
  long long sa_ld;               // elements between consecutive K blocks of sa (>= rows of A)
  const float* sa;               // [K/128, sa_ld]
  const float* sb;               // [G, N/128, K/128]
  const int* m_block_group;
  const int* num_m_blocks_dev;
  int* status;
  __nv_bfloat16* D;              // split-K path stores its column slices with plain stores
  long long ldd;
};

__device__ __forceinline__ uint32_t f8_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t f8_mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void f8_st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// every thread of every CTA of the cluster; release / acquire at cluster scope
__device__ __forceinline__ void f8_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void umma_f8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int KS>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_blockscaled_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                            const __grid_constant__ CUtensorMap tmD, const F8Args args) {
  constexpr int STAGE_BYTES = 2 * kF8TileBytes;
  constexpr uint32_t IDESC = umma_idesc_e4m3(kF8BM, kF8BN);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kF8Stages * STAGE_BYTES;            // 2 x [128 rows][128 B] bf16 images
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * kF8TileBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kF8Stages;
  uint64_t* pfull = bars + 2 * kF8Stages;        // [2] partial of a K block complete in tensor memory
  uint64_t* pempty = bars + 2 * kF8Stages + 2;   // [2] partial drained by the epilogue warps (4 arrivals)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kF8Stages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // split-K launches have exactly one cluster per tile; a cluster without a tile leaves as a whole (its threads
  // would otherwise meet the cluster barriers below in unequal numbers)
  if (KS > 1 && static_cast<int>(blockIdx.x) / KS >= args.num_m_blocks * args.num_n_blocks) return;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kF8Stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&pfull[s]), 1);
      mbar_init(smem_u32(&pempty[s]), 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  int mb_total = args.num_m_blocks;
  if (args.mode == 1 && args.num_m_blocks_dev) {
    const int v = *args.num_m_blocks_dev;
    mb_total = v < mb_total ? v : mb_total;
  }
  const int n_tiles = mb_total * args.num_n_blocks;
  // tile -> (row block, column block): column-major over row blocks so that a wave shares B tiles through L2
  auto tile_mn = [&](int tile, int& m_blk, int& n_blk) { m_blk = tile % mb_total; n_blk = tile / mb_total; };
  // KS = 1: persistent over tiles, whole K per tile. KS > 1: one tile per cluster, K blocks [kb_lo, kb_hi) per CTA.
  const int krank = KS > 1 ? static_cast<int>(f8_cluster_ctarank()) : 0;
  const int tile_first = KS > 1 ? static_cast<int>(blockIdx.x) / KS : static_cast<int>(blockIdx.x);
  const int tile_step = KS > 1 ? n_tiles : static_cast<int>(gridDim.x);       // KS > 1: a single iteration
  const int kb_lo = KS > 1 ? krank * args.kblocks / KS : 0;
  const int kb_hi = KS > 1 ? (krank + 1) * args.kblocks / KS : args.kblocks;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = tile_first; tile < n_tiles && ok; tile += tile_step) {
        int m_blk, n_blk;
        tile_mn(tile, m_blk, n_blk);
        const int grp = args.mode == 1 ? args.m_block_group[m_blk] : 0;
        const int b_row = grp * args.N + n_blk * kF8BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, STAGE_BYTES);
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, fb, kb * kF8BK, m_blk * kF8BM);
          tma_load_2d(a_dst + kF8TileBytes, &tmB, fb, kb * kF8BK, b_row);
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
    if constexpr (KS > 1) { f8_cluster_sync(); f8_cluster_sync(); }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t blk = 0;      // K blocks issued so far: partial buffer = blk & 1
      bool ok = true;
      for (int tile = tile_first; tile < n_tiles && ok; tile += tile_step) {
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++blk) {
          const int buf = blk & 1;
          ok = mbar_wait(smem_u32(&pempty[buf]), ((blk >> 1) & 1) ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_base = a_base + kF8TileBytes;
#pragma unroll
          for (int k = 0; k < kF8BK / 32; ++k)   // k = 32 per instruction for 8-bit operands: 32 bytes of the row
            umma_f8_ss(tmem_base + buf * kF8BN, umma_desc_kmajor_sw128(a_base + k * 32),
                       umma_desc_kmajor_sw128(b_base + k * 32), IDESC, k > 0 ? 1u : 0u);
          umma_commit(smem_u32(&empty_bar[stage]));
          umma_commit(smem_u32(&pfull[buf]));
          if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
    if constexpr (KS > 1) { f8_cluster_sync(); f8_cluster_sync(); }
  } else {
    const int ew = warp & 3;
    const int row = ew * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    const bool issuer = (threadIdx.x == 64);
    uint32_t blk = 0;
    bool ok = true;
    const int nkb = args.kblocks;
    for (int tile = tile_first; tile < n_tiles && ok; tile += tile_step) {
      int m_blk, n_blk;
      tile_mn(tile, m_blk, n_blk);
      const int grp = args.mode == 1 ? args.m_block_group[m_blk] : 0;
      const float* sa = args.sa + (long long)m_blk * kF8BM + row;
      const float* sb = args.sb + ((long long)grp * args.num_n_blocks + n_blk) * nkb;
      float acc[kF8BN];
#pragma unroll
      for (int i = 0; i < kF8BN; ++i) acc[i] = 0.f;
      // the scales of the next two K blocks are fetched ahead: their latency would otherwise sit between two partials
      float sc0 = kb_lo < kb_hi ? sa[(long long)kb_lo * args.sa_ld] * sb[kb_lo] : 0.f;
      float sc1 = kb_lo + 1 < kb_hi ? sa[(long long)(kb_lo + 1) * args.sa_ld] * sb[kb_lo + 1] : 0.f;
      for (int kb = kb_lo; kb < kb_hi; ++kb, ++blk) {
        const int buf = blk & 1;
        const float scale = sc0;
        sc0 = sc1;
        if (kb + 2 < kb_hi) sc1 = sa[(long long)(kb + 2) * args.sa_ld] * sb[kb + 2];
        ok = mbar_wait(smem_u32(&pfull[buf]), (blk >> 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
        ok = __all_sync(0xffffffffu, ok);             // the tensor-memory loads need the whole warp
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_base + buf * kF8BN + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(r[i]), scale, acc[c * 32 + i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&pempty[buf]));
      }
      if constexpr (KS > 1) {
        // ---- reduce-scatter of the K-slice partials over the cluster ----
        constexpr int W = kF8BN / KS;                 // columns owned by each CTA
        ok = named_bar_and(2, 128, ok);
        f8_cluster_sync();                            // every CTA of the cluster has drained its operand ring
        const bool live = ok && (m_blk * kF8BM + row < args.M);
        if (live) {
#pragma unroll
          for (int c = 0; c < KS; ++c) {
            // slot [krank][row][W] of CTA c's receive buffer (the start of its ring)
            const uint32_t dst = f8_mapa(smem_u32(smem) + ((krank * kF8BM + row) * W) * 4, c);
#pragma unroll
            for (int v = 0; v < W / 4; ++v)
              f8_st_cluster_v4(dst + v * 16, acc[c * W + 4 * v], acc[c * W + 4 * v + 1], acc[c * W + 4 * v + 2],
                               acc[c * W + 4 * v + 3]);
          }
        }
        f8_cluster_sync();                            // all slices have landed
        if (live) {
          float out[W];
#pragma unroll
          for (int i = 0; i < W; ++i) out[i] = 0.f;
          const float4* recv = reinterpret_cast<const float4*>(smem);
#pragma unroll
          for (int r = 0; r < KS; ++r) {
#pragma unroll
            for (int v = 0; v < W / 4; ++v) {
              const float4 x = recv[((r * kF8BM + row) * W) / 4 + v];
              out[4 * v] += x.x; out[4 * v + 1] += x.y; out[4 * v + 2] += x.z; out[4 * v + 3] += x.w;
            }
          }
          __nv_bfloat16* drow = args.D + (long long)(m_blk * kF8BM + row) * args.ldd + n_blk * kF8BN + krank * W;
#pragma unroll
          for (int v = 0; v < W / 8; ++v)
            *reinterpret_cast<uint4*>(drow + v * 8) =
                make_uint4(pack_bf16x2(out[8 * v], out[8 * v + 1]), pack_bf16x2(out[8 * v + 2], out[8 * v + 3]),
                           pack_bf16x2(out[8 * v + 4], out[8 * v + 5]), pack_bf16x2(out[8 * v + 6], out[8 * v + 7]));
        }
        break;                                        // one tile per cluster
      }
      ok = named_bar_and(2, 128, ok);                 // the four warps leave together or not at all
      if (!ok) break;
      // bf16 result -> two swizzled [128][128 B] images -> TMA store
      if (issuer) tma_wait_group_read<0>();
      named_bar_sync(1, 128);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint8_t* srow = staging + half * kF8TileBytes + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float* a8 = acc + half * 64 + j * 8;
          *reinterpret_cast<uint4*>(srow + ((j ^ (row & 7)) << 4)) =
              make_uint4(pack_bf16x2(a8[0], a8[1]), pack_bf16x2(a8[2], a8[3]), pack_bf16x2(a8[4], a8[5]),
                         pack_bf16x2(a8[6], a8[7]));
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1, 128);
      if (issuer) {
        tma_store_2d(&tmD, smem_u32(staging), n_blk * kF8BN, m_blk * kF8BM);
        tma_store_2d(&tmD, smem_u32(staging) + kF8TileBytes, n_blk * kF8BN + 64, m_blk * kF8BM);
        tma_commit_group();
      }
    }
    if (issuer) tma_wait_group<0>();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// x [T, K] bf16 -> q [T, K] e4m3 and sa [K/128, sa_ld] (scale = amax / 448 per row and block of 128);
// one warp per (row, block): lane handles 4 elements.
__global__ void quant_act_1x128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                                       long long ldq, float* __restrict__ sa, long long sa_ld, long long T, int kblocks) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= T * kblocks) return;
  const long long t = w / kblocks;
  const int kb = (int)(w - t * kblocks);
  const uint2 u = *reinterpret_cast<const uint2*>(x + t * ldx + kb * 128 + lane * 4);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  const float inv = 1.f / scale;
  const __nv_fp8_storage_t q0 = __nv_cvt_float_to_fp8(a.x * inv, __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8_storage_t q1 = __nv_cvt_float_to_fp8(a.y * inv, __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8_storage_t q2 = __nv_cvt_float_to_fp8(b.x * inv, __NV_SATFINITE, __NV_E4M3);
  const __nv_fp8_storage_t q3 = __nv_cvt_float_to_fp8(b.y * inv, __NV_SATFINITE, __NV_E4M3);
  *reinterpret_cast<uint32_t*>(q + t * ldq + kb * 128 + lane * 4) =
      (uint32_t)q0 | ((uint32_t)q1 << 8) | ((uint32_t)q2 << 16) | ((uint32_t)q3 << 24);
  if (lane == 0) sa[(long long)kb * sa_ld + t] = scale;
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// CTAs per cluster that share the K range of a tile (1 = no split). Splitting pays when one row block and few column
// tiles would leave most SMs without weights to stream; a cluster of 8 needs 8 free SMs in one GPC, so at most 128
// CTAs of such clusters are resident at a time.
static int g_f8_split_enabled = 1;
void mfb_gemm_fp8_enable_ksplit(int on) { g_f8_split_enabled = on ? 1 : 0; }   // for A/B timing

int mfb_gemm_fp8_ksplit(int M, int N, int K, int mode, long long ldd) {
  if (!g_f8_split_enabled || mode != 0 || M > kF8BM || ldd % 8) return 1;
  const int tiles = N / kF8BN, kblocks = K / kF8BK;
  if (tiles * 8 <= 128 && kblocks >= 16) return 8;
  if (tiles * 4 <= 144 && kblocks >= 8) return 4;
  if (tiles * 2 <= 148 && kblocks >= 4) return 2;
  return 1;
}

// See the file header. lda / ldb in bytes (= elements), ldd in bf16 elements. M is the row bound in mode 1.
int mfb_gemm_fp8_blockscaled(const void* A, const void* B, void* D, const float* sa, long long sa_ld, const float* sb,
                             int M, int N, int K, long long lda, long long ldb, long long ldd, int mode, int num_groups,
                             const int* m_block_group, const int* num_m_blocks_dev, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || N % kF8BN || K % kF8BK) {
    mfb_host::set_error("gemm_fp8: M=%d N=%d K=%d (N and K must be multiples of 128)", M, N, K);
    return 1;
  }
  if (mode == 1 && M % kF8BM) { mfb_host::set_error("gemm_fp8 grouped: rows %d must be a multiple of 128", M); return 1; }
  const int G = mode == 1 ? num_groups : 1;
  CUtensorMap tA, tB, tD;
  int rc;
  if ((rc = mfb_host::make_tmap_2d(&tA, A, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, M, K, lda, kF8BM, kF8BK))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tB, B, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint64_t)G * N, K, ldb, kF8BN, kF8BK))) return 30 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tD, D, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, M, N, ldd, kF8BM, 64))) return 40 + rc;
  F8Args a;
  a.M = M; a.N = N; a.K = K; a.kblocks = K / kF8BK;
  a.num_m_blocks = (M + kF8BM - 1) / kF8BM; a.num_n_blocks = N / kF8BN;
  a.mode = mode; a.num_groups = G; a.sa_ld = sa_ld; a.sa = sa; a.sb = sb;
  a.m_block_group = m_block_group; a.num_m_blocks_dev = num_m_blocks_dev; a.status = status;
  a.D = reinterpret_cast<__nv_bfloat16*>(D); a.ldd = ldd;
  constexpr int SMEM = kF8Stages * 2 * kF8TileBytes + 2 * kF8TileBytes + (2 * kF8Stages + 4) * 8 + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_blockscaled_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_fp8_blockscaled_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_fp8_blockscaled_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(gemm_fp8_blockscaled_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("gemm_fp8: cannot raise the shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  int tiles = a.num_m_blocks * a.num_n_blocks;
  const int ks = mfb_gemm_fp8_ksplit(M, N, K, mode, ldd);
  if (ks > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * ks);
    cfg.blockDim = dim3(kF8Threads);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ks; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = ks == 2   ? cudaLaunchKernelEx(&cfg, gemm_fp8_blockscaled_kernel<2>, tA, tB, tD, a)
                    : ks == 4 ? cudaLaunchKernelEx(&cfg, gemm_fp8_blockscaled_kernel<4>, tA, tB, tD, a)
                              : cudaLaunchKernelEx(&cfg, gemm_fp8_blockscaled_kernel<8>, tA, tB, tD, a);
    if (e != cudaSuccess) { mfb_host::set_error("gemm_fp8: split-K launch failed: %s", cudaGetErrorString(e)); return 11; }
    return 0;
  }
  int grid = tiles < 148 ? tiles : 148;
  gemm_fp8_blockscaled_kernel<1><<<grid, kF8Threads, SMEM, stream>>>(tA, tB, tD, a);
  if (cudaGetLastError() != cudaSuccess) { mfb_host::set_error("gemm_fp8: launch failed"); return 11; }
  return 0;
}

// x [T, K] bf16 (row pitch ldx) -> q [T, K] e4m3 (row pitch ldq bytes), sa [K/128, sa_ld] fp32
int mfb_quant_act_1x128(const void* x, long long ldx, void* q, long long ldq, float* sa, long long sa_ld, long long T, int K,
                        cudaStream_t stream) {
  if (K % 128 || T <= 0) { mfb_host::set_error("quant_act: K=%d must be a multiple of 128", K); return 1; }
  const int kb = K / 128;
  const long long warps = T * kb;
  const long long blocks = (warps * 32 + 255) / 256;
  quant_act_1x128_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (uint8_t*)q, ldq, sa, sa_ld, T, kb);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
