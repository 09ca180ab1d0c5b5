// bf16 GEMM for a few rows of activations (decode, 1 - 64 tokens): the WEIGHT is the M operand (sm_100a).
//
//   D[t, n] = sum_k X[t, k] * W[n, k]  (+ bias[n])
//
// With a handful of tokens the job is to stream every weight once at HBM speed. The general kernels put 128 token
// rows on the MMA rows: most of their activation tile is padding, a [T, N] problem has only N / 256 tiles (24 for a
// 6144-wide projection on 148 SMs), and the weight bytes in flight per SM are what fits beside the padded
// activations. Here, as in the fp8 decode kernel,
//
//   MMA M = 128 weight rows, N = NT tokens (16, 32 or 64), K = 16 per instruction (kind::f16, fp32 accumulation);
//   a stage is 16 KB of weights (128 rows x 64 k) + NT x 128 B of tokens: 11 / 10 / 8 stages, 128 - 176 KB of
//   weights in flight per SM;
//   one accumulator of NT columns per tile, two in tensor memory so that the epilogue of a tile runs under the
//   products of the next;
//   with fewer tiles than SMs the K range of a tile is split over the KS CTAs (2, 4 or 8) of a thread-block cluster,
//   which reduce-scatter their 128 x NT partials through distributed shared memory (CTA c owns NT / KS token
//   columns) and add them in rank order, so the result does not depend on timing;
//   the result is written transposed, D[token j, n]: the 32 threads of a warp store 32 consecutive n of one token.
//
// Roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2..5 epilogue (one weight row per
// thread). Every wait is bounded; after a timeout the status word is set and the CTA still runs through its cluster
// barriers, frees its tensor memory and exits.
#include "common.cuh"

namespace mfb {
namespace bd {

constexpr int kThreads = 192;
constexpr int kWTile = 128 * 128;          // bytes of a weight stage: 128 rows x 64 bf16

struct Args {
  int T, N, K, kblocks, n_tiles;
  const __nv_bfloat16* bias;      // [N] or null
  __nv_bfloat16* D;
  long long ldd;
  int* status;
};

// OCC = 2: half the stages, so that two CTAs share an SM (used when there are between one and two tiles per SM: all
// of them are then resident at once and share the memory bandwidth evenly, instead of half the SMs doing two rounds).
template <int NT, int OCC>
struct Cfg {
  static constexpr int kStages = OCC == 2 ? (NT == 64 ? 4 : 5) : (NT == 16 ? 11 : (NT == 32 ? 10 : 8));
  static constexpr int kXTile = NT * 128;
  static constexpr int kStageBytes = kWTile + kXTile;
  static constexpr int kTmemCols = 2 * NT < 32 ? 32 : 2 * NT;
  static constexpr int kSmem = kStages * kStageBytes + (2 * kStages + 4) * 8 + 16 + 1024;
};

template <int NT, int KS, int OCC>
__global__ void __launch_bounds__(kThreads, OCC)
gemm_bf16_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                        const Args args) {
  using C = Cfg<NT, OCC>;
  constexpr int STAGES = C::kStages;
  constexpr uint32_t IDESC = umma_idesc_bf16(128, NT, 0, 0);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;       // [2] accumulator complete in tensor memory
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] accumulator read out by the epilogue warps (4 arrivals)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (KS > 1) {
    // split-K launches have exactly one cluster per tile; a cluster without one leaves as a whole
    if (static_cast<int>(blockIdx.x) / KS >= args.n_tiles) return;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&acc_full[s]), 1);
      mbar_init(smem_u32(&acc_empty[s]), 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int krank = KS > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int kb_lo = KS > 1 ? krank * args.kblocks / KS : 0;
  const int kb_hi = KS > 1 ? (krank + 1) * args.kblocks / KS : args.kblocks;
  const int tile0 = KS > 1 ? static_cast<int>(blockIdx.x) / KS : static_cast<int>(blockIdx.x);
  const int tile_step = KS > 1 ? args.n_tiles : static_cast<int>(gridDim.x);   // split-K: one tile per cluster

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = tile0; tile < args.n_tiles && ok; tile += tile_step) {
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, C::kStageBytes);
          const uint32_t w_dst = smem_u32(smem + stage * C::kStageBytes);
          tma_load_2d(w_dst, &tmW, fb, kb * 64, tile * 128);              // rows past N read as zero
          tma_load_2d(w_dst + kWTile, &tmX, fb, kb * 64, 0);              // rows past T read as zero
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
    if constexpr (KS > 1) { cluster_sync_all(); cluster_sync_all(); }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, unit = 0;
      bool ok = true;
      for (int tile = tile0; tile < args.n_tiles && ok; tile += tile_step, ++unit) {
        const int buf = unit & 1;
        ok = mbar_wait(smem_u32(&acc_empty[buf]), ((unit >> 1) & 1) ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t w_base = smem_u32(smem + stage * C::kStageBytes);
          const uint32_t x_base = w_base + kWTile;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem_base + buf * NT, umma_desc_kmajor_sw128(w_base + k * 32),
                        umma_desc_kmajor_sw128(x_base + k * 32), IDESC, (kb > kb_lo || k > 0) ? 1u : 0u);
          umma_commit(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(smem_u32(&acc_full[buf]));
      }
    }
    __syncwarp();
    if constexpr (KS > 1) { cluster_sync_all(); cluster_sync_all(); }
  } else {
    const int ew = warp & 3;                          // warps 2..5 own TMEM lanes 64.., 96.., 0.., 32.. (warp % 4)
    const int row = ew * 32 + lane;                   // weight row of the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    uint32_t unit = 0;
    bool ok = true;
    for (int tile = tile0; tile < args.n_tiles; tile += tile_step, ++unit) {
      const int buf = unit & 1;
      const int n = tile * 128 + row;
      float acc[NT];
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[j] = 0.f;
      if (ok) {
        ok = mbar_wait(smem_u32(&acc_full[buf]), (unit >> 1) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < NT / 16; ++c) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(tmem_base + lane_base + buf * NT + c * 16, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c * 16 + j] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
      }
      const float bias = (args.bias != nullptr && n < args.N) ? __bfloat162float(args.bias[n]) : 0.f;
      if constexpr (KS > 1) {
        // ---- reduce-scatter of the K-slice partials over the cluster: CTA c owns W token columns ----
        constexpr int W = NT / KS;
        static_assert(W >= 4 || KS == 1, "a CTA of the cluster owns at least four token columns");
        ok = named_bar_and(2, 128, ok);
        cluster_sync_all();                           // every CTA of the cluster has drained its operand ring
        if (ok) {
#pragma unroll
          for (int c = 0; c < KS; ++c) {
            const uint32_t dst = mapa_shared(smem_u32(smem) + ((krank * 128 + row) * W) * 4, c);
#pragma unroll
            for (int v = 0; v < W / 4; ++v)
              asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + v * 16),
                           "f"(acc[c * W + 4 * v]), "f"(acc[c * W + 4 * v + 1]), "f"(acc[c * W + 4 * v + 2]),
                           "f"(acc[c * W + 4 * v + 3]) : "memory");
          }
        }
        cluster_sync_all();                           // all slices have landed
        if (ok && n < args.N) {
          float out[W];
#pragma unroll
          for (int i = 0; i < W; ++i) out[i] = 0.f;
          const float4* recv = reinterpret_cast<const float4*>(smem);
#pragma unroll
          for (int r = 0; r < KS; ++r) {
#pragma unroll
            for (int v = 0; v < W / 4; ++v) {
              const float4 x = recv[((r * 128 + row) * W) / 4 + v];
              out[4 * v] += x.x; out[4 * v + 1] += x.y; out[4 * v + 2] += x.z; out[4 * v + 3] += x.w;
            }
          }
#pragma unroll
          for (int j = 0; j < W; ++j) {
            const int t = krank * W + j;
            if (t < args.T) args.D[(long long)t * args.ldd + n] = __float2bfloat16_rn(out[j] + bias);
          }
        }
        break;                                        // one tile per cluster
      } else {
        if (ok && n < args.N) {
#pragma unroll
          for (int j = 0; j < NT; ++j)
            if (j < args.T) args.D[(long long)j * args.ldd + n] = __float2bfloat16_rn(acc[j] + bias);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int NT, int KS, int OCC>
static int launch(const CUtensorMap& tW, const CUtensorMap& tX, const Args& a, int grid, cudaStream_t stream) {
  constexpr int SMEM = Cfg<NT, OCC>::kSmem;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_bf16_decode_kernel<NT, KS, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("gemm_bf16_decode: cannot raise the shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = KS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = KS > 1 ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_bf16_decode_kernel<NT, KS, OCC>, tW, tX, a);
  if (e != cudaSuccess) { mfb_host::set_error("gemm_bf16_decode: launch failed: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

template <int NT>
static int launch_ks(const CUtensorMap& tW, const CUtensorMap& tX, const Args& a, int ks, int occ, cudaStream_t stream) {
  if constexpr (NT >= 32) {
    if (ks == 8) return launch<NT, 8, 1>(tW, tX, a, a.n_tiles * 8, stream);
  }
  if (ks >= 4) return launch<NT, 4, 1>(tW, tX, a, a.n_tiles * 4, stream);
  if (ks == 2) return launch<NT, 2, 1>(tW, tX, a, a.n_tiles * 2, stream);
  if (occ == 2) return launch<NT, 1, 2>(tW, tX, a, a.n_tiles < 296 ? a.n_tiles : 296, stream);
  return launch<NT, 1, 1>(tW, tX, a, a.n_tiles < 148 ? a.n_tiles : 148, stream);
}

}  // namespace bd
}  // namespace mfb

extern "C" {
using namespace mfb;

// 1 when the decode kernel serves D[T, N] = X[T, K] W[N, K]^T: at most 64 rows of X, K a multiple of 8.
int mfb_gemm_bf16_decode_supported(int T, int N, int K) {
  return (T >= 1 && T <= 64 && N >= 1 && K >= 64 && K % 8 == 0) ? 1 : 0;
}

// X [T, K] bf16 (row pitch ldx elements), W [N, K] bf16 (row pitch ldw), D [T, N] bf16 (row pitch ldd), bias [N] or null.
// force_ks > 0 fixes the K split (1, 2, 4, 8) for measurements, force_ks 16 one tile per CTA with two CTAs per SM;
// 0 lets the launcher choose.
int mfb_gemm_bf16_decode(const void* X, const void* W, void* D, const void* bias, int T, int N, int K, long long ldx,
                         long long ldw, long long ldd, int force_ks, int* status, cudaStream_t stream) {
  if (!mfb_gemm_bf16_decode_supported(T, N, K)) {
    mfb_host::set_error("gemm_bf16_decode: T=%d N=%d K=%d not supported", T, N, K);
    return 1;
  }
  const int NT = T <= 16 ? 16 : (T <= 32 ? 32 : 64);
  CUtensorMap tW, tX;
  int rc;
  if ((rc = mfb_host::make_tmap_2d(&tW, W, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, N, K, ldw, 128, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tX, X, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, T, K, ldx, NT, 64))) return 30 + rc;
  bd::Args a;
  a.T = T; a.N = N; a.K = K; a.kblocks = (K + 63) / 64; a.n_tiles = (N + 127) / 128;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.D = reinterpret_cast<__nv_bfloat16*>(D); a.ldd = ldd; a.status = status;
  // Fewer tiles than SMs: split K over a cluster until about two thirds of the SMs stream (each slice keeping at
  // least 8 K blocks). Between one and two tiles per SM: two CTAs per SM, every tile resident at once. More: one
  // persistent CTA per SM, or two if that leaves the last round fuller.
  int ks = 1, occ = 1;
  if (force_ks == 16) {
    occ = 2;
  } else if (force_ks > 0) {
    ks = force_ks;
  } else if (a.n_tiles <= 148) {
    while (ks < 8 && a.n_tiles * ks < 96 && a.n_tiles * ks * 2 <= 148 && a.kblocks / (ks * 2) >= 8 && NT / (ks * 2) >= 4)
      ks *= 2;
  } else if (a.n_tiles <= 296) {
    occ = 2;
  } else {
    const double e1 = (double)a.n_tiles / (double)(((a.n_tiles + 147) / 148) * 148);
    const double e2 = (double)a.n_tiles / (double)(((a.n_tiles + 295) / 296) * 296);
    occ = e2 > e1 + 0.05 ? 2 : 1;
  }
  while (ks > 1 && (NT / ks < 4 || a.kblocks < ks)) ks >>= 1;
  if (NT == 16) return bd::launch_ks<16>(tW, tX, a, ks, occ, stream);
  if (NT == 32) return bd::launch_ks<32>(tW, tX, a, ks, occ, stream);
  return bd::launch_ks<64>(tW, tX, a, ks, occ, stream);
}

}  // extern "C"
