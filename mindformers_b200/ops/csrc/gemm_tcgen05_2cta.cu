// Dense bf16 GEMM on CTA pairs (tcgen05 `cta_group::2`): one 256 x 256 output tile per
// cluster of two CTAs. Each CTA stages its own 128 rows of A and its own 128 rows of B
// (half of the tile's N) per 64-wide K block, so a K block costs 32 KB of shared-memory
// traffic per SM instead of the 48 KB of the single-CTA 128 x 256 tile, and leaves room
// for a deeper TMA ring. The MMA is issued by one thread of the even CTA for both SMs;
// each CTA owns the 128 accumulator rows of its half in its own tensor memory and runs
// its own epilogue.
//
//   D[M,N] = sum_k A(m,k) * B(n,k)      fp32 accumulation, same operand conventions as
//                                        gemm_tcgen05.cu (K-major / MN-major switches)
//
// Tail wave: with 74 clusters a problem of T tiles leaves T mod 74 tiles for a last,
// partly empty wave. When that remainder is at most half of the clusters, those tiles are
// cut along K into `slices` work units each. The units of the leading K ranges write their
// fp32 partial tiles to a workspace and publish a flag; the unit of the last K range adds
// them in its epilogue. Output modes that already reduce-add into D need no workspace.
//
// Synchronisation between the two CTAs of a pair:
//   full[s]    on the even CTA only: both producers' TMA loads complete_tx on it
//   empty[s]   in both CTAs, signalled together by a multicast tcgen05.commit
//   tfull[a]   in both CTAs (accumulator a complete), multicast commit
//   tempty[a]  on the even CTA: 8 arrivals (4 epilogue warps of each CTA)
// No TMA load uses cluster multicast: every CTA fetches its own operand halves.
#include "common.cuh"

namespace mfb {
namespace pair {

constexpr int kHalfM = 128;   // rows of A / D per CTA
constexpr int kHalfN = 128;   // rows of B per CTA (the MMA sees N = 256)
constexpr int kTileM = 256;
constexpr int kTileN = 256;
constexpr int kBK = 64;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kStagingBytes = 128 * 128;
constexpr int kMaxSlices = 4;

struct Args {
  int M, N, K;
  int num_m_tiles, num_n_tiles;
  int full_tiles;     // tiles processed whole
  int split_tiles;    // tiles cut into `slices` K ranges (the last ones in tile order)
  int slices;
  float* partials;    // [split_tiles][slices-1][2 CTAs][256 cols][128 rows] fp32
  int* flags;         // [split_tiles][slices-1][2 CTAs]
  int* status;
  int band;           // tile rows per raster band (see get_unit)
};

struct Unit {
  int m0, n0;         // first row / column of the 256 x 256 tile
  int kb0, kbn;       // K block range
  int role;           // 0 whole tile, 1 partial producer, 2 partial consumer
  int slot;           // split tile index
  int slice;
};

__device__ __forceinline__ Unit get_unit(const Args& g, int u) {
  Unit w;
  const int kb_total = (g.K + kBK - 1) / kBK;
  int tile;
  if (u < g.full_tiles) {
    tile = u;
    w.role = 0;
    w.slot = 0;
    w.slice = 0;
    w.kb0 = 0;
    w.kbn = kb_total;
  } else {
    const int j = u - g.full_tiles;
    w.slot = j % g.split_tiles;
    w.slice = j / g.split_tiles;
    tile = g.full_tiles + w.slot;
    w.kb0 = static_cast<int>((static_cast<long long>(kb_total) * w.slice) / g.slices);
    const int kb1 = static_cast<int>((static_cast<long long>(kb_total) * (w.slice + 1)) / g.slices);
    w.kbn = kb1 - w.kb0;
    w.role = (w.slice == g.slices - 1) ? 2 : 1;
  }
  // banded rasterisation: the tile rows of a band share their B tiles through L2, and the band's A rows stay resident
  // while the walk crosses all columns, so B is streamed from HBM once per band. The launcher picks the band as tall as
  // keeps the band's rows of A (band x 256 x K bf16) within a third of L2.
  const int kBand = g.band;
  const int tiles_per_band = kBand * g.num_n_tiles;
  const int band = tile / tiles_per_band;
  const int first_m = band * kBand;
  const int band_h = (g.num_m_tiles - first_m) < kBand ? (g.num_m_tiles - first_m) : kBand;
  const int r = tile - band * tiles_per_band;
  w.m0 = (first_m + r % band_h) * kTileM;
  w.n0 = (r / band_h) * kTileN;
  return w;
}

__device__ __forceinline__ int total_units(const Args& g) {
  return g.full_tiles + g.split_tiles * g.slices;
}

// OUT_MODE: 0 bf16 store, 1 f32 store, 2 f32 reduce-add, 3 bf16 reduce-add
template <int STAGES, bool A_MN, bool B_MN, int OUT_MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmD, const Args args) {
  constexpr int A_BYTES = kHalfM * kBK * 2;
  constexpr int B_BYTES = kHalfN * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * kTileN;
  constexpr bool OUT_F32 = (OUT_MODE == 1 || OUT_MODE == 2);
  constexpr bool OUT_REDUCE = (OUT_MODE >= 2);
  constexpr int CHUNK_COLS = OUT_F32 ? 32 : 64;
  constexpr int NUM_CHUNKS = kTileN / CHUNK_COLS;
  constexpr uint32_t IDESC = umma_idesc_bf16(kTileM, kTileN, A_MN ? 1 : 0, B_MN ? 1 : 0);

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
  const uint32_t cta = cluster_ctarank();     // 0 = even CTA (issues the MMAs), 1 = its peer
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tfull_bar[s]), 1);
      mbar_init(smem_u32(&tempty_bar[s]), 8);  // four epilogue warps in each CTA of the pair
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_holder), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int n_units = total_units(args);

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = cluster_id; u < n_units && ok; u += num_clusters) {
        const Unit w = get_unit(args, u);
        const int a_mn0 = w.m0 + static_cast<int>(cta) * kHalfM;
        const int b_mn0 = w.n0 + static_cast<int>(cta) * kHalfN;
        for (int kb = 0; kb < w.kbn; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, args.status,
                         kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb_local = smem_u32(&full_bar[stage]);
          const uint32_t fb = mapa_shared(fb_local, 0);
          if (cta == 0) mbar_expect_tx(fb_local, 2 * STAGE_BYTES);  // the bytes of both CTAs
          const uint32_t a_dst = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_BYTES;
          const int k0 = (w.kb0 + kb) * kBK;
          if (A_MN) {
#pragma unroll
            for (int at = 0; at < kHalfM / 64; ++at)
              tma_load_2d_pair(a_dst + at * (kBK * 128), &tmA, fb, a_mn0 + at * 64, k0);
          } else {
            tma_load_2d_pair(a_dst, &tmA, fb, k0, a_mn0);
          }
          if (B_MN) {
#pragma unroll
            for (int at = 0; at < kHalfN / 64; ++at)
              tma_load_2d_pair(b_dst + at * (kBK * 128), &tmB, fb, b_mn0 + at * 64, k0);
          } else {
            tma_load_2d_pair(b_dst, &tmB, fb, k0, b_mn0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ------------------------------
    if (lane == 0 && cta == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int u = cluster_id; u < n_units && ok; u += num_clusters) {
        const Unit w = get_unit(args, u);
        if (w.kbn == 0) continue;
        ok = mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, args.status,
                       kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kTileN;
        for (int kb = 0; kb < w.kbn; ++kb) {
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
            umma_f16_ss_pair(d_tmem, a_desc, b_desc, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(smem_u32(&empty_bar[stage]));  // frees the stage in both CTAs
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&tfull_bar[acc]));      // accumulator complete in both CTAs
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue (both CTAs, 128 rows each) ------------------------------
    const int ew = warp & 3;
    const int row = ew * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    const uint32_t tempty_leader0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = mapa_shared(smem_u32(&tempty_bar[1]), 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t chunk_counter = 0;
    bool ok = true;
    for (int u = cluster_id; u < n_units && ok; u += num_clusters) {
      const Unit w = get_unit(args, u);
      const bool have_acc = (w.kbn > 0);
      if (have_acc) {
        ok = mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, args.status,
                       kStatusWaitTimeoutEpilogue);
      }
      ok = named_bar_and(2, kEpiThreads, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * kTileN;
      const int d_row = w.m0 + static_cast<int>(cta) * kHalfM;
      const int role = OUT_REDUCE ? 0 : w.role;

      if (role == 1) {
        // leading K range of a split tile: publish the fp32 partial, column-major so that the 32
        // lanes of a warp write 32 consecutive rows of one column
        float* dst = args.partials +
                     ((static_cast<size_t>(w.slot) * (args.slices - 1) + w.slice) * 2 + cta) *
                         (static_cast<size_t>(kTileN) * kHalfM);
#pragma unroll 1
        for (int c = 0; c < kTileN / 32; ++c) {
          uint32_t v[32];
          if (have_acc) {
            tmem_ld_32x32b_x32(t_addr + c * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[(c * 32 + i) * kHalfM + row] = __uint_as_float(v[i]);
        }
        __threadfence();
        named_bar_sync(1, kEpiThreads);
        if (issuer) {
          int* flag = args.flags + (static_cast<size_t>(w.slot) * (args.slices - 1) + w.slice) * 2 + cta;
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
        }
      } else {
        if (role == 2) {
          // last K range: the partials of the leading ranges must have landed
          if (issuer) {
            for (int s = 0; s < args.slices - 1 && ok; ++s) {
              int* flag = args.flags + (static_cast<size_t>(w.slot) * (args.slices - 1) + s) * 2 + cta;
              const uint64_t t0 = globaltimer_ns();
              int seen = 0;
              uint32_t it = 0;
              while (true) {
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
                if (seen != 0) break;
                if (((++it) & 0x3f) == 0) {
                  if (*abort_flag || globaltimer_ns() - t0 > MFB_WAIT_LIMIT_NS) {
                    *abort_flag = 1;
                    if (args.status) atomicCAS(args.status, 0, kStatusWaitTimeoutEpilogue);
                    ok = false;
                    break;
                  }
                }
              }
            }
          }
          ok = named_bar_and(2, kEpiThreads, ok);
          if (!ok) break;
        }
#pragma unroll 1
        for (int c = 0; c < NUM_CHUNKS; ++c) {
          uint32_t packed[32];
          if (OUT_F32) {
            if (have_acc) {
              tmem_ld_32x32b_x32(t_addr + c * 32, packed);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) packed[i] = 0;
            }
            if (role == 2) {
              for (int s = 0; s < args.slices - 1; ++s) {
                const float* src = args.partials +
                                   ((static_cast<size_t>(w.slot) * (args.slices - 1) + s) * 2 + cta) *
                                       (static_cast<size_t>(kTileN) * kHalfM);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  packed[i] = __float_as_uint(__uint_as_float(packed[i]) +
                                              __ldcg(src + (c * 32 + i) * kHalfM + row));
              }
            }
          } else {
            uint32_t v0[32], v1[32];
            if (have_acc) {
              tmem_ld_32x32b_x32(t_addr + c * 64, v0);
              tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) { v0[i] = 0; v1[i] = 0; }
            }
            if (role == 2) {
              for (int s = 0; s < args.slices - 1; ++s) {
                const float* src = args.partials +
                                   ((static_cast<size_t>(w.slot) * (args.slices - 1) + s) * 2 + cta) *
                                       (static_cast<size_t>(kTileN) * kHalfM);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  v0[i] = __float_as_uint(__uint_as_float(v0[i]) +
                                          __ldcg(src + (c * 64 + i) * kHalfM + row));
                  v1[i] = __float_as_uint(__uint_as_float(v1[i]) +
                                          __ldcg(src + (c * 64 + 32 + i) * kHalfM + row));
                }
              }
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              packed[i] = pack_bf16x2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1]));
              packed[16 + i] = pack_bf16x2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1]));
            }
          }
          const int buf = chunk_counter & 1;
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
            const int x = w.n0 + c * CHUNK_COLS;
            if (x < args.N && d_row < args.M) {
              const uint32_t src = smem_u32(staging + buf * kStagingBytes);
              if (OUT_REDUCE) tma_reduce_add_2d(&tmD, src, x, d_row);
              else tma_store_2d(&tmD, src, x, d_row);
            }
            tma_commit_group();
          }
          ++chunk_counter;
        }
        if (role == 2) {
          // the partials are consumed: re-arm the flags for the next launch
          named_bar_sync(1, kEpiThreads);
          if (issuer) {
            for (int s = 0; s < args.slices - 1; ++s)
              args.flags[(static_cast<size_t>(w.slot) * (args.slices - 1) + s) * 2 + cta] = 0;
          }
        }
      }
      if (have_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc == 0 ? tempty_leader0 : tempty_leader1);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    if (issuer) tma_wait_group<0>();
  }

  // both CTAs are done with tensor memory and with each other's barriers before either leaves
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace pair
}  // namespace mfb

// ---------------------------------------------------------------------------------------
// host launcher
// ---------------------------------------------------------------------------------------
namespace {

using namespace mfb;
using namespace mfb::pair;

int pair_num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

template <int STAGES, bool A_MN, bool B_MN, int OUT_MODE>
int launch_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tD, const Args& args,
                int clusters, cudaStream_t stream) {
  constexpr int STAGE_BYTES = (kHalfM + kHalfN) * kBK * 2;
  constexpr int SMEM = STAGES * STAGE_BYTES + 2 * kStagingBytes + (2 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(SMEM <= 232448, "shared memory budget exceeded");
  auto kern = gemm_bf16_pair_kernel<STAGES, A_MN, B_MN, OUT_MODE>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) {
      mfb_host::set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return 10;
    }
    attr_set = true;
  }
  kern<<<2 * clusters, kThreads, SMEM, stream>>>(tA, tB, tD, args);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    mfb_host::set_error("gemm pair launch: %s", cudaGetErrorString(e));
    return 11;
  }
  return 0;
}

int dispatch_pair(int a_mn, int b_mn, int out_mode, const CUtensorMap& tA, const CUtensorMap& tB,
                  const CUtensorMap& tD, const Args& args, int clusters, cudaStream_t stream) {
#define MFB_PAIR_CASE(AM, BMJ, OM)                                                   \
  if (a_mn == AM && b_mn == BMJ && out_mode == OM)                                   \
    return launch_pair<6, AM != 0, BMJ != 0, OM>(tA, tB, tD, args, clusters, stream);
  MFB_PAIR_CASE(0, 0, 0)
  MFB_PAIR_CASE(0, 0, 1)
  MFB_PAIR_CASE(0, 0, 2)
  MFB_PAIR_CASE(0, 1, 0)
  MFB_PAIR_CASE(0, 1, 1)
  MFB_PAIR_CASE(1, 1, 0)
  MFB_PAIR_CASE(1, 1, 1)
  MFB_PAIR_CASE(1, 1, 2)
  MFB_PAIR_CASE(1, 1, 3)
  MFB_PAIR_CASE(1, 0, 0)
#undef MFB_PAIR_CASE
  mfb_host::set_error("gemm pair: unsupported combination a_mn=%d b_mn=%d out_mode=%d", a_mn, b_mn, out_mode);
  return 12;
}

}  // namespace

namespace {
int g_pair_band = 0;
}

extern "C" {

// Raster band of the CTA-pair GEMM in tile rows: 0 = chosen from K (see the launcher), > 0 = fixed (for benchmarks).
void mfb_gemm_pair_set_band(int band) { g_pair_band = band; }


// Bytes of workspace `mfb_gemm_bf16_pair` may use for the split tail wave (partials, then flags).
// The caller allocates it once, zero-filled, and passes the same buffer to every call on one stream;
// calls that overlap on the GPU need buffers of their own.
long long mfb_gemm_pair_workspace_bytes() {
  const long long max_split = 74 / 2;  // at most half of the clusters hold split tiles
  const long long partial = static_cast<long long>(max_split) * (kMaxSlices - 1) * 2 * kTileN * kHalfM * 4;
  const long long flags = max_split * (kMaxSlices - 1) * 2 * 4;
  return partial + ((flags + 255) / 256) * 256;
}

// Plan of the tail-wave split for a problem: returns the number of K slices (1 = no split) and, through
// the pointers, the number of whole and split tiles. `max_slices` <= 1 turns the split off.
int mfb_gemm_pair_plan(int M, int N, int K, int clusters, int max_slices, int* full_tiles, int* split_tiles) {
  const int tiles = ((M + kTileM - 1) / kTileM) * ((N + kTileN - 1) / kTileN);
  const int kb = (K + kBK - 1) / kBK;
  int rem = tiles % clusters;
  int slices = 1;
  // beyond a few dozen waves the last one is a small share of the run time and the split only adds traffic
  if (max_slices > 1 && rem > 0 && 2 * rem <= clusters && tiles / clusters < 40) {
    slices = clusters / rem;
    if (slices > max_slices) slices = max_slices;
    if (slices > kMaxSlices) slices = kMaxSlices;
    while (slices > 1 && kb / slices < 8) --slices;   // keep at least 8 K blocks per slice
  }
  if (slices <= 1) { slices = 1; rem = 0; }
  if (full_tiles) *full_tiles = tiles - rem;
  if (split_tiles) *split_tiles = rem;
  return slices;
}

// Dense bf16 GEMM on CTA pairs; operand conventions and `out_mode` as in `mfb_gemm_bf16` (mode 0).
// `workspace` (see `mfb_gemm_pair_workspace_bytes`) may be null: the tail wave is then not split.
// `sm_limit` > 0 restricts the persistent grid to that many SMs (rounded down to whole pairs).
int mfb_gemm_bf16_pair(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd,
                       int a_mn_major, int b_mn_major, int out_mode, void* workspace, int max_slices,
                       int* status, int sm_limit, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) {
    mfb_host::set_error("gemm pair: bad shape M=%d N=%d K=%d", M, N, K);
    return 1;
  }
  const bool out_f32 = (out_mode == 1 || out_mode == 2);
  CUtensorMap tA, tB, tD;
  int rc = 0;
  const uint64_t a_rows = a_mn_major ? K : M, a_cols = a_mn_major ? M : K;
  const uint64_t b_rows = b_mn_major ? K : N, b_cols = b_mn_major ? N : K;
  if (a_mn_major) rc = mfb_host::make_tmap_2d(&tA, A, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a_rows, a_cols, lda, kBK, 64);
  else            rc = mfb_host::make_tmap_2d(&tA, A, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a_rows, a_cols, lda, kHalfM, kBK);
  if (rc) return 20 + rc;
  if (b_mn_major) rc = mfb_host::make_tmap_2d(&tB, B, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b_rows, b_cols, ldb, kBK, 64);
  else            rc = mfb_host::make_tmap_2d(&tB, B, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b_rows, b_cols, ldb, kHalfN, kBK);
  if (rc) return 30 + rc;
  if (out_f32) rc = mfb_host::make_tmap_2d(&tD, D, 4, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, M, N, ldd, kHalfM, 32);
  else         rc = mfb_host::make_tmap_2d(&tD, D, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, M, N, ldd, kHalfM, 64);
  if (rc) return 40 + rc;

  int sms = pair_num_sms();
  if (sm_limit > 0 && sm_limit < sms) sms = sm_limit;
  int clusters = sms / 2;
  if (clusters < 1) clusters = 1;

  Args args;
  args.M = M; args.N = N; args.K = K;
  args.num_m_tiles = (M + kTileM - 1) / kTileM;
  args.num_n_tiles = (N + kTileN - 1) / kTileN;
  const int tiles = args.num_m_tiles * args.num_n_tiles;
  if (tiles < clusters) clusters = tiles;
  const bool reduce_out = (out_mode >= 2);
  args.slices = mfb_gemm_pair_plan(M, N, K, clusters, (workspace || reduce_out) ? max_slices : 1,
                                   &args.full_tiles, &args.split_tiles);
  if (args.split_tiles > 74 / 2 && !reduce_out) {   // beyond what the workspace was sized for
    args.slices = 1; args.full_tiles = tiles; args.split_tiles = 0;
  }
  const long long partial_bytes = static_cast<long long>(74 / 2) * (kMaxSlices - 1) * 2 * kTileN * kHalfM * 4;
  args.partials = reinterpret_cast<float*>(workspace);
  args.flags = workspace ? reinterpret_cast<int*>(reinterpret_cast<char*>(workspace) + partial_bytes) : nullptr;
  args.status = status;
  {
    // 16 tile rows per band while the band's rows of A stay near 32 MB (K <= 4096), else 8. Measured under the power
    // cap at 8192 x 28672 x 4096: 1337 / 1372 / 1266 TFLOP/s for bands of 8 / 16 / 32 (cuBLAS 1366); at K = 14336 a
    // band of 8 is best. `g_pair_band` > 0 overrides the choice (benchmarks).
    long long band = (K <= 4096) ? 16 : 8;
    if (g_pair_band > 0) band = g_pair_band;
    if (band > args.num_m_tiles) band = args.num_m_tiles;
    args.band = static_cast<int>(band);
  }
  return dispatch_pair(a_mn_major, b_mn_major, out_mode, tA, tB, tD, args, clusters, stream);
}

}  // extern "C"
