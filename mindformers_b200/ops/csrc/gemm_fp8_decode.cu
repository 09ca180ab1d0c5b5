// Block-scaled fp8 (e4m3) GEMM for a few tokens per weight tile (decode): the WEIGHT is the M operand.
//
//   D[t, n] = sum_kb  sa[kb, t] * sb[g, n / 128, kb] * sum_{k in block kb} X[t, k] * W[g * N + n, k]
//
// Same operands and scales as gemm_fp8.cu. That kernel puts 128 token rows on the MMA rows; with 1 - 64 tokens most
// of its activation tile is padding, its stage carries 16 KB of it next to 16 KB of weights, and its epilogue does
// 128 multiply-adds per thread and K block whatever the number of tokens. At these sizes the job is to stream the
// weight once at HBM speed, so here
//
//   MMA M = 128 weight rows, N = NT tokens (32 or 64), K = 32 per instruction (kind::f8f6f4);
//   a stage is 16 KB of weights + NT x 128 B of tokens: 9 stages (NT = 32) or 7 (NT = 64) fit, i.e. 112 - 144 KB
//   of weights in flight per SM instead of 80 KB;
//   the TMEM partial of a K block is 128 lanes x NT columns; an epilogue thread owns one weight row and does NT
//   multiply-adds per K block: acc[j] += partial[j] * (sa[kb, token j] * sb[kb]);
//   256 / NT partials are in flight (4 or 8): the chain MMA -> commit -> epilogue wakes -> TMEM load -> arrive ->
//   MMA thread wakes is a few thousand cycles long, and with two partials it, not HBM, set the time per K block;
//   the scales of a unit (sa of its NT tokens and sb of its weight tile, for every K block) are staged in shared
//   memory once per unit: fetched from global memory per K block, their latency was the time per K block;
//   the result is written transposed, D[token j, n]: the 32 threads of a warp store 32 consecutive n of one token.
//
// mode 0 (dense): tiles = (N / 128) x ceil(T / NT); with few tiles the K range of a tile is split over the KS CTAs of a
// thread-block cluster, which reduce-scatter their 128 x NT partials through distributed shared memory (CTA c owns
// NT / KS token columns) and add them in rank order.
// mode 1 (grouped, MoE experts): rows of X are expert segments padded to 128-row blocks; `seg_fill` / `group_offsets`
// give the rows in use, and a work item (row block, weight tile) walks the token sub-blocks of NT rows that hold any.
// With one to three tokens per expert that is one pass over every expert's weights with 4 KB of tokens per stage.
#include <cuda_fp8.h>

#include "common.cuh"

namespace mfb {

constexpr int kFdThreads = 192;
constexpr int kFdWTile = 128 * 128;       // weight tile of a stage: 128 rows x 128 k (bytes)
constexpr int kFdMaxKb = 144;             // K blocks per CTA whose scales are staged in shared memory (K <= 18432)

struct FdArgs {
  int T, N, K, kblocks, num_n_blocks;
  int mode, num_groups;
  long long sa_ld;
  const float* sa;               // [K/128, sa_ld]
  const float* sb;               // [G, N/128, K/128]
  const int* m_block_group;      // grouped: expert of every 128-row block
  const int* num_m_blocks_dev;   // grouped: row blocks in use
  const int* group_offsets;      // grouped: [G + 1] first row of every expert segment
  const int* seg_fill;           // grouped: [G] rows in use per segment
  int num_m_blocks;              // grouped: upper bound of row blocks
  __nv_bfloat16* D;
  long long ldd;
  int* status;
};

__device__ __forceinline__ void fd_umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ uint32_t fd_cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t fd_mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void fd_st_cluster_v4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void fd_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One unit of work: 128 weight rows x up to NT tokens over K blocks [kb_lo, kb_hi).
struct FdUnit {
  int w_row;      // first row of the weight tile in [G * N, K]
  int tok0;       // first token row
  int ntok;       // tokens in use (<= NT)
  int n0;         // first output column
  int sb_off;     // offset of the tile's weight scales in sb
};

// Enumerates the units of this CTA in the same order for every role.
template <int NT, int KS>
struct FdWalker {
  const FdArgs& a;
  int item, item_step, n_items, mb_total;
  int tb, n_tb, m_blk, n_blk, grp, fill;
  __device__ FdWalker(const FdArgs& args) : a(args) {
    if (a.mode == 0) {
      n_items = a.num_n_blocks * ((a.T + NT - 1) / NT);
      mb_total = 0;
    } else {
      mb_total = a.num_m_blocks;
      if (a.num_m_blocks_dev) {
        const int v = *a.num_m_blocks_dev;
        mb_total = v < mb_total ? v : mb_total;
      }
      n_items = mb_total * a.num_n_blocks;
    }
    item = KS > 1 ? static_cast<int>(blockIdx.x) / KS : static_cast<int>(blockIdx.x);
    item_step = KS > 1 ? n_items : static_cast<int>(gridDim.x);
    tb = 0;
    n_tb = 0;
    load_item();
  }
  __device__ void load_item() {
    // skips items without tokens (grouped: a row block past the end of its segment's rows)
    while (item < n_items) {
      if (a.mode == 0) {
        n_blk = item % a.num_n_blocks;
        m_blk = item / a.num_n_blocks;      // token block
        grp = 0;
        fill = a.T - m_blk * NT;
        if (fill > NT) fill = NT;
        n_tb = 1;
      } else {
        m_blk = item % mb_total;
        n_blk = item / mb_total;
        grp = a.m_block_group[m_blk];
        fill = a.seg_fill[grp] - (m_blk * 128 - a.group_offsets[grp]);
        if (fill > 128) fill = 128;
        n_tb = fill > 0 ? (fill + NT - 1) / NT : 0;
      }
      tb = 0;
      if (n_tb > 0) return;
      item += item_step;
    }
  }
  __device__ bool valid() const { return item < n_items; }
  __device__ FdUnit unit() const {
    FdUnit u;
    u.w_row = grp * a.N + n_blk * 128;
    u.n0 = n_blk * 128;
    u.sb_off = (grp * a.num_n_blocks + n_blk) * a.kblocks;
    if (a.mode == 0) {
      u.tok0 = m_blk * NT;
      u.ntok = fill;
    } else {
      u.tok0 = m_blk * 128 + tb * NT;
      u.ntok = fill - tb * NT < NT ? fill - tb * NT : NT;
    }
    return u;
  }
  __device__ void next() {
    if (++tb < n_tb) return;
    item += item_step;
    load_item();
  }
};

template <int NT, int KS>
__global__ void __launch_bounds__(kFdThreads, 1)
gemm_fp8_decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const FdArgs args) {
  constexpr int STAGES = NT == 32 ? 9 : 7;
  constexpr int XTILE = NT * 128;
  constexpr int STAGE_BYTES = kFdWTile + XTILE;
  constexpr int NBUF = 256 / NT;                // partials in flight in tensor memory
  constexpr uint32_t IDESC = umma_idesc_e4m3(128, NT);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* pfull = bars + 2 * STAGES;          // [NBUF] partial of a K block complete in tensor memory
  uint64_t* pempty = bars + 2 * STAGES + NBUF;  // [NBUF] partial drained by the epilogue warps (4 arrivals)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * NBUF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float4* s_sa = reinterpret_cast<float4*>(tmem_holder + 4);         // [kFdMaxKb][NT / 4] token scales of the unit
  float* s_sb = reinterpret_cast<float*>(s_sa + kFdMaxKb * (NT / 4));  // [kFdMaxKb] weight scales of the unit
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (KS > 1) {
    // split-K launches have exactly one cluster per tile; a cluster without one leaves as a whole
    const int n_items = args.num_n_blocks * ((args.T + NT - 1) / NT);
    if (static_cast<int>(blockIdx.x) / KS >= n_items) return;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < NBUF; ++s) {
      mbar_init(smem_u32(&pfull[s]), 1);
      mbar_init(smem_u32(&pempty[s]), 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  constexpr int TMEM_COLS = NBUF * NT;
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int krank = KS > 1 ? static_cast<int>(fd_cluster_ctarank()) : 0;
  const int kb_lo = KS > 1 ? krank * args.kblocks / KS : 0;
  const int kb_hi = KS > 1 ? (krank + 1) * args.kblocks / KS : args.kblocks;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (FdWalker<NT, KS> w(args); w.valid() && ok; w.next()) {
        const FdUnit u = w.unit();
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, STAGE_BYTES);
          const uint32_t w_dst = smem_u32(smem + stage * STAGE_BYTES);
          tma_load_2d(w_dst, &tmW, fb, kb * 128, u.w_row);
          tma_load_2d(w_dst + kFdWTile, &tmX, fb, kb * 128, u.tok0);     // rows past T read as zero
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
    if constexpr (KS > 1) { fd_cluster_sync(); fd_cluster_sync(); }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t blk = 0;
      bool ok = true;
      for (FdWalker<NT, KS> w(args); w.valid() && ok; w.next()) {
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++blk) {
          const int buf = blk % NBUF;
          ok = mbar_wait(smem_u32(&pempty[buf]), ((blk / NBUF) & 1) ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t w_base = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t x_base = w_base + kFdWTile;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            fd_umma(tmem_base + buf * NT, umma_desc_kmajor_sw128(w_base + k * 32), umma_desc_kmajor_sw128(x_base + k * 32),
                    IDESC, k > 0 ? 1u : 0u);
          umma_commit(smem_u32(&empty_bar[stage]));
          umma_commit(smem_u32(&pfull[buf]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
    if constexpr (KS > 1) { fd_cluster_sync(); fd_cluster_sync(); }
  } else {
    const int ew = warp & 3;
    const int row = ew * 32 + lane;                   // weight row of the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    uint32_t blk = 0;
    bool ok = true;
    for (FdWalker<NT, KS> w(args); w.valid() && ok; w.next()) {
      const FdUnit u = w.unit();
      const float* sb = args.sb + u.sb_off;
      const float* sa = args.sa + u.tok0;             // token scales of K block kb: sa[kb * sa_ld + j]
      // stage the scales of this unit (the previous unit's reads are over after the barrier)
      named_bar_sync(1, 128);
      {
        const int tid = threadIdx.x - 64, nkb = kb_hi - kb_lo;
        for (int i = tid; i < nkb * (NT / 4); i += 128) {
          const int kb = i / (NT / 4), q = i - kb * (NT / 4);
          s_sa[i] = __ldg(reinterpret_cast<const float4*>(sa + (long long)(kb_lo + kb) * args.sa_ld) + q);
        }
        for (int i = tid; i < nkb; i += 128) s_sb[i] = sb[kb_lo + i];
      }
      named_bar_sync(1, 128);
      float acc[NT];
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[j] = 0.f;
      for (int kb = kb_lo; kb < kb_hi; ++kb, ++blk) {
        const int buf = blk % NBUF;
        const float sbw = s_sb[kb - kb_lo];
        const float4* st = s_sa + (kb - kb_lo) * (NT / 4);
        ok = mbar_wait(smem_u32(&pfull[buf]), (blk / NBUF) & 1, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < NT / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_base + buf * NT + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 s4 = st[c * 8 + q];
            acc[c * 32 + 4 * q] = fmaf(__uint_as_float(r[4 * q]), s4.x * sbw, acc[c * 32 + 4 * q]);
            acc[c * 32 + 4 * q + 1] = fmaf(__uint_as_float(r[4 * q + 1]), s4.y * sbw, acc[c * 32 + 4 * q + 1]);
            acc[c * 32 + 4 * q + 2] = fmaf(__uint_as_float(r[4 * q + 2]), s4.z * sbw, acc[c * 32 + 4 * q + 2]);
            acc[c * 32 + 4 * q + 3] = fmaf(__uint_as_float(r[4 * q + 3]), s4.w * sbw, acc[c * 32 + 4 * q + 3]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&pempty[buf]));
      }
      if constexpr (KS > 1) {
        // ---- reduce-scatter of the K-slice partials over the cluster: CTA c owns W token columns ----
        constexpr int W = NT / KS;
        ok = named_bar_and(2, 128, ok);
        fd_cluster_sync();                            // every CTA of the cluster has drained its operand ring
        if (ok) {
#pragma unroll
          for (int c = 0; c < KS; ++c) {
            const uint32_t dst = fd_mapa(smem_u32(smem) + ((krank * 128 + row) * W) * 4, c);
#pragma unroll
            for (int v = 0; v < W / 4; ++v)
              fd_st_cluster_v4(dst + v * 16, acc[c * W + 4 * v], acc[c * W + 4 * v + 1], acc[c * W + 4 * v + 2],
                               acc[c * W + 4 * v + 3]);
          }
        }
        fd_cluster_sync();                            // all slices have landed
        if (ok) {
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
            if (t < u.ntok) args.D[(long long)(u.tok0 + t) * args.ldd + u.n0 + row] = __float2bfloat16_rn(out[j]);
          }
        }
        break;                                        // one tile per cluster
      }
      ok = named_bar_and(2, 128, ok);                 // the four warps go on to the next unit together or not at all
      if (!ok) break;
#pragma unroll
      for (int j = 0; j < NT; ++j)
        if (j < u.ntok) args.D[(long long)(u.tok0 + j) * args.ldd + u.n0 + row] = __float2bfloat16_rn(acc[j]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int NT, int KS>
static int fd_launch(const CUtensorMap& tW, const CUtensorMap& tX, const FdArgs& a, int grid, cudaStream_t stream) {
  constexpr int STAGES = NT == 32 ? 9 : 7;
  constexpr int SMEM = STAGES * (kFdWTile + NT * 128) + (2 * STAGES + 2 * (256 / NT)) * 8 + 16 + kFdMaxKb * (NT + 1) * 4 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_fp8_decode_kernel<NT, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("gemm_fp8_decode: cannot raise the shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFdThreads);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = KS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = KS > 1 ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_fp8_decode_kernel<NT, KS>, tW, tX, a);
  if (e != cudaSuccess) { mfb_host::set_error("gemm_fp8_decode: launch failed: %s", cudaGetErrorString(e)); return 11; }
  return 0;
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// 1 when the decode kernel serves this call: dense with at most 64 tokens, or grouped with the segment fill known
// on the device. N and K must be multiples of 128.
int mfb_gemm_fp8_decode_supported(int T, int N, int K, int mode) {
  if (N % 128 || K % 128 || T <= 0 || K / 128 > kFdMaxKb) return 0;
  return mode == 1 ? 1 : (T <= 64 ? 1 : 0);
}

// X [T, K] e4m3 (row pitch ldx bytes), W [G * N, K] e4m3 (row pitch ldw), D [T, N] bf16 (row pitch ldd elements).
// mode 1: m_block_group / num_m_blocks_dev / group_offsets / seg_fill as produced by the expert plan; T is the row
// bound of X (a multiple of 128).
int mfb_gemm_fp8_decode(const void* X, const void* W, void* D, const float* sa, long long sa_ld, const float* sb, int T,
                        int N, int K, long long ldx, long long ldw, long long ldd, int mode, int num_groups,
                        const int* m_block_group, const int* num_m_blocks_dev, const int* group_offsets,
                        const int* seg_fill, int* status, cudaStream_t stream) {
  if (!mfb_gemm_fp8_decode_supported(T, N, K, mode) || (sa_ld % 4) || (reinterpret_cast<uintptr_t>(sa) & 15)) {
    mfb_host::set_error("gemm_fp8_decode: T=%d N=%d K=%d mode=%d sa_ld=%lld not supported", T, N, K, mode, sa_ld);
    return 1;
  }
  if (mode == 1 && (T % 128 || !m_block_group || !group_offsets || !seg_fill)) {
    mfb_host::set_error("gemm_fp8_decode grouped: rows %d must be a multiple of 128 and the plan arrays are required", T);
    return 1;
  }
  const int G = mode == 1 ? num_groups : 1;
  const int NT = (mode == 1 || T <= 32) ? 32 : 64;
  CUtensorMap tW, tX;
  int rc;
  if ((rc = mfb_host::make_tmap_2d(&tW, W, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint64_t)G * N, K, ldw, 128, 128))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tX, X, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, T, K, ldx, NT, 128))) return 30 + rc;
  FdArgs a;
  a.T = T; a.N = N; a.K = K; a.kblocks = K / 128; a.num_n_blocks = N / 128; a.mode = mode; a.num_groups = G;
  a.sa_ld = sa_ld; a.sa = sa; a.sb = sb; a.m_block_group = m_block_group; a.num_m_blocks_dev = num_m_blocks_dev;
  a.group_offsets = group_offsets; a.seg_fill = seg_fill; a.num_m_blocks = T / 128;
  a.D = reinterpret_cast<__nv_bfloat16*>(D); a.ldd = ldd; a.status = status;
  if (mode == 1) {
    const int items = a.num_m_blocks * a.num_n_blocks;
    return fd_launch<32, 1>(tW, tX, a, items < 148 ? items : 148, stream);
  }
  const int tiles = a.num_n_blocks;            // T <= 64: one token block
  int ks = 1;
  if (tiles * 8 <= 128 && a.kblocks >= 16) ks = 8;
  else if (tiles * 4 <= 144 && a.kblocks >= 8) ks = 4;
  else if (tiles * 2 <= 148 && a.kblocks >= 4) ks = 2;
  if (NT == 32) {
    if (ks == 8) return fd_launch<32, 8>(tW, tX, a, tiles * 8, stream);
    if (ks == 4) return fd_launch<32, 4>(tW, tX, a, tiles * 4, stream);
    if (ks == 2) return fd_launch<32, 2>(tW, tX, a, tiles * 2, stream);
    return fd_launch<32, 1>(tW, tX, a, tiles < 148 ? tiles : 148, stream);
  }
  if (ks == 8) return fd_launch<64, 8>(tW, tX, a, tiles * 8, stream);
  if (ks == 4) return fd_launch<64, 4>(tW, tX, a, tiles * 4, stream);
  if (ks == 2) return fd_launch<64, 2>(tW, tX, a, tiles * 2, stream);
  return fd_launch<64, 1>(tW, tX, a, tiles < 148 ? tiles : 148, stream);
}

}  // extern "C"
