// W8A8 GEMM for sm_100a: int8 activations x int8 weights, int32 accumulation in tensor memory, per-row and
// per-column fp32 scales applied in the epilogue.
//
//   D[m, n] = bf16( sa[m] * sb[n] * sum_k A[m, k] * B[n, k] )            (+ bias[n] when given)
//
//   A  [M, K]  int8, K-major: activations quantised per token (dynamic) or with one calibrated scale
//   B  [N, K]  int8, K-major: weights quantised per output channel
//   sa [M], sb [N] fp32;  D [M, N] bf16
//
// tcgen05.mma kind::i8 (M 128, N 256, K 32 per instruction) reads both operands from shared memory, where TMA puts
// them with the 128-byte swizzle (128 int8 = one swizzle row, so a stage holds a K block of 128). The integer sum is
// exact, so the result does not depend on the tile walk. Two accumulators of 256 columns alternate between the MMA
// issuer and the four epilogue warps; the epilogue turns int32 into float, scales, rounds to bf16 and leaves through
// swizzled staging and TMA stores (which clip rows past M and columns past N). Persistent grid, one CTA per SM.
//
// The reference quantises to int8 through an external toolkit and runs the product on the vendor's quantised matmul
// (mindformers/utils/quantization_config.py:204-595 holds the configuration side); this is the product itself.
//
// `mfb_quant_act_int8` is the per-token dynamic quantiser for A: one warp per row, absmax / 127.
#include "common.cuh"

namespace mfb {
namespace i8 {

constexpr int kBM = 128, kBN = 256, kBK = 128;     // bytes == elements
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kABytes = kBM * kBK, kBBytes = kBN * kBK;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kStagingBytes = 128 * 128;
constexpr int kTmemCols = 2 * kBN;

struct Args {
  int M, N, K;
  int num_m_blocks, num_n_blocks;
  const float* sa;
  const float* sb;
  const __nv_bfloat16* bias;   // may be null
  int* status;
};

// kind::i8, signed 8-bit operands (both K-major), 32-bit integer accumulator
__host__ __device__ constexpr uint32_t idesc_s8(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void umma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tile_of(const Args& g, int tile, int& m_blk, int& n_blk) {
  constexpr int kBand = 16;                       // 16 row blocks share their weight tiles through L2
  const int per_band = kBand * g.num_n_blocks;
  const int band = tile / per_band;
  const int first = band * kBand;
  const int h = (g.num_m_blocks - first) < kBand ? (g.num_m_blocks - first) : kBand;
  const int r = tile - band * per_band;
  m_blk = first + r % h;
  n_blk = r / h;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_w8a8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmD, const Args args) {
  constexpr uint32_t IDESC = idesc_s8(kBM, kBN);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tfull_bar = bars + 2 * kStages;
  uint64_t* tempty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tfull_bar[s]), 1);
      mbar_init(smem_u32(&tempty_bar[s]), 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const int n_tiles = args.num_m_blocks * args.num_n_blocks;
  const int k_blocks = (args.K + kBK - 1) / kBK;   // TMA zero-fills the tail of K: zeros add nothing

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_of(args, tile, m_blk, n_blk);
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, kStageBytes);
          const uint32_t a_dst = smem_u32(smem + stage * kStageBytes);
          tma_load_2d(a_dst, &tmA, fb, kb * kBK, m_blk * kBM);
          // the weight tile arrives as two boxes of 128 rows (a TMA box has at most 256 rows; two keep the map
          // shared with narrower outputs)
          tma_load_2d(a_dst + kABytes, &tmB, fb, kb * kBK, n_blk * kBN);
          tma_load_2d(a_dst + kABytes + 128 * kBK, &tmB, fb, kb * kBK, n_blk * kBN + 128);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(smem_u32(&tempty_bar[acc]), acc_phase ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, args.status, kStatusWaitTimeoutMma);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * kStageBytes);
          const uint32_t b_base = a_base + kABytes;
#pragma unroll
          for (int k = 0; k < kBK / 32; ++k) {
            const uint64_t a_desc = umma_desc_kmajor_sw128(a_base + k * 32);
            const uint64_t b_desc = umma_desc_kmajor_sw128(b_base + k * 32);
            umma_i8_ss(d_tmem, a_desc, b_desc, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&tfull_bar[acc]));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int ew = warp & 3;
    const int row = ew * 32 + lane;
    const bool issuer = (threadIdx.x == 64);
    int acc = 0;
    uint32_t acc_phase = 0, chunk_counter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_of(args, tile, m_blk, n_blk);
      ok = mbar_wait(smem_u32(&tfull_bar[acc]), acc_phase, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, kEpiThreads, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * kBN;
      const int grow = m_blk * kBM + row;
      const float sa = grow < args.M ? __ldg(args.sa + grow) : 0.f;
#pragma unroll 1
      for (int c = 0; c < kBN / 64; ++c) {
        uint32_t v0[32], v1[32], packed[32];
        tmem_ld_32x32b_x32(t_addr + c * 64, v0);
        tmem_ld_32x32b_x32(t_addr + c * 64 + 32, v1);
        tmem_ld_wait();
        const int col0 = n_blk * kBN + c * 64;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float f[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int cc = (j < 2) ? (2 * i + j) : (32 + 2 * i + (j - 2));
            const int col = col0 + cc;
            const int raw = static_cast<int>(j < 2 ? v0[2 * i + j] : v1[2 * i + (j - 2)]);
            float x = 0.f;
            if (col < args.N) {
              x = static_cast<float>(raw) * sa * __ldg(args.sb + col);
              if (args.bias) x += __bfloat162float(args.bias[col]);
            }
            f[j] = x;
          }
          packed[i] = pack_bf16x2(f[0], f[1]);
          packed[16 + i] = pack_bf16x2(f[2], f[3]);
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
          if (col0 < args.N) tma_store_2d(&tmD, smem_u32(staging + buf * kStagingBytes), col0, m_blk * kBM);
          tma_commit_group();
        }
        ++chunk_counter;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (issuer) tma_wait_group<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// One warp per row: scale = absmax / 127 (1 for an all-zero row), q = round(x / scale) clamped to [-127, 127].
__global__ void quant_act_int8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int8_t* __restrict__ q,
                                      long long ldq, float* __restrict__ scale, const float* __restrict__ smooth,
                                      long long T, int K) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const __nv_bfloat16* xr = x + row * ldx;
  float m = 0.f;
  for (int k = lane; k < K; k += 32) {
    float v = __bfloat162float(xr[k]);
    if (smooth) v /= smooth[k];
    m = fmaxf(m, fabsf(v));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float s = m > 0.f ? m / 127.f : 1.f;
  const float inv = 1.f / s;
  int8_t* qr = q + row * ldq;
  for (int k = lane; k < K; k += 32) {
    float v = __bfloat162float(xr[k]);
    if (smooth) v /= smooth[k];
    int r = __float2int_rn(v * inv);
    r = r > 127 ? 127 : (r < -127 ? -127 : r);
    qr[k] = static_cast<int8_t>(r);
  }
  if (lane == 0) scale[row] = s;
}

}  // namespace i8
}  // namespace mfb

extern "C" {
using namespace mfb;

// A [M, K] int8 (row pitch lda bytes), B [N, K] int8 (row pitch ldb), D [M, N] bf16 (row pitch ldd elements);
// K, lda and ldb multiples of 16 (TMA), N and ldd multiples of 8.
int mfb_gemm_w8a8(const void* A, const void* B, void* D, const float* sa, const float* sb, const void* bias, int M, int N,
                  int K, long long lda, long long ldb, long long ldd, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 16 || lda % 16 || ldb % 16 || N % 8 || ldd % 8) {
    mfb_host::set_error("gemm_w8a8: M=%d N=%d K=%d lda=%lld ldb=%lld ldd=%lld (K, lda, ldb multiples of 16; N, ldd of 8)",
                        M, N, K, lda, ldb, ldd);
    return 1;
  }
  CUtensorMap tA, tB, tD;
  int rc;
  if ((rc = mfb_host::make_tmap_2d(&tA, A, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, M, K, lda, i8::kBM, i8::kBK))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tB, B, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, N, K, ldb, 128, i8::kBK))) return 30 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tD, D, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, M, N, ldd, i8::kBM, 64))) return 40 + rc;
  i8::Args a;
  a.M = M; a.N = N; a.K = K;
  a.num_m_blocks = (M + i8::kBM - 1) / i8::kBM;
  a.num_n_blocks = (N + i8::kBN - 1) / i8::kBN;
  a.sa = sa; a.sb = sb; a.bias = reinterpret_cast<const __nv_bfloat16*>(bias); a.status = status;
  constexpr int SMEM = i8::kStages * i8::kStageBytes + 2 * i8::kStagingBytes + (2 * i8::kStages + 4) * 8 + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(i8::gemm_w8a8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("gemm_w8a8: cannot raise the shared memory limit to %d", SMEM);
      return 10;
    }
    attr_set = true;
  }
  const int tiles = a.num_m_blocks * a.num_n_blocks;
  int sms = 148;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const int grid = tiles < sms ? tiles : sms;
  i8::gemm_w8a8_kernel<<<grid, i8::kThreads, SMEM, stream>>>(tA, tB, tD, a);
  if (cudaGetLastError() != cudaSuccess) { mfb_host::set_error("gemm_w8a8: launch failed"); return 11; }
  return 0;
}

// x [T, K] bf16 -> q [T, K] int8 and scale [T] fp32 (per-token dynamic quantisation); `smooth` [K] (may be null)
// divides the activations first (SmoothQuant).
int mfb_quant_act_int8(const void* x, long long ldx, void* q, long long ldq, float* scale, const float* smooth,
                       long long T, int K, cudaStream_t stream) {
  if (T <= 0 || K <= 0) { mfb_host::set_error("quant_act_int8: T=%lld K=%d", T, K); return 1; }
  const long long blocks = (T * 32 + 255) / 256;
  i8::quant_act_int8_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<int8_t*>(q), ldq, scale, smooth, T, K);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
