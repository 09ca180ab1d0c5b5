// Flash attention forward for sm_100a (bf16, GQA, causal or full), tcgen05 + TMA. Head dim 128, or the
// multi-latent-attention shape: 192 for Q/K (128 + 64 rope columns) with 128 for V and the output.
//
// One CTA owns a tile of 128 query rows of one head and walks over the key/value tiles:
//   S = Q K^T          tcgen05.mma, both operands K-major from shared memory, S in tensor memory
//   P = exp2(S - m)    128 "softmax" threads, one query row each, read S with tcgen05.ld
//   O += P V           P written as bf16 to shared memory (K-major A operand), V is the MN-major
//                      B operand, O accumulates in tensor memory
// S is double-buffered in TMEM so the tensor core computes S_{j+1} while the softmax threads work
// on S_j. The running maximum is updated lazily: O is rescaled in TMEM only when the row maximum
// grew by more than 2^8, which keeps exp2 arguments bounded without touching O on most tiles.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 = softmax,
// O rescale and epilogue. Every wait is bounded (see common.cuh).
#include "common.cuh"

namespace mfb {

constexpr int kFaThreads = 192;
constexpr int kTile = 128;         // query rows per CTA and keys per step
constexpr int kHd = 128;           // head dimension
constexpr int kSubBytes = kTile * 128;      // one [128 rows][128 B] swizzled sub-tile (64 bf16 columns)
constexpr int kTileBytes = 2 * kSubBytes;   // 128 x 128 bf16
constexpr float kRescaleThreshold = 8.0f;   // log2 units

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA pipe (x <= 0): round-to-nearest split x = n + f, cubic for 2^f on [-0.5, 0.5]
// (max relative error 7.5e-5), n added to the exponent field. The MUFU unit does 16 ex2 per clock
// per SM, which is the bottleneck of the softmax; half of the exponentials go through this path.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -125.f);
  const float xr = x + 12582912.f;            // 1.5 * 2^23: low mantissa bits now hold n
  const float f = x - (xr - 12582912.f);
  float p = fmaf(0.05517165f, f, 0.24261112f);
  p = fmaf(p, f, 0.69326099f);
  p = fmaf(p, f, 0.99992807f);
  return __uint_as_float(__float_as_uint(p) + (__float_as_uint(xr) << 23));
}

struct FaArgs {
  int seq_q, seq_k;      // tokens per sequence
  int q_off_tiles;       // causal: query row i sits at key position q_off_tiles * 128 + i
  int num_q_heads, group;  // group = q heads per kv head
  int causal;
  float scale_log2;      // softmax scale * log2(e)
  float* lse;            // [B, Hq, Sq] natural-log LSE
  int* status;
};

// HDQK: width of a Q / K head (128 or 192). With 192 the K tile is single-buffered so that everything still fits
// in shared memory; the next K tile then loads while the softmax of the current one runs.
template <int HDQK>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                      const FaArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int QK_SUBS = HDQK / 64;                 // 64-column sub-tiles of a Q / K tile
  constexpr int QK_BYTES = QK_SUBS * kSubBytes;
  constexpr int KST = (HDQK == 128) ? 2 : 1;         // K stages
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + QK_BYTES;               // KST stages
  uint8_t* sV = sK + KST * QK_BYTES;         // 2 stages
  uint8_t* sP = sV + 2 * kTileBytes;         // 2 P tiles; the first doubles as the O staging buffer
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * kTileBytes);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* s_empty = bars + 11;    // 2
  uint64_t* p_ready = bars + 13;    // 2
  uint64_t* pv_done = bars + 15;    // 2
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_tile = gridDim.x - 1 - blockIdx.x;   // heavy (late) tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / args.group;
  const int diag_tile = args.q_off_tiles + q_tile;   // key tile that holds the causal diagonal of this query tile
  const int n_kv_all = args.seq_k / kTile;
  const int n_kv = args.causal ? (diag_tile + 1 < n_kv_all ? diag_tile + 1 : n_kv_all) : n_kv_all;
  const int q_row0 = batch * args.seq_q + q_tile * kTile;
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
      mbar_init(smem_u32(&s_empty[s]), 128);
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
  const uint32_t tmem_S = tmem_base;          // two buffers: +0, +128
  const uint32_t tmem_O = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t qb = smem_u32(q_full);
      mbar_expect_tx(qb, QK_BYTES);
#pragma unroll
      for (int i = 0; i < QK_SUBS; ++i)
        tma_load_2d(smem_u32(sQ) + i * kSubBytes, &tmQ, qb, head * HDQK + 64 * i, q_row0);
      bool ok = true;
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kst = j % KST;
        const uint32_t kph = (j / KST) & 1;
        ok = mbar_wait(smem_u32(&k_empty[kst]), kph ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) break;
        const uint32_t kb = smem_u32(&k_full[kst]);
        mbar_expect_tx(kb, QK_BYTES);
        const uint32_t kd = smem_u32(sK + kst * QK_BYTES);
#pragma unroll
        for (int i = 0; i < QK_SUBS; ++i)
          tma_load_2d(kd + i * kSubBytes, &tmK, kb, kv_head * HDQK + 64 * i, k_row0 + j * kTile);
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
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = umma_idesc_bf16(kTile, kTile, 0, 0);  // A=Q K-major, B=K K-major
      constexpr uint32_t IDESC_PV = umma_idesc_bf16(kTile, kHd, 0, 1);    // A=P K-major, B=V MN-major
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kst = j % KST;
        const uint32_t kph = (j / KST) & 1;
        if (!mbar_wait(smem_u32(&k_full[kst]), kph, abort_flag, args.status, kStatusWaitTimeoutMma)) return false;
        if (!mbar_wait(smem_u32(&s_empty[st]), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + kst * QK_BYTES);
#pragma unroll
        for (int k = 0; k < HDQK / 16; ++k) {
          const uint32_t off = (k >> 2) * kSubBytes + (k & 3) * 32;
          umma_f16_ss(tmem_S + st * kTile, umma_desc_kmajor_sw128(qa + off), umma_desc_kmajor_sw128(ka + off),
                      IDESC_QK, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_full[st]));
        umma_commit(smem_u32(&k_empty[kst]));
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(smem_u32(&p_ready[st]), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        ok = mbar_wait(smem_u32(&v_full[st]), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        const uint32_t pa = smem_u32(sP + st * kTileBytes), va = smem_u32(sV + st * kTileBytes);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {
          // A: P[q, key] K-major, 64-key sub-tiles; B: V[key, hd] MN-major, 64-column atoms 16 KB apart
          const uint64_t a_desc = umma_desc_kmajor_sw128(pa + (k >> 2) * kSubBytes + (k & 3) * 32);
          const uint64_t b_desc = umma_desc_mnmajor_sw128(va + k * 16 * 128, kSubBytes);
          umma_f16_ss(tmem_O, a_desc, b_desc, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&pv_done[st]));
        umma_commit(smem_u32(&v_empty[st]));
      }
    }
    __syncwarp();
  } else {
    const int ew = warp & 3;
    const int row = ew * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ok = mbar_wait(smem_u32(&s_full[st]), ph, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, 128, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[kTile];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t (&r)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sr[c * 32]);
        tmem_ld_32x32b_x32(tmem_S + st * kTile + lane_base + c * 32, r);
      }
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&s_empty[st]));
      float* s = reinterpret_cast<float*>(sr);
      if (args.causal && j == diag_tile) {
#pragma unroll
        for (int i = 0; i < kTile; ++i)
          if (i > row) s[i] = -INFINITY;
      }
      // eight independent chains: with one softmax warp per scheduler, dependent-issue latency
      // would otherwise dominate the row reductions
      float mxs[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) mxs[a] = s[a];
#pragma unroll
      for (int i = 8; i < kTile; i += 8) {
#pragma unroll
        for (int a = 0; a < 8; ++a) mxs[a] = fmaxf(mxs[a], s[i + a]);
      }
      float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                       fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
      mx *= args.scale_log2;   // the scale is positive, so the maximum commutes with it
      float alpha = 1.f;
      if (j == 0) {
        m_used = mx;
      } else if (mx > m_used + kRescaleThreshold) {
        alpha = ex2_approx(m_used - mx);
        m_used = mx;
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      float rsum[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) rsum[a] = 0.f;
#pragma unroll
      for (int i = 0; i < kTile; i += 8) {
#pragma unroll
        for (int a = 0; a < 8; ++a) {
          s[i + a] = ex2_approx(fmaf(s[i + a], args.scale_log2, neg_m));
          rsum[a] += s[i + a];
        }
      }
      l_sum = l_sum * alpha + ((rsum[0] + rsum[1]) + (rsum[2] + rsum[3])) + ((rsum[4] + rsum[5]) + (rsum[6] + rsum[7]));
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O may only be touched once the previous P.V has completed
        ok = mbar_wait(smem_u32(&pv_done[(j - 1) & 1]), ((j - 1) >> 1) & 1, abort_flag, args.status,
                       kStatusWaitTimeoutEpilogue);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint32_t r[16];
            tmem_ld_32x32b_x16(tmem_O + lane_base + c * 16, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x16(tmem_O + lane_base + c * 16, r);
          }
          tmem_st_wait();
        }
      }
      if (j > 1) {
        // this P buffer was last read by the P.V of tile j-2
        ok = ok && mbar_wait(smem_u32(&pv_done[st]), ((j - 2) >> 1) & 1, abort_flag, args.status,
                             kStatusWaitTimeoutEpilogue);
      }
      ok = named_bar_and(2, 128, ok);
      if (!ok) break;
      // P (bf16) -> shared memory, K-major with 128-byte swizzle: two sub-tiles of 64 keys
      uint8_t* prow = sP + st * kTileBytes + row * 128;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint4 v = make_uint4(pack_bf16x2(s[c * 8 + 0], s[c * 8 + 1]), pack_bf16x2(s[c * 8 + 2], s[c * 8 + 3]),
                             pack_bf16x2(s[c * 8 + 4], s[c * 8 + 5]), pack_bf16x2(s[c * 8 + 6], s[c * 8 + 7]));
        *reinterpret_cast<uint4*>(prow + (c >> 3) * kSubBytes + (((c & 7) ^ (row & 7)) << 4)) = v;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&p_ready[st]));
    }
    if (ok) {
      ok = mbar_wait(smem_u32(&pv_done[(n_kv - 1) & 1]), ((n_kv - 1) >> 1) & 1, abort_flag, args.status,
                     kStatusWaitTimeoutEpilogue);
      if (ok && n_kv > 1)
        ok = mbar_wait(smem_u32(&pv_done[n_kv & 1]), ((n_kv - 2) >> 1) & 1, abort_flag, args.status,
                       kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, 128, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.f / l_sum;
      uint8_t* orow = sP + row * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_O + lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = c * 4 + q;  // 16-byte chunk index along the 128 output columns
          uint4 v = make_uint4(
              pack_bf16x2(__uint_as_float(r[q * 8 + 0]) * inv_l, __uint_as_float(r[q * 8 + 1]) * inv_l),
              pack_bf16x2(__uint_as_float(r[q * 8 + 2]) * inv_l, __uint_as_float(r[q * 8 + 3]) * inv_l),
              pack_bf16x2(__uint_as_float(r[q * 8 + 4]) * inv_l, __uint_as_float(r[q * 8 + 5]) * inv_l),
              pack_bf16x2(__uint_as_float(r[q * 8 + 6]) * inv_l, __uint_as_float(r[q * 8 + 7]) * inv_l));
          *reinterpret_cast<uint4*>(orow + (chunk >> 3) * kSubBytes + (((chunk & 7) ^ (row & 7)) << 4)) = v;
        }
      }
      if (args.lse) {
        const size_t idx = (static_cast<size_t>(batch) * args.num_q_heads + head) * args.seq_q + q_tile * kTile + row;
        args.lse[idx] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
      }
      fence_proxy_async_smem();
      named_bar_sync(1, 128);
      if (threadIdx.x == 64) {
        tma_store_2d(&tmO, smem_u32(sP), head * kHd, q_row0);
        tma_store_2d(&tmO, smem_u32(sP) + kSubBytes, head * kHd + 64, q_row0);
        tma_commit_group();
        tma_wait_group<0>();
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

}  // namespace mfb

namespace {
using namespace mfb;

// q: [B*Sq, q_ld] bf16 rows with head h at columns [h*128, h*128+128); k, v likewise with Hkv heads.
// o: [B*Sq, o_ld]; lse: [B, Hq, Sq] fp32 (may be null). Sq, Sk multiples of 128. Causal: query i of a sequence sits
// at key position q_offset + i (q_offset a multiple of 128, q_offset + Sq <= Sk) and sees keys up to itself.
template <int HDQK>
int fa_fwd_launch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                         int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld, long long o_ld,
                         int causal, int q_offset, float scale, int* status, cudaStream_t stream) {
  if (Sq % kTile || Sk % kTile || Hq % Hkv || B <= 0 || q_offset % kTile || q_offset < 0 ||
      (causal && q_offset + Sq > Sk)) {
    mfb_host::set_error("flash_attn_fwd: unsupported shape B=%d Sq=%d Sk=%d Hq=%d Hkv=%d causal=%d q_offset=%d", B, Sq,
                        Sk, Hq, Hkv, causal, q_offset);
    return 1;
  }
  CUtensorMap tQ, tK, tV, tO;
  int rc;
  if ((rc = mfb_host::make_tmap_2d(&tQ, q, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)B * Sq, (uint64_t)Hq * HDQK, q_ld, kTile, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tK, k, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)B * Sk, (uint64_t)Hkv * HDQK, k_ld, kTile, 64))) return 30 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tV, v, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)B * Sk, (uint64_t)Hkv * kHd, v_ld, kTile, 64))) return 40 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tO, o, 2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)B * Sq, (uint64_t)Hq * kHd, o_ld, kTile, 64))) return 50 + rc;
  FaArgs a;
  a.seq_q = Sq; a.seq_k = Sk; a.q_off_tiles = q_offset / kTile; a.num_q_heads = Hq; a.group = Hq / Hkv;
  a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.lse = lse; a.status = status;
  constexpr int QK_BYTES = (HDQK / 64) * kSubBytes;
  constexpr int SMEM = (1 + (HDQK == 128 ? 2 : 1)) * QK_BYTES + 4 * kTileBytes + 18 * 8 + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_attn_fwd_kernel<HDQK>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("flash_attn_fwd: cannot raise shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  dim3 grid(Sq / kTile, Hq, B);
  flash_attn_fwd_kernel<HDQK><<<grid, kFaThreads, SMEM, stream>>>(tQ, tK, tV, tO, a);
  if (cudaGetLastError() != cudaSuccess) {
    mfb_host::set_error("flash_attn_fwd: launch failed");
    return 11;
  }
  return 0;
}

}  // namespace

extern "C" {
using namespace mfb;

int mfb_flash_attn_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                        int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld, long long o_ld, int causal,
                        int q_offset, float scale, int* status, cudaStream_t stream);

static int g_fa_fwd_variant = 2;   // 2: two query tiles per CTA (flash_attention_fwd2.cu); 1: one tile per CTA
void mfb_flash_attn_set_fwd_variant(int v) { g_fa_fwd_variant = (v == 1) ? 1 : 2; }

int mfb_flash_attn_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                          int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld, long long o_ld,
                          int causal, int q_offset, float scale, int* status, cudaStream_t stream) {
  if (g_fa_fwd_variant == 2)
    return mfb_flash_attn_fwd2(q, k, v, o, lse, B, Sq, Sk, Hq, Hkv, q_ld, k_ld, v_ld, o_ld, causal, q_offset, scale,
                               status, stream);
  return fa_fwd_launch<128>(q, k, v, o, lse, B, Sq, Sk, Hq, Hkv, q_ld, k_ld, v_ld, o_ld, causal, q_offset, scale, status,
                            stream);
}

// Multi-latent-attention shape: q, k heads of 192 columns (head h at columns [h*192, h*192+192)), v and o heads of 128.
int mfb_flash_attn_fwd_mla(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                           int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld, long long o_ld,
                           int causal, int q_offset, float scale, int* status, cudaStream_t stream) {
  return fa_fwd_launch<192>(q, k, v, o, lse, B, Sq, Sk, Hq, Hkv, q_ld, k_ld, v_ld, o_ld, causal, q_offset, scale, status,
                            stream);
}

int mfb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                       int Hq, int Hkv, long long q_ld, long long k_ld, long long v_ld, long long o_ld,
                       int causal, float scale, int* status, cudaStream_t stream) {
  if (causal && Sq != Sk) {
    mfb_host::set_error("flash_attn_fwd: causal with Sq != Sk needs mfb_flash_attn_fwd_ex and a query offset");
    return 1;
  }
  return mfb_flash_attn_fwd_ex(q, k, v, o, lse, B, Sq, Sk, Hq, Hkv, q_ld, k_ld, v_ld, o_ld, causal, 0, scale, status,
                               stream);
}

}  // extern "C"

// =================================================================================================
// Backward
// =================================================================================================
// One CTA owns a tile of 128 keys of one KV head and loops over the query heads of its group and
// the query tiles that see it. Per (head, query tile):
//   S  = Q K^T, dP = dO V^T                      (tensor memory, lanes = query rows)
//   P  = exp2(S*scale - lse), dS = P (dP - delta) scale     (softmax threads -> bf16 in smem)
//   dV += P^T dO, dK += dS^T Q                   (accumulate in tensor memory over the whole loop)
//   dQ_part = dS K  -> fp32 atomics into a scratch accumulator (converted to bf16 afterwards)
// The same [query][key] shared-memory image of P / dS serves as MN-major A operand (for the
// transposed products) and as K-major A operand (for dQ).
namespace mfb {

struct FaBwdArgs {
  int seq_q, seq_k;      // tokens per sequence on the query / key side
  int q_off_tiles;       // causal: query row i sits at key position q_off_tiles * 128 + i
  int num_q_heads, num_kv_heads, group;
  int causal;
  float scale, scale_log2;
  const float* lse;      // [B, Hq, S]
  const float* delta;    // [B, Hq, S]
  float* dq_accum;       // [B*S, Hq*128] fp32, zero-initialised
  int* status;
};

__global__ void __launch_bounds__(kFaThreads, 1)
flash_attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      const __grid_constant__ CUtensorMap tmdK, const __grid_constant__ CUtensorMap tmdV,
                      const __grid_constant__ CUtensorMap tmdQ, const FaBwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQ = sV + kTileBytes;
  uint8_t* sdO = sQ + kTileBytes;
  uint8_t* sP = sdO + kTileBytes;
  uint8_t* sdS = sP + kTileBytes;
  uint8_t* sdQ = sdS + kTileBytes;   // fp32 staging of half a dQ_part tile: two [128 rows][32 floats] swizzled images
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdQ + kTileBytes);
  uint64_t* kv_full = bars;        // K and V of this CTA arrived
  uint64_t* qdo_full = bars + 1;   // Q_i and dO_i arrived
  uint64_t* qdo_empty = bars + 2;  // dV and dK MMAs done: the Q / dO buffers are reusable
  uint64_t* sdp_full = bars + 3;   // S and dP ready in tensor memory
  uint64_t* pds_ready = bars + 4;  // P and dS written to shared memory (128 arrivals)
  uint64_t* s_free = bars + 5;     // dQ_part consumed: the dP columns are reusable (128 arrivals)
  uint64_t* dq_ready = bars + 6;   // dQ_part is complete in tensor memory
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv_tile = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const int n_q_tiles = args.seq_q / kTile;
  int first_q = args.causal ? kv_tile - args.q_off_tiles : 0;   // first query tile that sees this key tile
  if (first_q < 0) first_q = 0;
  if (first_q > n_q_tiles) first_q = n_q_tiles;
  const int iters_per_head = n_q_tiles - first_q;
  const int n_iter = iters_per_head * args.group;
  const int row_base = batch * args.seq_q;       // query-side rows (Q, dO, dQ)
  const int krow_base = batch * args.seq_k;      // key-side rows (K, V, dK, dV)

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(kv_full), 1);
    mbar_init(smem_u32(qdo_full), 1);
    mbar_init(smem_u32(qdo_empty), 1);
    mbar_init(smem_u32(sdp_full), 1);
    mbar_init(smem_u32(pds_ready), 128);
    mbar_init(smem_u32(s_free), 128);
    mbar_init(smem_u32(dq_ready), 1);
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
  // dQ_part shares the dP columns, so S of the next iteration can be issued while dQ_part is still being drained
  const uint32_t tmem_dQ = tmem_dP;

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t kvb = smem_u32(kv_full);
      mbar_expect_tx(kvb, 2 * kTileBytes);
      const int krow = krow_base + kv_tile * kTile;
      tma_load_2d(smem_u32(sK), &tmK, kvb, kv_head * kHd, krow);
      tma_load_2d(smem_u32(sK) + kSubBytes, &tmK, kvb, kv_head * kHd + 64, krow);
      tma_load_2d(smem_u32(sV), &tmV, kvb, kv_head * kHd, krow);
      tma_load_2d(smem_u32(sV) + kSubBytes, &tmV, kvb, kv_head * kHd + 64, krow);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int hq = kv_head * args.group + it / iters_per_head;
        const int qi = first_q + it % iters_per_head;
        ok = mbar_wait(smem_u32(qdo_empty), (it & 1) ^ 1, abort_flag, args.status, kStatusWaitTimeoutProducer);
        if (!ok) break;
        const uint32_t fb = smem_u32(qdo_full);
        mbar_expect_tx(fb, 2 * kTileBytes);
        const int qrow = row_base + qi * kTile;
        tma_load_2d(smem_u32(sQ), &tmQ, fb, hq * kHd, qrow);
        tma_load_2d(smem_u32(sQ) + kSubBytes, &tmQ, fb, hq * kHd + 64, qrow);
        tma_load_2d(smem_u32(sdO), &tmdO, fb, hq * kHd, qrow);
        tma_load_2d(smem_u32(sdO) + kSubBytes, &tmdO, fb, hq * kHd + 64, qrow);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC_KK = umma_idesc_bf16(kTile, kTile, 0, 0);   // K-major x K-major
      constexpr uint32_t IDESC_MM = umma_idesc_bf16(kTile, kHd, 1, 1);     // MN-major x MN-major
      constexpr uint32_t IDESC_KM = umma_idesc_bf16(kTile, kHd, 0, 1);     // K-major x MN-major
      bool ok = mbar_wait(smem_u32(kv_full), 0, abort_flag, args.status, kStatusWaitTimeoutMma);
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV), qa = smem_u32(sQ), doa = smem_u32(sdO);
      const uint32_t pa = smem_u32(sP), dsa = smem_u32(sdS);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        ok = mbar_wait(smem_u32(qdo_full), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
        // the S columns were last read by the softmax threads before pds_ready of the previous iteration
#pragma unroll
        for (int k = 0; k < kHd / 16; ++k) {
          const uint32_t off = (k >> 2) * kSubBytes + (k & 3) * 32;
          umma_f16_ss(tmem_S, umma_desc_kmajor_sw128(qa + off), umma_desc_kmajor_sw128(ka + off), IDESC_KK,
                      k > 0 ? 1u : 0u);
        }
        // the dP columns hold dQ_part of the previous iteration until the softmax threads have drained it
        ok = mbar_wait(smem_u32(s_free), ph ^ 1, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kHd / 16; ++k) {
          const uint32_t off = (k >> 2) * kSubBytes + (k & 3) * 32;
          umma_f16_ss(tmem_dP, umma_desc_kmajor_sw128(doa + off), umma_desc_kmajor_sw128(va + off), IDESC_KK,
                      k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(sdp_full));
        ok = mbar_wait(smem_u32(pds_ready), ph, abort_flag, args.status, kStatusWaitTimeoutMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {   // reduction over the 128 query rows
          const uint32_t koff = k * 16 * 128;
          umma_f16_ss(tmem_dV, umma_desc_mnmajor_sw128(pa + koff, kSubBytes),
                      umma_desc_mnmajor_sw128(doa + koff, kSubBytes), IDESC_MM, (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {
          const uint32_t koff = k * 16 * 128;
          umma_f16_ss(tmem_dK, umma_desc_mnmajor_sw128(dsa + koff, kSubBytes),
                      umma_desc_mnmajor_sw128(qa + koff, kSubBytes), IDESC_MM, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(qdo_empty));          // Q and dO can be overwritten by the next loads
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k) {   // dQ_part = dS K, reduction over the 128 keys
          const uint64_t a_desc = umma_desc_kmajor_sw128(dsa + (k >> 2) * kSubBytes + (k & 3) * 32);
          const uint64_t b_desc = umma_desc_mnmajor_sw128(ka + k * 16 * 128, kSubBytes);
          umma_f16_ss(tmem_dQ, a_desc, b_desc, IDESC_KM, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(dq_ready));
      }
    }
    __syncwarp();
  } else {
    const int ew = warp & 3;
    const int row = ew * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(ew * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const uint32_t ph = it & 1;
      const int hq = kv_head * args.group + it / iters_per_head;
      const int qi = first_q + it % iters_per_head;
      const size_t stat_idx = (static_cast<size_t>(batch) * args.num_q_heads + hq) * args.seq_q + qi * kTile + row;
      const float lse2 = args.lse[stat_idx] * 1.4426950408889634f;
      const float dlt = args.delta[stat_idx];
      ok = mbar_wait(smem_u32(sdp_full), ph, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, 128, ok);
      if (!ok) break;
      tc_fence_after();
      const bool diag = args.causal && (qi + args.q_off_tiles == kv_tile);
      uint8_t* prow = sP + row * 128;
      uint8_t* dsrow = sdS + row * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32b_x32(tmem_S + lane_base + c * 32, rs);
        tmem_ld_32x32b_x32(tmem_dP + lane_base + c * 32, rp);
        tmem_ld_wait();
        float p[32], ds[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float pv = ex2_approx(__uint_as_float(rs[i]) * args.scale_log2 - lse2);
          if (diag && (c * 32 + i) > row) pv = 0.f;
          p[i] = pv;
          ds[i] = pv * (__uint_as_float(rp[i]) - dlt) * args.scale;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = c * 4 + q;
          const int off = (chunk >> 3) * kSubBytes + (((chunk & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(prow + off) =
              make_uint4(pack_bf16x2(p[q * 8 + 0], p[q * 8 + 1]), pack_bf16x2(p[q * 8 + 2], p[q * 8 + 3]),
                         pack_bf16x2(p[q * 8 + 4], p[q * 8 + 5]), pack_bf16x2(p[q * 8 + 6], p[q * 8 + 7]));
          *reinterpret_cast<uint4*>(dsrow + off) =
              make_uint4(pack_bf16x2(ds[q * 8 + 0], ds[q * 8 + 1]), pack_bf16x2(ds[q * 8 + 2], ds[q * 8 + 3]),
                         pack_bf16x2(ds[q * 8 + 4], ds[q * 8 + 5]), pack_bf16x2(ds[q * 8 + 6], ds[q * 8 + 7]));
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(pds_ready));
      // dQ_part lands in the dP columns once the last MMA group has completed
      ok = mbar_wait(smem_u32(dq_ready), ph, abort_flag, args.status, kStatusWaitTimeoutEpilogue);
      ok = named_bar_and(2, 128, ok);
      if (!ok) break;
      tc_fence_after();
      // dQ_part -> fp32 accumulator in global memory through the TMA reduce-add path: 64 columns at a time are
      // staged in shared memory (swizzled 128-byte rows) and added by one bulk reduction per 32-column image,
      // which costs the L2 one full-line reduction per row instead of eight 16-byte atomics per thread
      const int qrow = row_base + qi * kTile;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (threadIdx.x == 64) tma_wait_group_read<0>();      // the previous reduction has read the staging buffer
        named_bar_sync(1, 128);
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_dQ + lane_base + half * 64 + sub * 32, r);
          tmem_ld_wait();
          uint8_t* drow = sdQ + sub * (kTile * 128) + row * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(drow + ((ch ^ (row & 7)) << 4)) = make_uint4(r[ch * 4], r[ch * 4 + 1], r[ch * 4 + 2], r[ch * 4 + 3]);
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (threadIdx.x == 64) {
          tma_reduce_add_2d(&tmdQ, smem_u32(sdQ), hq * kHd + half * 64, qrow);
          tma_reduce_add_2d(&tmdQ, smem_u32(sdQ) + kTile * 128, hq * kHd + half * 64 + 32, qrow);
          tma_commit_group();
        }
      }
      tc_fence_before();
      mbar_arrive(smem_u32(s_free));
    }
    if (ok) {
      // all MMAs have completed (last dq_ready wait above); write dK and dV of this tile
      const int krow = krow_base + kv_tile * kTile;
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tmem_dK : tmem_dV;
        uint8_t* stage = which == 0 ? sP : sdS;
        uint8_t* orow = stage + row * 128;
        if (n_iter > 0) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(src + lane_base + c * 32, r);
            tmem_ld_wait();
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
        } else {
          // no query tile sees this key tile (keys beyond the last query's diagonal): its gradients are zero
#pragma unroll
          for (int chunk = 0; chunk < 16; ++chunk)
            *reinterpret_cast<uint4*>(orow + (chunk >> 3) * kSubBytes + ((chunk & 7) << 4)) = make_uint4(0, 0, 0, 0);
        }
      }
      fence_proxy_async_smem();
      named_bar_sync(1, 128);
      if (threadIdx.x == 64) {
        tma_store_2d(&tmdK, smem_u32(sP), kv_head * kHd, krow);
        tma_store_2d(&tmdK, smem_u32(sP) + kSubBytes, kv_head * kHd + 64, krow);
        tma_store_2d(&tmdV, smem_u32(sdS), kv_head * kHd, krow);
        tma_store_2d(&tmdV, smem_u32(sdS) + kSubBytes, kv_head * kHd + 64, krow);
        tma_commit_group();
        tma_wait_group<0>();
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

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (token, head)
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
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

// dq (bf16, row pitch dq_ld) = dq_accum (fp32, contiguous [T, width])
__global__ void fa_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long T,
                                     int width, long long dq_ld) {
  const int wv = width / 4;
  const long long total = T * wv;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / wv;
    const int c = static_cast<int>(i - t * wv);
    const float4 v = reinterpret_cast<const float4*>(acc + t * width)[c];
    uint2 o = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    *reinterpret_cast<uint2*>(dq + t * dq_ld + c * 4) = o;
  }
}

}  // namespace mfb

extern "C" {
using namespace mfb;

int mfb_flash_attn_bwd2(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                        void* dq, void* dk, void* dv, void* scratch, int B, int S, int Sk, int Hq, int Hkv,
                        long long q_ld, long long k_ld, long long v_ld, long long o_ld, long long do_ld,
                        long long dq_ld, long long dk_ld, long long dv_ld, int causal, int q_offset, float scale,
                        int* status, cudaStream_t stream);
long long mfb_flash_attn_bwd2_scratch_bytes(int B, int Sq, int Sk, int Hq, int Hkv);

static int g_fa_bwd_variant = 2;   // 2: pipelined kernel with keys on the lanes (flash_attention_bwd2.cu); 1: the serial one
void mfb_flash_attn_set_bwd_variant(int v) { g_fa_bwd_variant = (v == 1) ? 1 : 2; }

// Number of bytes of scratch that mfb_flash_attn_bwd / _ex need for Sq queries and Sk keys per sequence (either
// kernel variant): fp32 dQ accumulator, delta, and the fp32 dK / dV accumulators of a split query-head group.
long long mfb_flash_attn_bwd_scratch_bytes_ex(int B, int Sq, int Sk, int Hq, int Hkv) {
  return mfb_flash_attn_bwd2_scratch_bytes(B, Sq, Sk, Hq, Hkv);
}
// The same for Sq == Sk with the number of KV heads unknown (bounded by the query heads).
long long mfb_flash_attn_bwd_scratch_bytes(int B, int S, int Hq) {
  return mfb_flash_attn_bwd2_scratch_bytes(B, S, S, Hq, Hq);
}

// Gradients of attention with Sq queries and Sk keys per sequence (causal: query i at key position q_offset + i).
// q/k/v/o/do as in the forward; dq/dk/dv are written with their own row pitches (they may be column ranges of one
// packed gradient buffer); dk/dv cover all Sk keys. `scratch` must hold mfb_flash_attn_bwd_scratch_bytes(B, Sq, Hq)
// bytes; this call zeroes the part it accumulates into.
int mfb_flash_attn_bwd_ex(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                          const float* lse, void* dq, void* dk, void* dv, void* scratch, int B, int S, int Sk, int Hq,
                          int Hkv, long long q_ld, long long k_ld, long long v_ld, long long o_ld, long long do_ld,
                          long long dq_ld, long long dk_ld, long long dv_ld, int causal, int q_offset, float scale,
                          int* status, cudaStream_t stream) {
  if (g_fa_bwd_variant == 2)
    return mfb_flash_attn_bwd2(q, k, v, o, d_o, lse, dq, dk, dv, scratch, B, S, Sk, Hq, Hkv, q_ld, k_ld, v_ld, o_ld, do_ld,
                               dq_ld, dk_ld, dv_ld, causal, q_offset, scale, status, stream);
  if (S % kTile || Sk % kTile || Hq % Hkv || B <= 0 || q_offset % kTile || q_offset < 0 ||
      (causal && q_offset + S > Sk)) {
    mfb_host::set_error("flash_attn_bwd: unsupported shape B=%d Sq=%d Sk=%d Hq=%d Hkv=%d q_offset=%d", B, S, Sk, Hq, Hkv,
                        q_offset);
    return 1;
  }
  const long long T = static_cast<long long>(B) * S;
  const long long Tk = static_cast<long long>(B) * Sk;
  float* dq_accum = reinterpret_cast<float*>(scratch);
  float* delta = dq_accum + T * Hq * kHd;
  cudaMemsetAsync(dq_accum, 0, T * Hq * kHd * sizeof(float), stream);
  {
    const long long warps = T * Hq;
    const int threads = 256;
    const long long blocks = (warps * 32 + threads - 1) / threads;
    fa_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>((const __nv_bfloat16*)d_o, (const __nv_bfloat16*)o, delta,
                                                             B, S, Hq, do_ld, o_ld);
  }
  CUtensorMap tQ, tK, tV, tdO, tdK, tdV, tdQ;
  int rc;
  const CUtensorMapDataType BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if ((rc = mfb_host::make_tmap_2d(&tdQ, dq_accum, 4, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, T, (uint64_t)Hq * kHd,
                                   (uint64_t)Hq * kHd, kTile, 32, true))) return 80 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tQ, q, 2, BF, T, (uint64_t)Hq * kHd, q_ld, kTile, 64))) return 20 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tK, k, 2, BF, Tk, (uint64_t)Hkv * kHd, k_ld, kTile, 64))) return 30 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tV, v, 2, BF, Tk, (uint64_t)Hkv * kHd, v_ld, kTile, 64))) return 40 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdO, d_o, 2, BF, T, (uint64_t)Hq * kHd, do_ld, kTile, 64))) return 50 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdK, dk, 2, BF, Tk, (uint64_t)Hkv * kHd, dk_ld, kTile, 64))) return 60 + rc;
  if ((rc = mfb_host::make_tmap_2d(&tdV, dv, 2, BF, Tk, (uint64_t)Hkv * kHd, dv_ld, kTile, 64))) return 70 + rc;
  FaBwdArgs a;
  a.seq_q = S; a.seq_k = Sk; a.q_off_tiles = q_offset / kTile; a.num_q_heads = Hq; a.num_kv_heads = Hkv;
  a.group = Hq / Hkv; a.causal = causal;
  a.scale = scale; a.scale_log2 = scale * 1.4426950408889634f;
  a.lse = lse; a.delta = delta; a.dq_accum = dq_accum; a.status = status;
  constexpr int SMEM = 7 * kTileBytes + 9 * 8 + 16 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
      mfb_host::set_error("flash_attn_bwd: cannot raise shared memory limit");
      return 10;
    }
    attr_set = true;
  }
  dim3 grid(Sk / kTile, Hkv, B);
  flash_attn_bwd_kernel<<<grid, kFaThreads, SMEM, stream>>>(tQ, tK, tV, tdO, tdK, tdV, tdQ, a);
  {
    const long long total = T * (Hq * kHd / 4);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    fa_dq_convert_kernel<<<(unsigned)blocks, 256, 0, stream>>>(dq_accum, (__nv_bfloat16*)dq, T, Hq * kHd, dq_ld);
  }
  if (cudaGetLastError() != cudaSuccess) {
    mfb_host::set_error("flash_attn_bwd: launch failed");
    return 11;
  }
  return 0;
}

int mfb_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                       const float* lse, void* dq, void* dk, void* dv, void* scratch, int B, int S, int Hq, int Hkv,
                       long long q_ld, long long k_ld, long long v_ld, long long o_ld, long long do_ld,
                       long long dq_ld, long long dk_ld, long long dv_ld, int causal, float scale, int* status,
                       cudaStream_t stream) {
  return mfb_flash_attn_bwd_ex(q, k, v, o, d_o, lse, dq, dk, dv, scratch, B, S, S, Hq, Hkv, q_ld, k_ld, v_ld, o_ld,
                               do_ld, dq_ld, dk_ld, dv_ld, causal, 0, scale, status, stream);
}

}  // extern "C"
