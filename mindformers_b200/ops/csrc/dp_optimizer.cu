// Data-parallel sharded optimizer fused with its collectives over NVLink peer memory (sm_100a).
//
// Each data-parallel rank owns the slice [begin, begin + n) of a flat gradient / parameter buffer that
// lives in peer-mapped ("symmetric") memory on every rank. One optimizer step is three launches:
//
//   dp_reduce_kernel   reduce-scatter by pulling: every rank sums its slice of all peers' gradient
//                      buffers with 16-byte peer loads (fp32 accumulation in rank order, so every run
//                      gives the same bits), writes the reduced slice locally and produces block partials
//                      of the squared norm. Before the first remote load each CTA waits (bounded) until all
//                      peers have announced that their backward pass is complete.
//   dp_adamw_kernel    clip + AdamW on the reduced slice, then the new bf16 parameters are stored to the
//                      parameter buffer of EVERY rank (all-gather by pushing, 16-byte peer stores). The last
//                      CTA to finish releases this rank's "parameters published" flag on all peers.
//   dp_wait_kernel     one CTA that waits (bounded) for the "published" flags of all peers, so the next
//                      forward pass on this stream sees complete parameters.
//
// Overlap with the backward pass: the layers' gradient ranges are reduced in buckets while the backward pass of
// the last micro-batch is still running. After the backward kernels of a bucket, dp_announce_kernel (launching
// stream) releases this rank's "bucket final" flag on every peer; on a side stream dp_wait_row_kernel (one warp,
// bounded) waits for all peers' flags of that bucket and a dp_reduce_kernel without announce / wait sums the part
// of the bucket that this rank owns. Only the one-warp wait kernel ever waits for another GPU, so the reduce
// kernel cannot hold resources while waiting and the compute stream never waits for the side stream before the
// end of the backward pass.
//
// Flags carry the step number (identical on all ranks), so they never need a reset. A rank cannot run ahead:
// dp_wait of step t needs every peer's dp_adamw of step t, and a peer's dp_reduce of step t + 1 (the only
// reader of this rank's gradients) comes after that in its stream. Every wait gives up after
// MFB_WAIT_LIMIT_NS, records kStatusPeerFlagTimeout in the status word and lets the kernel finish.
#include "common.cuh"

namespace mfb {

constexpr int kDpMaxRanks = 8;
constexpr int kDpThreads = 256;

struct DpArgs {
  int world, rank, epoch;
  long long begin, n;                 // slice owned by this rank (elements); n is a multiple of 8
  const float* peer_grad[kDpMaxRanks];  // full gradient buffer of every rank (fp32)
  __nv_bfloat16* peer_param[kDpMaxRanks];  // full parameter buffer of every rank (bf16)
  int* flags_peer[kDpMaxRanks];       // flag array [2][kDpMaxRanks] of every rank
  int* flags_local;
  int* status;
  int* ticket;                        // local counter, zero before launch (reset by the last CTA)
};

__device__ __forceinline__ void dp_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int dp_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 dp_ld_nc_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"  // L2-coherent: never served from a stale L1 line
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

// Thread 0 of the CTA waits until flags[0..world) >= want; returns false after the time limit.
__device__ bool dp_wait_all(const int* flags, int world, int want, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint64_t t0 = globaltimer_ns();
    for (int p = 0; p < world && ok; ++p) {
      uint32_t it = 0;
      while (dp_ld_acquire_sys(flags + p) < want) {
        if (((++it) & 0x3f) == 0 && globaltimer_ns() - t0 > MFB_WAIT_LIMIT_NS) {
          ok = 0;
          if (status) atomicCAS(status, 0, kStatusPeerFlagTimeout);
          break;
        }
        __nanosleep(128);
      }
    }
  }
  __syncthreads();
  return ok != 0;
}

constexpr int kDpBucketRows = 64;      // bucket flag rows per step
constexpr int kDpBucketFlagBase = 32;  // first int of the "gradients final" bucket rows inside a rank's flag array
constexpr int kDpPublishFlagBase = kDpBucketFlagBase + kDpBucketRows * kDpMaxRanks;   // "parameters published" rows

// SYNC: announce "gradients final" and wait for all peers inside the kernel (the pass after the backward pass).
// !SYNC: the caller has already waited (dp_wait_row_kernel earlier in the stream); a wait that timed out left its
// code in the status word, and the kernel then reads nothing.
template <bool SYNC>
__global__ void __launch_bounds__(kDpThreads)
dp_reduce_kernel(DpArgs a, float* __restrict__ reduced, float* __restrict__ partials) {
  bool ok;
  if (SYNC) {
    // announce: this rank's gradients are final (they were written by earlier kernels of this stream)
    if (blockIdx.x == 0 && threadIdx.x < a.world)
      dp_st_release_sys(a.flags_peer[threadIdx.x] + a.rank, a.epoch);
    ok = dp_wait_all(a.flags_local, a.world, a.epoch, a.status);
  } else {
    ok = a.status == nullptr || *reinterpret_cast<volatile int*>(a.status) == 0;
  }
  float acc = 0.f;
  if (ok) {
    const long long nvec = a.n >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      float4 g[kDpMaxRanks];
#pragma unroll
      for (int p = 0; p < kDpMaxRanks; ++p)      // all peers' loads in flight together
        if (p < a.world) g[p] = dp_ld_nc_f4(a.peer_grad[p] + a.begin + 4 * i);
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < kDpMaxRanks; ++p)      // fixed summation order: bit-identical on every run
        if (p < a.world) { s.x += g[p].x; s.y += g[p].y; s.z += g[p].z; s.w += g[p].w; }
      reinterpret_cast<float4*>(reduced)[i] = s;
      acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
    }
  }
  __shared__ float red[kDpThreads / 32];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < kDpThreads / 32; ++w) t += red[w];
    partials[blockIdx.x] = t;
  }
}

__global__ void dp_sum_partials_kernel(const float* __restrict__ partials, int parts, float* __restrict__ out,
                                       int accumulate) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < parts; i += blockDim.x) acc += partials[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) *out = accumulate ? *out + t : t;
  }
}

struct DpAdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, skip_threshold, grad_scale;
  long long decay_end;  // elements [0, decay_end) of the slice get weight decay
  int publish_row;      // >= 0: release this row of the "parameters published" bucket flags instead of the step's one flag
  int zero_grads;       // the kernel leaves zeros in the gradients it consumed (the next step's accumulation starts there)
};

__global__ void __launch_bounds__(kDpThreads)
dp_adamw_kernel(DpArgs a, DpAdamArgs h, unsigned short* __restrict__ lo, float* __restrict__ m,
                float* __restrict__ v, float* __restrict__ g, const float* __restrict__ sumsq,
                int* __restrict__ skipped) {
  float clip = h.grad_scale;
  bool bad = false;
  if (sumsq) {
    const float ss = *sumsq;
    const float nrm = sqrtf(ss) * fabsf(h.grad_scale);
    bad = !isfinite(ss) || (h.skip_threshold > 0.f && nrm >= h.skip_threshold);
    if (bad && blockIdx.x == 0 && threadIdx.x == 0 && skipped) *skipped = 1;
    if (!bad && h.max_norm > 0.f && nrm >= h.max_norm) clip *= h.max_norm / (nrm + 1e-6f);
  }
  if (!bad) {
    const float lr_t = h.lr / h.bc1;
    const float inv_bc2 = 1.f / h.bc2;
    const float decay = 1.f - h.lr * h.wd;
    __nv_bfloat16* own = a.peer_param[a.rank] + a.begin;
    const long long nvec = a.n >> 3;  // 8 elements (one 16-byte bf16 vector) per thread and iteration
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      const long long e0 = i * 8;
      const uint4 pv = *reinterpret_cast<const uint4*>(own + e0);
      const uint4 lv = *reinterpret_cast<const uint4*>(lo + e0);
      const unsigned short* ph = reinterpret_cast<const unsigned short*>(&pv);
      const unsigned short* pl = reinterpret_cast<const unsigned short*>(&lv);
      float gg[8], mm[8], vv[8];
      *reinterpret_cast<float4*>(gg) = *reinterpret_cast<const float4*>(g + e0);
      *reinterpret_cast<float4*>(gg + 4) = *reinterpret_cast<const float4*>(g + e0 + 4);
      *reinterpret_cast<float4*>(mm) = *reinterpret_cast<const float4*>(m + e0);
      *reinterpret_cast<float4*>(mm + 4) = *reinterpret_cast<const float4*>(m + e0 + 4);
      *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(v + e0);
      *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(v + e0 + 4);
      uint4 np, nl;
      unsigned short* nph = reinterpret_cast<unsigned short*>(&np);
      unsigned short* npl = reinterpret_cast<unsigned short*>(&nl);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float w = __uint_as_float(((uint32_t)ph[j] << 16) + (uint32_t)(int32_t)(int16_t)pl[j]);
        const float gr = gg[j] * clip;
        mm[j] = h.beta1 * mm[j] + (1.f - h.beta1) * gr;
        vv[j] = h.beta2 * vv[j] + (1.f - h.beta2) * gr * gr;
        if (e0 + j < h.decay_end) w *= decay;
        w -= lr_t * mm[j] / (sqrtf(vv[j] * inv_bc2) + h.eps);
        const uint32_t wb = __float_as_uint(w);
        const uint32_t nhi = (wb + 0x8000u) >> 16;
        nph[j] = (unsigned short)nhi;
        npl[j] = (unsigned short)((wb - (nhi << 16)) & 0xffffu);
      }
      *reinterpret_cast<float4*>(m + e0) = *reinterpret_cast<float4*>(mm);
      *reinterpret_cast<float4*>(m + e0 + 4) = *reinterpret_cast<float4*>(mm + 4);
      *reinterpret_cast<float4*>(v + e0) = *reinterpret_cast<float4*>(vv);
      *reinterpret_cast<float4*>(v + e0 + 4) = *reinterpret_cast<float4*>(vv + 4);
      *reinterpret_cast<uint4*>(lo + e0) = nl;
      if (h.zero_grads) {
        *reinterpret_cast<float4*>(g + e0) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(g + e0 + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      // publish: own copy first, then every peer's copy of this slice
      for (int p = 0; p < a.world; ++p) {
        const int q = (a.rank + p) % a.world;
        *reinterpret_cast<uint4*>(a.peer_param[q] + a.begin + e0) = np;
      }
    }
  }
  if (bad && h.zero_grads) {
    const long long nvec = a.n >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x)
      reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // completion: the last CTA releases the "published" flag on every peer
  __threadfence_system();
  __syncthreads();
  __shared__ int last;
  if (threadIdx.x == 0) last = (atomicAdd(a.ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (last) {
    __threadfence_system();
    const int off = h.publish_row >= 0 ? kDpPublishFlagBase + h.publish_row * kDpMaxRanks : kDpMaxRanks;
    if (threadIdx.x < a.world) dp_st_release_sys(a.flags_peer[threadIdx.x] + off + a.rank, a.epoch);
    if (threadIdx.x == 0) *a.ticket = 0;
  }
}

__global__ void dp_wait_kernel(DpArgs a) {
  dp_wait_all(a.flags_local + kDpMaxRanks, a.world, a.epoch, a.status);
}

// Bucket protocol: row `row` of the bucket flags. The announce follows the bucket's backward kernels in its stream.
__global__ void dp_announce_kernel(DpArgs a, int row) {
  if (threadIdx.x < a.world)
    dp_st_release_sys(a.flags_peer[threadIdx.x] + kDpBucketFlagBase + row * kDpMaxRanks + a.rank, a.epoch);
}
__global__ void dp_wait_row_kernel(DpArgs a, int row) {
  dp_wait_all(a.flags_local + kDpBucketFlagBase + row * kDpMaxRanks, a.world, a.epoch, a.status);
}
__global__ void dp_wait_published_row_kernel(DpArgs a, int row) {
  dp_wait_all(a.flags_local + kDpPublishFlagBase + row * kDpMaxRanks, a.world, a.epoch, a.status);
}

static inline int dp_grid(long long nvec, int max_ctas = 148 * 4) {
  long long blocks = (nvec + kDpThreads - 1) / kDpThreads;
  const long long cap = max_ctas > 0 && max_ctas < 148 * 4 ? max_ctas : 148 * 4;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// Number of floats of scratch that mfb_dp_reduce needs (block partials of the squared norm).
int mfb_dp_reduce_scratch() { return 148 * 4; }
// Number of ints in the per-rank flag array (two rows of kDpMaxRanks) plus the ticket word.
int mfb_dp_flag_words() { return kDpPublishFlagBase + kDpBucketRows * kDpMaxRanks; }
// Number of gradient buckets per step that the bucket flag rows can tell apart.
int mfb_dp_bucket_rows() { return kDpBucketRows; }

static int fill_dp_args(DpArgs* a, int world, int rank, int epoch, long long begin, long long n,
                        const long long* peer_grad, const long long* peer_param, const long long* peer_flags,
                        int* status) {
  if (world < 1 || world > kDpMaxRanks || rank < 0 || rank >= world) {
    mfb_host::set_error("dp optimizer: world %d / rank %d out of range (max %d ranks)", world, rank, kDpMaxRanks);
    return 1;
  }
  if ((n & 7) != 0 || (begin & 7) != 0) {
    mfb_host::set_error("dp optimizer: slice begin %lld / length %lld must be multiples of 8", begin, n);
    return 1;
  }
  a->world = world; a->rank = rank; a->epoch = epoch; a->begin = begin; a->n = n; a->status = status;
  for (int p = 0; p < world; ++p) {
    a->peer_grad[p] = peer_grad ? reinterpret_cast<const float*>(peer_grad[p]) : nullptr;
    a->peer_param[p] = peer_param ? reinterpret_cast<__nv_bfloat16*>(peer_param[p]) : nullptr;
    a->flags_peer[p] = reinterpret_cast<int*>(peer_flags[p]);
  }
  a->flags_local = a->flags_peer[rank];
  a->ticket = a->flags_local + 2 * kDpMaxRanks;
  return 0;
}

// reduced[0, n) = sum_p peer_grad[p][begin, begin + n);  *sumsq (+)= sum(reduced^2).
// peer_* are host arrays of `world` device addresses (this rank's own buffer at index `rank`).
int mfb_dp_reduce(int world, int rank, int epoch, long long begin, long long n, const long long* peer_grad,
                  const long long* peer_flags, float* reduced, float* scratch, float* sumsq, int accumulate,
                  int* status, cudaStream_t stream) {
  DpArgs a;
  if (fill_dp_args(&a, world, rank, epoch, begin, n, peer_grad, nullptr, peer_flags, status)) return 1;
  const int grid = dp_grid(n >> 2);
  dp_reduce_kernel<true><<<grid, kDpThreads, 0, stream>>>(a, reduced, scratch);
  dp_sum_partials_kernel<<<1, 256, 0, stream>>>(scratch, grid, sumsq, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Bucket `row` of step `epoch`: this rank's gradients of the bucket are final (stream order) -> tell every peer.
int mfb_dp_announce(int world, int rank, int epoch, int row, const long long* peer_flags, cudaStream_t stream) {
  DpArgs a;
  if (fill_dp_args(&a, world, rank, epoch, 0, 0, nullptr, nullptr, peer_flags, nullptr)) return 1;
  if (row < 0 || row >= kDpBucketRows) {
    mfb_host::set_error("dp optimizer: bucket row %d out of range (%d rows)", row, kDpBucketRows);
    return 1;
  }
  dp_announce_kernel<<<1, 32, 0, stream>>>(a, row);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Waits (one warp, bounded) until every peer has announced bucket `row`, then reduces [begin, begin + n) of it
// (the part this rank owns; n may be 0: wait only) and adds the squared norm of the result to *sumsq.
int mfb_dp_reduce_bucket(int world, int rank, int epoch, int row, long long begin, long long n,
                         const long long* peer_grad, const long long* peer_flags, float* reduced, float* scratch,
                         float* sumsq, int max_ctas, int* status, cudaStream_t stream) {
  DpArgs a;
  if (fill_dp_args(&a, world, rank, epoch, begin, n, peer_grad, nullptr, peer_flags, status)) return 1;
  if (row < 0 || row >= kDpBucketRows) {
    mfb_host::set_error("dp optimizer: bucket row %d out of range (%d rows)", row, kDpBucketRows);
    return 1;
  }
  dp_wait_row_kernel<<<1, 32, 0, stream>>>(a, row);
  if (n > 0) {
    const int grid = dp_grid(n >> 2, max_ctas);
    dp_reduce_kernel<false><<<grid, kDpThreads, 0, stream>>>(a, reduced, scratch);
    dp_sum_partials_kernel<<<1, 256, 0, stream>>>(scratch, grid, sumsq, 1);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// AdamW on the reduced slice + publication of the new bf16 parameters to every rank + completion wait.
int mfb_dp_adamw_allgather(int world, int rank, int epoch, long long begin, long long n,
                           const long long* peer_param, const long long* peer_flags, void* lo, float* m, float* v,
                           const float* reduced, const float* sumsq, int* skipped, long long decay_end, float lr,
                           float beta1, float beta2, float eps, float wd, float bc1, float bc2, float max_norm,
                           float skip_threshold, float grad_scale, int* status, cudaStream_t stream) {
  DpArgs a;
  if (fill_dp_args(&a, world, rank, epoch, begin, n, nullptr, peer_param, peer_flags, status)) return 1;
  DpAdamArgs h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.wd = wd; h.bc1 = bc1; h.bc2 = bc2;
  h.max_norm = max_norm; h.skip_threshold = skip_threshold; h.grad_scale = grad_scale; h.decay_end = decay_end;
  h.publish_row = -1; h.zero_grads = 0;
  dp_adamw_kernel<<<dp_grid(n >> 3), kDpThreads, 0, stream>>>(a, h, (unsigned short*)lo, m, v, const_cast<float*>(reduced),
                                                              sumsq, skipped);
  dp_wait_kernel<<<1, 32, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// One piece [begin, begin + n) of this rank's slice (n may be 0: publish only): AdamW, publication of the new
// parameters to every rank, zeros left in the consumed gradients, then release of row `row` of the "parameters
// published" flags on every rank. No wait: the consumer waits per row with mfb_dp_wait_published.
// piece_off: offset of the piece inside the rank's slice (index into lo / m / v / reduced, and into decay_end's frame).
int mfb_dp_adamw_publish(int world, int rank, int epoch, int row, long long begin, long long n, long long piece_off,
                         const long long* peer_param, const long long* peer_flags, void* lo, float* m, float* v,
                         float* reduced, const float* sumsq, int* skipped, long long decay_end, float lr, float beta1,
                         float beta2, float eps, float wd, float bc1, float bc2, float max_norm, float skip_threshold,
                         float grad_scale, int* status, cudaStream_t stream) {
  DpArgs a;
  if (fill_dp_args(&a, world, rank, epoch, begin, n, nullptr, peer_param, peer_flags, status)) return 1;
  if (row < 0 || row >= kDpBucketRows || (piece_off & 7)) {
    mfb_host::set_error("dp optimizer: publish row %d / piece offset %lld", row, piece_off);
    return 1;
  }
  DpAdamArgs h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.wd = wd; h.bc1 = bc1; h.bc2 = bc2;
  h.max_norm = max_norm; h.skip_threshold = skip_threshold; h.grad_scale = grad_scale;
  h.decay_end = decay_end - piece_off;          // the kernel indexes the piece from 0
  h.publish_row = row; h.zero_grads = 1;
  dp_adamw_kernel<<<dp_grid(n >> 3), kDpThreads, 0, stream>>>(a, h, (unsigned short*)lo + piece_off, m + piece_off,
                                                              v + piece_off, reduced + piece_off, sumsq, skipped);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Waits (one warp, bounded) until every rank has published row `row` of step `epoch`.
int mfb_dp_wait_published(int world, int rank, int epoch, int row, const long long* peer_flags, int* status,
                          cudaStream_t stream) {
  DpArgs a;
  if (fill_dp_args(&a, world, rank, epoch, 0, 0, nullptr, nullptr, peer_flags, status)) return 1;
  if (row < 0 || row >= kDpBucketRows) { mfb_host::set_error("dp optimizer: publish row %d", row); return 1; }
  dp_wait_published_row_kernel<<<1, 32, 0, stream>>>(a, row);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
