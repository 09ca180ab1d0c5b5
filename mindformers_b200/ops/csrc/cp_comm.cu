// Context-parallel K/V exchange over NVLink peer memory (sm_100a).
//
// Every rank of the context-parallel group holds K and V of its own sequence chunk(s) in a peer-mapped staging
// buffer [2][S_local][W] (W = kv_heads * head_dim). Two kernels move the data that ring attention would pass around:
//
//   cp_gather_kernel          all-gather by pulling: each rank reads every peer's staging buffer with 16-byte peer
//                             loads and writes K and V of the whole sequence, in natural token order, into its own
//                             memory, where the attention kernel reads them with TMA. The first CTA instructions
//                             announce "my staging buffer is complete" and wait (bounded) for the same announcement
//                             of all peers.
//   cp_reduce_scatter_kernel  the transpose for the backward pass: every rank holds partial dK / dV for the whole
//                             sequence [2][S_total][W] (bf16, peer-mapped); each rank sums the rows of its own
//                             chunk(s) over all peers in fp32, in rank order, and writes bf16.
//   cp_barrier_kernel         release + bounded wait, used after each of the two so that a staging buffer is not
//                             overwritten while a peer still reads it.
//
// Chunk layout: `zigzag` = 0: rank r owns tokens [r*S_local, (r+1)*S_local); `zigzag` = 1 (causal load balance):
// the sequence is cut into 2*cp chunks of S_local/2 tokens and rank r owns chunks r and 2*cp-1-r, in that order.
#include "common.cuh"

namespace mfb {

constexpr int kCpMaxRanks = 16;
constexpr int kCpThreads = 256;

struct CpArgs {
  int world, rank, epoch, phase, zigzag;
  long long s_local;   // tokens per rank
  int row_vecs;        // W * 2 / 16: 16-byte vectors per token row
  const uint4* stage_peer[kCpMaxRanks];   // [2][S_local][W] staging buffer of every rank
  uint4* full_peer[kCpMaxRanks];          // [2][S_total][W] full-sequence buffer of every rank (reduce-scatter source)
  int* flags_peer[kCpMaxRanks];           // [4][kCpMaxRanks] flag rows
  int* status;
};

__device__ __forceinline__ void cp_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int cp_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 cp_ld_cg(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ bool cp_wait_all(const int* flags, int world, int want, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint64_t t0 = globaltimer_ns();
    for (int p = 0; p < world && ok; ++p) {
      uint32_t it = 0;
      while (cp_ld_acquire_sys(flags + p) < want) {
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

// global token row of local row `i` of rank `r`
__device__ __forceinline__ long long cp_global_row(long long i, int r, int world, long long s_local, int zigzag) {
  if (!zigzag) return (long long)r * s_local + i;
  const long long h = s_local >> 1;
  return i < h ? (long long)r * h + i : (long long)(2 * world - 1 - r) * h + (i - h);
}

__global__ void __launch_bounds__(kCpThreads)
cp_gather_kernel(CpArgs a, uint4* __restrict__ full) {
  if (a.world > 1) {
    if (blockIdx.x == 0 && threadIdx.x < a.world)
      cp_st_release_sys(a.flags_peer[threadIdx.x] + a.phase * kCpMaxRanks + a.rank, a.epoch);
    if (!cp_wait_all(a.flags_peer[a.rank] + a.phase * kCpMaxRanks, a.world, a.epoch, a.status)) return;
  }
  const long long s_total = a.s_local * a.world;
  const long long per_rank = 2 * a.s_local * a.row_vecs;      // vectors in one staging buffer
  const long long total = per_rank * a.world;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int pr = (int)(i / per_rank);
    const int p = (a.rank + pr) % a.world;                    // own chunk first, then the peers round-robin
    const long long j = i - (long long)pr * per_rank;
    const int which = (int)(j / (a.s_local * a.row_vecs));    // 0 = K, 1 = V
    const long long rem = j - (long long)which * a.s_local * a.row_vecs;
    const long long row = rem / a.row_vecs;
    const int v = (int)(rem - row * a.row_vecs);
    const uint4 val = cp_ld_cg(a.stage_peer[p] + j);
    const long long grow = cp_global_row(row, p, a.world, a.s_local, a.zigzag);
    full[((long long)which * s_total + grow) * a.row_vecs + v] = val;
  }
}

__global__ void __launch_bounds__(kCpThreads)
cp_reduce_scatter_kernel(CpArgs a, uint4* __restrict__ out) {
  if (a.world > 1) {
    if (blockIdx.x == 0 && threadIdx.x < a.world)
      cp_st_release_sys(a.flags_peer[threadIdx.x] + a.phase * kCpMaxRanks + a.rank, a.epoch);
    if (!cp_wait_all(a.flags_peer[a.rank] + a.phase * kCpMaxRanks, a.world, a.epoch, a.status)) return;
  }
  const long long s_total = a.s_local * a.world;
  const long long total = 2 * a.s_local * a.row_vecs;
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < total;
       j += (long long)gridDim.x * blockDim.x) {
    const int which = (int)(j / (a.s_local * a.row_vecs));
    const long long rem = j - (long long)which * a.s_local * a.row_vecs;
    const long long row = rem / a.row_vecs;
    const int v = (int)(rem - row * a.row_vecs);
    const long long grow = cp_global_row(row, a.rank, a.world, a.s_local, a.zigzag);
    const long long src = ((long long)which * s_total + grow) * a.row_vecs + v;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int p = 0; p < a.world; ++p) {
      const uint4 q = cp_ld_cg(a.full_peer[p] + src);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) ho[i] = __float22bfloat162_rn(make_float2(acc[2 * i], acc[2 * i + 1]));
    out[j] = o;
  }
}

__global__ void cp_barrier_kernel(CpArgs a) {
  if (a.world <= 1) return;
  __threadfence_system();
  if (threadIdx.x < a.world) cp_st_release_sys(a.flags_peer[threadIdx.x] + a.phase * kCpMaxRanks + a.rank, a.epoch);
  cp_wait_all(a.flags_peer[a.rank] + a.phase * kCpMaxRanks, a.world, a.epoch, a.status);
}

}  // namespace mfb

extern "C" {
using namespace mfb;

int mfb_cp_flag_words() { return 4 * kCpMaxRanks; }

static int cp_fill(CpArgs* a, int world, int rank, int epoch, int phase, int zigzag, long long s_local, int width,
                   const long long* peer_stage, const long long* peer_full, const long long* peer_flags, int* status) {
  if (world < 1 || world > kCpMaxRanks || rank < 0 || rank >= world || phase < 0 || phase > 3) {
    mfb_host::set_error("cp exchange: world=%d rank=%d phase=%d out of range (max %d ranks)", world, rank, phase, kCpMaxRanks);
    return 1;
  }
  if ((width * 2) % 16 != 0 || s_local <= 0 || (zigzag && (s_local & 1))) {
    mfb_host::set_error("cp exchange: row width %d elements must be a multiple of 8; s_local=%lld", width, s_local);
    return 1;
  }
  a->world = world; a->rank = rank; a->epoch = epoch; a->phase = phase; a->zigzag = zigzag; a->s_local = s_local;
  a->row_vecs = width * 2 / 16; a->status = status;
  for (int p = 0; p < world; ++p) {
    a->stage_peer[p] = peer_stage ? reinterpret_cast<const uint4*>(peer_stage[p]) : nullptr;
    a->full_peer[p] = peer_full ? reinterpret_cast<uint4*>(peer_full[p]) : nullptr;
    a->flags_peer[p] = peer_flags ? reinterpret_cast<int*>(peer_flags[p]) : nullptr;
    if ((peer_stage && (peer_stage[p] & 15)) || (peer_full && (peer_full[p] & 15))) {
      mfb_host::set_error("cp exchange: buffers must be 16-byte aligned");
      return 1;
    }
  }
  return 0;
}

static inline int cp_grid(long long n) {
  long long b = (n + kCpThreads - 1) / kCpThreads;
  if (b > 148 * 8) b = 148 * 8;
  return b < 1 ? 1 : (int)b;
}

// full [2][S_local * world][width] (bf16, local) <- every rank's staging buffer [2][S_local][width]
int mfb_cp_gather(int world, int rank, int epoch, int phase, int zigzag, long long s_local, int width,
                  const long long* peer_stage, const long long* peer_flags, void* full, int* status, cudaStream_t stream) {
  CpArgs a;
  if (cp_fill(&a, world, rank, epoch, phase, zigzag, s_local, width, peer_stage, nullptr, peer_flags, status)) return 1;
  if (reinterpret_cast<uintptr_t>(full) & 15) { mfb_host::set_error("cp gather: output not 16-byte aligned"); return 1; }
  cp_gather_kernel<<<cp_grid(2 * s_local * a.row_vecs * world), kCpThreads, 0, stream>>>(a, (uint4*)full);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// out [2][S_local][width] (bf16, local) = sum over ranks of their [2][S_total][width] buffers, rows of this rank's chunk
int mfb_cp_reduce_scatter(int world, int rank, int epoch, int phase, int zigzag, long long s_local, int width,
                          const long long* peer_full, const long long* peer_flags, void* out, int* status,
                          cudaStream_t stream) {
  CpArgs a;
  if (cp_fill(&a, world, rank, epoch, phase, zigzag, s_local, width, nullptr, peer_full, peer_flags, status)) return 1;
  if (reinterpret_cast<uintptr_t>(out) & 15) { mfb_host::set_error("cp reduce-scatter: output not 16-byte aligned"); return 1; }
  cp_reduce_scatter_kernel<<<cp_grid(2 * s_local * a.row_vecs), kCpThreads, 0, stream>>>(a, (uint4*)out);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_cp_barrier(int world, int rank, int epoch, int phase, const long long* peer_flags, int* status,
                   cudaStream_t stream) {
  if (world <= 1) return 0;
  CpArgs a;
  if (cp_fill(&a, world, rank, epoch, phase, 0, 2, 8, nullptr, nullptr, peer_flags, status)) return 1;
  cp_barrier_kernel<<<1, 32, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
