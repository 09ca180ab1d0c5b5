// Low-latency all-reduce of small bf16 tensors over NVLink peer memory (sm_100a): one launch, no flags, no barrier.
//
// For the row-parallel layers of tensor-parallel decoding the message is a few hundred kilobytes and the cost of an
// all-reduce is latency: a flag-based exchange pays a system-scope release / acquire round per hop. Here the DATA
// carries its own arrival: every rank's receive buffer is pre-filled with a sentinel (bf16 negative zero, 0x8000, which
// the sender never transmits: it sends +0 instead), each rank stores its whole contribution with 16-byte stores into
// slot [its rank] of every peer's buffer, and then polls its own buffer vector by vector until no lane holds the
// sentinel, adding the contributions in rank order (fp32), so every rank computes the same bits.
//
// Three generations of the receive buffer rotate: call k receives in generation k % 3 and resets generation
// (k + 2) % 3 (the one call k - 1 used) to the sentinel. A peer can be at most one call ahead (it cannot finish call
// k + 1 without this rank's data of call k + 1), so what it writes meanwhile goes to generation (k + 1) % 3, which
// was reset during call k - 1. The call counter and the sizes of the last calls live in device memory and are
// advanced by the kernel itself: the launch has no host-side epoch and can be captured in a CUDA graph and replayed.
//
// Every poll is bounded (MFB_WAIT_LIMIT_NS): on a timeout the status word is set and the kernel finishes.
#include "common.cuh"

namespace mfb {
namespace llar {

constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;
constexpr uint32_t kSentinel2 = 0x80008000u;   // two bf16 negative zeros

struct Args {
  int world, rank;
  long long n_vec;                 // 16-byte vectors (8 bf16) of this call
  long long cap_vec;               // vectors per (generation, source rank) slot
  const uint4* in;
  uint4* out;
  uint4* peer_buf[kMaxRanks];      // every rank's receive buffer [3][world][cap_vec]
  int* state;                      // device words: [0] call counter, [1..3] vectors used per generation, [4] ticket
  int* status;
};

__device__ __forceinline__ uint32_t no_neg_zero(uint32_t v) {
  if ((v & 0xffffu) == 0x8000u) v &= 0xffff0000u;
  if ((v >> 16) == 0x8000u) v &= 0x0000ffffu;
  return v;
}
__device__ __forceinline__ bool has_sentinel(uint32_t v) {
  return (v & 0xffffu) == 0x8000u || (v >> 16) == 0x8000u;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__global__ void __launch_bounds__(kThreads) ll_allreduce_kernel(const Args a) {
  const int k = *reinterpret_cast<volatile int*>(a.state);
  const int gen = k % 3, clr = (k + 2) % 3;
  const long long n_clr = a.state[1 + clr];
  const long long stride = static_cast<long long>(gridDim.x) * kThreads;
  const long long tid = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  // ---- send: this rank's contribution into slot [rank] of generation `gen` on every rank (own copy included) ----
  for (long long i = tid; i < a.n_vec; i += stride) {
    uint4 v = a.in[i];
    v.x = no_neg_zero(v.x); v.y = no_neg_zero(v.y); v.z = no_neg_zero(v.z); v.w = no_neg_zero(v.w);
    const long long off = (static_cast<long long>(gen) * a.world + a.rank) * a.cap_vec + i;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p)
      if (p < a.world) st_volatile_v4(a.peer_buf[(a.rank + p) % a.world] + off, v);
  }
  // ---- reset the generation that the previous call used ----
  uint4* mine = a.peer_buf[a.rank];
  const uint4 fill = make_uint4(kSentinel2, kSentinel2, kSentinel2, kSentinel2);
  for (int r = 0; r < a.world; ++r)
    for (long long i = tid; i < n_clr; i += stride)
      mine[(static_cast<long long>(clr) * a.world + r) * a.cap_vec + i] = fill;
  // ---- receive: poll every source's vector until it is complete, add in rank order ----
  bool ok = true;
  const uint64_t t0 = globaltimer_ns();
  for (long long i = tid; i < a.n_vec; i += stride) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < a.world; ++r) {
      const uint4* src = mine + (static_cast<long long>(gen) * a.world + r) * a.cap_vec + i;
      uint4 v = ld_volatile_v4(src);
      uint32_t spins = 0;
      while (ok && (has_sentinel(v.x) || has_sentinel(v.y) || has_sentinel(v.z) || has_sentinel(v.w))) {
        if (((++spins) & 0xff) == 0 && globaltimer_ns() - t0 > MFB_WAIT_LIMIT_NS) {
          ok = false;
          if (a.status) atomicCAS(a.status, 0, kStatusPeerFlagTimeout);
          break;
        }
        v = ld_volatile_v4(src);
      }
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    a.out[i] = o;
  }
  // ---- the last CTA advances the call counter and records this call's size for the reset two calls later ----
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(a.state + 4, 1) == static_cast<int>(gridDim.x) - 1) {
      a.state[1 + gen] = static_cast<int>(a.n_vec);
      a.state[4] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(a.state) = k + 1;
    }
  }
}

__global__ void ll_fill_kernel(uint4* buf, long long n_vec) {
  const uint4 fill = make_uint4(kSentinel2, kSentinel2, kSentinel2, kSentinel2);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    buf[i] = fill;
}

}  // namespace llar
}  // namespace mfb

extern "C" {
using namespace mfb;

// Bytes of the receive buffer of one rank for messages of up to max_bytes, and the number of state words.
long long mfb_ll_allreduce_buffer_bytes(int world, long long max_bytes) {
  const long long cap_vec = (max_bytes + 15) / 16;
  return 3ll * world * cap_vec * 16;
}
int mfb_ll_allreduce_state_words() { return 8; }

// Fills a receive buffer with the sentinel (once, before the first call; every rank, then a barrier on the host).
int mfb_ll_allreduce_init(void* buf, long long bytes, cudaStream_t stream) {
  llar::ll_fill_kernel<<<296, 256, 0, stream>>>(reinterpret_cast<uint4*>(buf), bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// out = sum over ranks of in (bf16, `bytes` a multiple of 16 and at most max_bytes of the buffer). peer_bufs: host
// array of `world` device addresses of the ranks' receive buffers (own at index rank); state: this rank's words.
int mfb_ll_allreduce(const void* in, void* out, long long bytes, long long max_bytes, int world, int rank,
                     const long long* peer_bufs, int* state, int* status, cudaStream_t stream) {
  if (world < 1 || world > llar::kMaxRanks || rank < 0 || rank >= world || bytes <= 0 || (bytes & 15) || bytes > max_bytes ||
      (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) {
    mfb_host::set_error("ll_allreduce: world %d rank %d bytes %lld (max %lld) or misaligned pointers", world, rank, bytes,
                        max_bytes);
    return 1;
  }
  llar::Args a;
  a.world = world; a.rank = rank; a.n_vec = bytes / 16; a.cap_vec = (max_bytes + 15) / 16;
  a.in = reinterpret_cast<const uint4*>(in); a.out = reinterpret_cast<uint4*>(out);
  for (int p = 0; p < world; ++p) a.peer_buf[p] = reinterpret_cast<uint4*>(peer_bufs[p]);
  a.state = state; a.status = status;
  long long blocks = (a.n_vec + llar::kThreads - 1) / llar::kThreads;
  if (blocks > 296) blocks = 296;
  llar::ll_allreduce_kernel<<<static_cast<int>(blocks), llar::kThreads, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
