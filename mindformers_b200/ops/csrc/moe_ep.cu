// Expert-parallel MoE token exchange fused with the router permutation, over NVLink peer memory (sm_100a).
//
// Every rank of the expert-parallel group owns E_local experts and a row buffer [rows_cap, H] in peer-mapped
// ("symmetric") memory. A token copy (t, j) routed to global expert e lives in row
//     seg_start[e] + sum_{r' < src} count[r'][e] + (rank of the copy among the source's copies for e)
// of the buffer of rank e / E_local; expert segments are padded to multiples of 128 rows so that the grouped
// tcgen05 GEMM maps whole row blocks to experts. Nothing is sized or indexed on the host:
//
//   moe_rank_kernel     one CTA per global expert: stable rank of every copy within its expert + counts
//   moe_plan_kernel     one CTA: writes this rank's counts into every peer's table (peer stores + release flag),
//                       waits (bounded) for all peers' rows, then derives segment starts, this rank's write
//                       offsets, and the grouped-GEMM plan (group offsets, block -> expert map, block count)
//   moe_scatter_kernel  "permute + all-to-all send": one warp per copy stores the (optionally weighted) token row
//                       straight into the destination rank's buffer with 16-byte peer stores; padding rows of
//                       the local buffer are cleared by the same launch
//   moe_barrier_kernel  one CTA: release "my writes/results are complete", wait (bounded) for all peers
//   moe_gather_kernel   "all-to-all receive + unpermute": out[t] = sum_j w[t,j] * peer_buf[rank_j][row_j] with
//                       16-byte peer loads and fp32 accumulation in j order; optionally also the dot products
//                       <g[t], row> that the backward pass needs for d(probs)
//
// With a single rank the same kernels are the local permute / unpermute (no flags are touched).
// Flags carry a per-call epoch that the kernels take from a counter in device memory and advance themselves (every
// rank runs the same sequence of calls, so the counters agree), which lets a CUDA graph replay them; every wait is
// bounded and reports kStatusPeerFlagTimeout in the status word.
#include "common.cuh"

namespace mfb {

constexpr int kMoeMaxRanks = 8;
constexpr int kMoeBlock = 128;      // row block of the grouped GEMM
constexpr int kMoeMaxExperts = 512;
constexpr int kStatusMoeOverflow = 6;

__device__ __forceinline__ void moe_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int moe_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 moe_ld_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// thread 0 waits until flags[0..world) >= want
__device__ bool moe_wait_all(const int* flags, int world, int want, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint64_t t0 = globaltimer_ns();
    for (int p = 0; p < world && ok; ++p) {
      uint32_t it = 0;
      while (moe_ld_acquire_sys(flags + p) < want) {
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

// ---------------------------------------------------------------------------------------------------------------
// rank of each copy within its expert (stable in copy order) and the per-expert counts
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_rank_kernel(const long long* __restrict__ ids, int n, int* __restrict__ rank_in_e, int* __restrict__ counts) {
  const int e = blockIdx.x;
  __shared__ int warp_tot[32];
  __shared__ int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const bool hit = i < n && (int)ids[i] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_tot[warp] = __popc(m);
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (hit) rank_in_e[i] = running + before + __popc(m & ((1u << lane) - 1u));
    __syncthreads();
    if (threadIdx.x == 0) {
      int t = 0;
      for (int w = 0; w < nwarps; ++w) t += warp_tot[w];
      running += t;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = running;
}

// ---------------------------------------------------------------------------------------------------------------
// count exchange + layout plan
// ---------------------------------------------------------------------------------------------------------------
struct MoePlanArgs {
  int world, rank, E, E_local, rows_cap, nblocks_cap;
  int* epoch_ctr;                    // device counter of this rank: the call uses *epoch_ctr + 1 and stores it back
  const int* counts;                 // [E] of this rank
  int* table_peer[kMoeMaxRanks];     // [world][E + 1] table of every rank: row r = counts of rank r, then its rows_cap
  int* owner_cap;                    // out [kMoeMaxRanks]: rows_cap of every rank's buffer
  int* flags_peer[kMoeMaxRanks];     // [3][kMoeMaxRanks] flag rows: 0 = counts, 1 / 2 = barriers
  int* write_base;                   // out [E]: first row (in the owner's buffer) for this rank's copies of e
  int* group_offsets;                // out [E_local + 1]: padded segment starts of the local experts
  int* seg_fill;                     // out [E_local]: rows actually used in each local segment
  int* block_group;                  // out [nblocks_cap]
  int* num_blocks;                   // out [1]
  int* status;
};

__global__ void __launch_bounds__(kMoeMaxExperts)
moe_plan_kernel(MoePlanArgs a) {
  __shared__ int tot[kMoeMaxExperts];     // copies per global expert over all sources
  __shared__ int mine[kMoeMaxExperts];    // copies from sources before this rank
  __shared__ int seg[kMoeMaxExperts + 1];
  const int e = threadIdx.x;
  int* table_local = a.table_peer[a.rank];
  if (a.world > 1) {
    for (int p = 0; p < a.world; ++p) {
      if (e < a.E) a.table_peer[p][a.rank * (a.E + 1) + e] = a.counts[e];
      if (e == 0) a.table_peer[p][a.rank * (a.E + 1) + a.E] = a.rows_cap;
    }
    __shared__ int s_epoch;
    if (e == 0) s_epoch = *a.epoch_ctr + 1;
    __threadfence_system();
    __syncthreads();
    const int epoch = s_epoch;
    if (e < a.world) moe_st_release_sys(a.flags_peer[e] + a.rank, epoch);
    moe_wait_all(a.flags_peer[a.rank], a.world, epoch, a.status);
    if (e == 0) *a.epoch_ctr = epoch;
  }
  if (e < a.E) {
    int t = 0, b = 0;
    for (int r = 0; r < a.world; ++r) {
      const int c = a.world > 1 ? moe_ld_acquire_sys(table_local + r * (a.E + 1) + e) : a.counts[e];
      if (r < a.rank) b += c;
      t += c;
    }
    tot[e] = t;
    mine[e] = b;
  }
  if (e < kMoeMaxRanks)
    a.owner_cap[e] = e >= a.world ? 0 : (a.world > 1 ? moe_ld_acquire_sys(table_local + e * (a.E + 1) + a.E) : a.rows_cap);
  __syncthreads();
  // padded segment starts per owner rank (every rank computes all of them: they are the senders' bases)
  if (e < a.world) {
    int off = 0;
    for (int le = 0; le < a.E_local; ++le) {
      const int ge = e * a.E_local + le;
      seg[ge] = off;
      off += (tot[ge] + kMoeBlock - 1) / kMoeBlock * kMoeBlock;
    }
    if (e == a.rank) {
      seg[a.E] = off;
      // overflow has a word of its own right behind the wait status, so neither can hide the other
      if (off > a.rows_cap && a.status) atomicExch(a.status + 1, 1);
    }
  }
  __syncthreads();
  if (e < a.E) a.write_base[e] = seg[e] + mine[e];
  // on overflow every consumer of the plan (grouped GEMM row blocks, per-expert weight-gradient ranges) stays inside
  // the buffer: segments are cut at the last whole block that fits
  int total = seg[a.E];
  if (total > a.rows_cap) total = a.rows_cap / kMoeBlock * kMoeBlock;
  if (e < a.E_local) {
    const int ge = a.rank * a.E_local + e;
    const int start = seg[ge] < total ? seg[ge] : total;
    int fill = tot[ge];
    if (fill > total - start) fill = total - start;
    a.group_offsets[e] = start;
    a.seg_fill[e] = fill;
  }
  if (e == 0) {
    a.group_offsets[a.E_local] = total;
    a.num_blocks[0] = total / kMoeBlock;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < a.nblocks_cap; b += blockDim.x) {
    const int row = b * kMoeBlock;
    int g = a.E_local - 1;
    for (int le = 0; le < a.E_local; ++le) {
      const int ge = a.rank * a.E_local + le;
      const int end = seg[ge] + (tot[ge] + kMoeBlock - 1) / kMoeBlock * kMoeBlock;
      if (row < end) { g = le; break; }
    }
    a.block_group[b] = g;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// scatter (permute + send) and gather (receive + unpermute)
// ---------------------------------------------------------------------------------------------------------------
struct MoeMoveArgs {
  int world, rank, T, k, H, E_local, rows_cap;
  const long long* ids;       // [T, k]
  const int* rank_in_e;       // [T * k]
  const int* write_base;      // [E]
  const int* owner_cap;       // [kMoeMaxRanks] rows of every rank's buffer
  __nv_bfloat16* buf_peer[kMoeMaxRanks];  // row buffer [rows_cap, H] of every rank
  const float* weights;       // [T, k] or null
  int* dest_row;              // [T * k] out (scatter) / in (gather): row in the owner's buffer, -1 = dropped
  const int* group_offsets;   // local plan (for the padding rows)
  const int* seg_fill;
  int* status;
};

__global__ void __launch_bounds__(256)
moe_scatter_kernel(MoeMoveArgs a, const __nv_bfloat16* __restrict__ x) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long gw = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * warps_per_cta;
  const int n = a.T * a.k;
  const int vecs = a.H >> 3;
  // one work item = 128 vectors (2 KB) of one copy: a decode batch of a few hundred copies still fills the GPU
  const int chunks = (vecs + 127) >> 7;
  for (long long item = gw; item < (long long)n * chunks; item += nwarps) {
    const long long c = item / chunks;
    const int v_lo = (int)(item - c * chunks) << 7;
    const int t = (int)(c / a.k);
    const int e = (int)a.ids[c];
    const int owner = e / a.E_local;
    const int row = a.write_base[e] + a.rank_in_e[c];
    const bool ok = e >= 0 && owner < a.world && row >= 0 && row < a.owner_cap[owner];
    if (lane == 0 && v_lo == 0) a.dest_row[c] = ok ? row : -1;
    if (!ok) continue;
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * a.H);
    uint4* dst = reinterpret_cast<uint4*>(a.buf_peer[owner] + (long long)row * a.H);
    const float w = a.weights ? a.weights[c] : 1.f;
    uint4 q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v_lo + u * 32 + lane;
      if (v < vecs) q[u] = src[v];
    }
    if (a.weights) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q[u]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(h[i]);
          f.x *= w; f.y *= w;
          h[i] = __float22bfloat162_rn(f);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v_lo + u * 32 + lane;
      if (v < vecs) dst[v] = q[u];
    }
  }
  // padding rows of the local segments start as zero: the weight-gradient GEMM sums over them. Without a plan
  // (inference: rows are independent and padding rows are never gathered) they are left as they are.
  if (a.group_offsets) {
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int le = 0; le < a.E_local; ++le) {
      const int first = a.group_offsets[le] + a.seg_fill[le];
      int last = a.group_offsets[le + 1];
      if (last > a.rows_cap) last = a.rows_cap;
      for (long long r = first + gw; r < last; r += nwarps) {
        uint4* dst = reinterpret_cast<uint4*>(a.buf_peer[a.rank] + r * a.H);
        for (int v = lane; v < vecs; v += 32) dst[v] = z;
      }
    }
  }
  __threadfence_system();
}

struct MoeBarrierArgs {
  int world, rank, phase;
  int* epoch_ctr;
  int* flags_peer[kMoeMaxRanks];
  int* status;
};

__global__ void moe_barrier_kernel(MoeBarrierArgs a) {
  if (a.world <= 1) return;
  __shared__ int s_epoch;
  if (threadIdx.x == 0) s_epoch = *a.epoch_ctr + 1;
  __threadfence_system();
  __syncthreads();
  const int epoch = s_epoch;
  if (threadIdx.x < a.world)
    moe_st_release_sys(a.flags_peer[threadIdx.x] + a.phase * kMoeMaxRanks + a.rank, epoch);
  moe_wait_all(a.flags_peer[a.rank] + a.phase * kMoeMaxRanks, a.world, epoch, a.status);
  if (threadIdx.x == 0) *a.epoch_ctr = epoch;
}

// out[t] = sum_j w[t,j] * row(t,j)  (w == null: plain sum); dots[t,j] = <g[t], row(t,j)> when g is given
__global__ void __launch_bounds__(256)
moe_gather_kernel(MoeMoveArgs a, __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ g,
                  float* __restrict__ dots) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long gw = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * warps_per_cta;
  const int vecs = a.H >> 3;
  if (!g) {
    // forward / inference: one work item = 32 vectors of one token, the k rows are fetched four at a time
    if (!out) return;
    const int chunks = (vecs + 31) >> 5;
    for (long long item = gw; item < (long long)a.T * chunks; item += nwarps) {
      const long long t = item / chunks;
      const int v = ((int)(item - t * chunks) << 5) + lane;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j0 = 0; j0 < a.k; j0 += 4) {
        uint4 q[4];
        float w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          w[u] = 0.f;
          q[u] = make_uint4(0, 0, 0, 0);
          const int j = j0 + u;
          if (j < a.k) {
            const long long c = t * a.k + j;
            const int row = a.dest_row[c];
            const int owner = (int)a.ids[c] / a.E_local;
            if (row >= 0 && owner >= 0 && owner < a.world && v < vecs) {
              q[u] = moe_ld_cg(a.buf_peer[owner] + (long long)row * a.H + 8 * v);
              w[u] = a.weights ? a.weights[c] : 1.f;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q[u]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            acc[2 * i] += w[u] * f.x;
            acc[2 * i + 1] += w[u] * f.y;
          }
        }
      }
      if (v < vecs) {
        uint4 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __float22bfloat162_rn(make_float2(acc[2 * i], acc[2 * i + 1]));
        reinterpret_cast<uint4*>(out + t * a.H)[v] = q;
      }
    }
    return;
  }
  for (long long t = gw; t < a.T; t += nwarps) {
    for (int v0 = 0; v0 < vecs; v0 += 32) {
      const int v = v0 + lane;
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      float gv[8];
      if (g && v < vecs) {
        const uint4 q = reinterpret_cast<const uint4*>(g + t * a.H)[v];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); gv[2 * i] = f.x; gv[2 * i + 1] = f.y; }
      }
      // the k rows of a token sit on up to k peers: four loads in flight before the first is used, since one peer
      // load takes microseconds to return
      for (int j0 = 0; j0 < a.k; j0 += 4) {
        uint4 q4[4];
        bool have[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          have[u] = false;
          const int j = j0 + u;
          if (j < a.k) {
            const long long c = t * a.k + j;
            const int row = a.dest_row[c];
            const int owner = (int)a.ids[c] / a.E_local;
            if (row >= 0 && owner >= 0 && owner < a.world && v < vecs) {
              q4[u] = moe_ld_cg(a.buf_peer[owner] + (long long)row * a.H + 8 * v);
              have[u] = true;
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = j0 + u;
          if (j >= a.k) break;
          const long long c = t * a.k + j;
          float dot = 0.f;
          if (have[u]) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q4[u]);
            const float w = a.weights ? a.weights[c] : 1.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(h[i]);
              acc[2 * i] += w * f.x;
              acc[2 * i + 1] += w * f.y;
              if (g) dot += gv[2 * i] * f.x + gv[2 * i + 1] * f.y;
            }
          }
          if (g) {
            dot = warp_sum(dot);
            if (lane == 0) {
              if (v0 == 0) dots[c] = dot; else dots[c] += dot;
            }
          }
        }
      }
      if (out && v < vecs) {
        uint4 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __float22bfloat162_rn(make_float2(acc[2 * i], acc[2 * i + 1]));
        reinterpret_cast<uint4*>(out + t * a.H)[v] = q;
      }
    }
  }
}

}  // namespace mfb

extern "C" {
using namespace mfb;

int mfb_moe_flag_words() { return 3 * kMoeMaxRanks; }

static int moe_check(int world, int rank, int E, int E_local, int H) {
  if (world < 1 || world > kMoeMaxRanks || rank < 0 || rank >= world || E != E_local * world || E > kMoeMaxExperts) {
    mfb_host::set_error("moe: world=%d rank=%d E=%d E_local=%d not supported (max %d ranks, %d experts)", world, rank, E,
                        E_local, kMoeMaxRanks, kMoeMaxExperts);
    return 1;
  }
  if (H % 8 != 0) {
    mfb_host::set_error("moe: hidden size %d must be a multiple of 8", H);
    return 1;
  }
  return 0;
}

// ids [T*k] int64 -> rank_in_e [T*k] int32, counts [E] int32
int mfb_moe_rank(const long long* ids, int n, int E, int* rank_in_e, int* counts, cudaStream_t stream) {
  if (E < 1 || E > kMoeMaxExperts) { mfb_host::set_error("moe: E=%d out of range", E); return 1; }
  moe_rank_kernel<<<E, 1024, 0, stream>>>(ids, n, rank_in_e, counts);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// peer_tables / peer_flags: host arrays of `world` device addresses.
int mfb_moe_plan(int world, int rank, int* epoch_ctr, int E, int E_local, int rows_cap, const int* counts,
                 const long long* peer_tables, const long long* peer_flags, int* write_base, int* owner_cap,
                 int* group_offsets, int* seg_fill, int* block_group, int* num_blocks, int* status,
                 cudaStream_t stream) {
  if (moe_check(world, rank, E, E_local, 8)) return 1;
  MoePlanArgs a;
  if (world > 1 && !epoch_ctr) { mfb_host::set_error("moe plan: the epoch counter is missing"); return 1; }
  a.world = world; a.rank = rank; a.epoch_ctr = epoch_ctr; a.E = E; a.E_local = E_local; a.rows_cap = rows_cap;
  a.nblocks_cap = rows_cap / kMoeBlock; a.counts = counts;
  for (int p = 0; p < world; ++p) {
    a.table_peer[p] = peer_tables ? reinterpret_cast<int*>(peer_tables[p]) : nullptr;
    a.flags_peer[p] = peer_flags ? reinterpret_cast<int*>(peer_flags[p]) : nullptr;
  }
  a.write_base = write_base; a.owner_cap = owner_cap; a.group_offsets = group_offsets; a.seg_fill = seg_fill; a.block_group = block_group;
  a.num_blocks = num_blocks; a.status = status;
  moe_plan_kernel<<<1, kMoeMaxExperts, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

static int aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static void fill_move(MoeMoveArgs* a, int world, int rank, int T, int k, int H, int E_local, int rows_cap,
                      const long long* ids, const int* rank_in_e, const int* write_base, const int* owner_cap,
                      const long long* peer_bufs,
                      const float* weights, int* dest_row, const int* group_offsets, const int* seg_fill, int* status) {
  a->world = world; a->rank = rank; a->T = T; a->k = k; a->H = H; a->E_local = E_local; a->rows_cap = rows_cap;
  a->ids = ids; a->rank_in_e = rank_in_e; a->write_base = write_base; a->owner_cap = owner_cap; a->weights = weights;
  a->dest_row = dest_row;
  a->group_offsets = group_offsets; a->seg_fill = seg_fill; a->status = status;
  for (int p = 0; p < world; ++p) a->buf_peer[p] = reinterpret_cast<__nv_bfloat16*>(peer_bufs[p]);
}

int mfb_moe_scatter(int world, int rank, int T, int k, int H, int E_local, int rows_cap, const void* x,
                    const long long* ids, const int* rank_in_e, const int* write_base, const int* owner_cap,
                    const long long* peer_bufs, const float* weights, int* dest_row, const int* group_offsets,
                    const int* seg_fill, int* status, cudaStream_t stream) {
  if (moe_check(world, rank, E_local * world, E_local, H)) return 1;
  for (int p = 0; p < world; ++p)
    if (!aligned16(reinterpret_cast<const void*>(peer_bufs[p])) || !aligned16(x)) {
      mfb_host::set_error("moe scatter: row buffers and the source must be 16-byte aligned");
      return 1;
    }
  MoeMoveArgs a;
  fill_move(&a, world, rank, T, k, H, E_local, rows_cap, ids, rank_in_e, write_base, owner_cap, peer_bufs, weights,
            dest_row, group_offsets, seg_fill, status);
  moe_scatter_kernel<<<148 * 4, 256, 0, stream>>>(a, (const __nv_bfloat16*)x);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_moe_barrier(int world, int rank, int* epoch_ctr, int phase, const long long* peer_flags, int* status,
                    cudaStream_t stream) {
  if (world <= 1) return 0;
  if (world > kMoeMaxRanks || phase < 1 || phase > 2 || !epoch_ctr) { mfb_host::set_error("moe barrier: bad world/phase/counter"); return 1; }
  MoeBarrierArgs a;
  a.world = world; a.rank = rank; a.epoch_ctr = epoch_ctr; a.phase = phase; a.status = status;
  for (int p = 0; p < world; ++p) a.flags_peer[p] = reinterpret_cast<int*>(peer_flags[p]);
  moe_barrier_kernel<<<1, 32, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int mfb_moe_gather(int world, int rank, int T, int k, int H, int E_local, int rows_cap, void* out,
                   const long long* ids, const int* dest_row, const long long* peer_bufs, const float* weights,
                   const void* g, float* dots, int* status, cudaStream_t stream) {
  if (moe_check(world, rank, E_local * world, E_local, H)) return 1;
  for (int p = 0; p < world; ++p)
    if (!aligned16(reinterpret_cast<const void*>(peer_bufs[p])) || !aligned16(out) || !aligned16(g)) {
      mfb_host::set_error("moe gather: row buffers, the output and the gradient must be 16-byte aligned");
      return 1;
    }
  MoeMoveArgs a;
  fill_move(&a, world, rank, T, k, H, E_local, rows_cap, ids, nullptr, nullptr, nullptr, peer_bufs, weights,
            const_cast<int*>(dest_row), nullptr, nullptr, status);
  moe_gather_kernel<<<148 * 4, 256, 0, stream>>>(a, (__nv_bfloat16*)out, (const __nv_bfloat16*)g, dots);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
