// Device-side token selection and decode-state update (sm_100a).
//
// One launch per decode step, captured in the same CUDA graph as the model's forward pass, so that a run of decode
// steps replays without any host work: one CTA per sequence picks the next token from the sequence's logits row
// (greedy, or an exact sample from softmax(logits / temperature) by the Gumbel-max rule with a counter-based hash as
// the random source) and advances, in place, everything the next forward pass reads: the token id, its position,
// the context length and the slot of the paged KV cache that the token's key / value go to (looked up in the block
// table, whose blocks were reserved for the whole generation beforehand). The chosen token is also appended to a
// per-sequence history row that the host reads back once per burst of steps. A sequence that has produced an
// end-of-sequence token or reached its length limit is marked finished; from then on its state stops moving, its
// slot is -1 (the cache write skips it) and its history entries are -1.
#include "common.cuh"

namespace mfb {

constexpr int kAdvThreads = 1024;
constexpr int kAdvMaxEos = 8;

struct AdvanceArgs {
  const float* logits;   // [B, ld]
  int ld, vocab, batch;
  long long* tok;        // [B] token fed to the next step
  long long* pos;        // [B] its position
  int* lens;             // [B] context length of the next step (pos + 1)
  int* slots;            // [B] cache slot of the next step's key / value
  const int* table;      // [B, width] block ids
  int width, block;
  int* hist;             // [B, cap]
  int cap;
  int* count;            // [B] history entries written
  int* finished;         // [B]
  const int* limit;      // [B] total length (prompt + generated) at which the sequence stops
  const int* params;     // device words: [0..7] end-of-sequence ids (-1: unused), [8] inverse temperature (float
                         // bits, 0: greedy), [10..11] seed. Read from memory so that a captured launch can be
                         // replayed with other sampling settings.
};

__device__ __forceinline__ float gumbel_noise(unsigned long long seed, unsigned int step, unsigned int row,
                                              unsigned int col) {
  // splitmix64 of (seed, step, row, col) -> uniform in (0, 1) -> -log(-log(u))
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (static_cast<unsigned long long>(step) + 1);
  z ^= (static_cast<unsigned long long>(row) << 32) | col;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  const float u = (static_cast<float>(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
  return -__logf(-__logf(u));
}

__global__ void __launch_bounds__(kAdvThreads) decode_advance_kernel(const AdvanceArgs a) {
  const int b = blockIdx.x;
  const int c = a.count[b];
  const bool was_finished = a.finished[b] != 0;
  const float inv_temp = __int_as_float(a.params[8]);
  const unsigned long long seed = *reinterpret_cast<const unsigned long long*>(a.params + 10);
  __shared__ float s_val[kAdvThreads / 32];
  __shared__ int s_idx[kAdvThreads / 32];
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  if (!was_finished) {
    const float* row = a.logits + static_cast<size_t>(b) * a.ld;
    for (int i = threadIdx.x; i < a.vocab; i += kAdvThreads) {
      float v = row[i];
      if (inv_temp > 0.f) v = v * inv_temp + gumbel_noise(seed, static_cast<unsigned int>(c), b, i);
      if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }    // NaN never wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = best_i; }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (was_finished) {
    if (c < a.cap) a.hist[static_cast<size_t>(b) * a.cap + c] = -1;
    a.count[b] = c + 1;
    return;
  }
  for (int w = 0; w < kAdvThreads / 32; ++w)
    if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) { best = s_val[w]; best_i = s_idx[w]; }
  if (best_i >= a.vocab) best_i = 0;              // a row of NaN: still a valid token id
  const long long p = a.pos[b] + 1;               // position of the token just chosen
  const int len = static_cast<int>(p) + 1;        // sequence length with it
  if (c < a.cap) a.hist[static_cast<size_t>(b) * a.cap + c] = best_i;
  a.count[b] = c + 1;
  bool stop = len >= a.limit[b] || p / a.block >= a.width;
  for (int e = 0; e < kAdvMaxEos; ++e) stop = stop || best_i == a.params[e];
  if (stop) {
    a.finished[b] = 1;
    a.slots[b] = -1;
    return;
  }
  a.tok[b] = best_i;
  a.pos[b] = p;
  a.lens[b] = len;
  const int blk = a.table[static_cast<size_t>(b) * a.width + p / a.block];
  a.slots[b] = blk < 0 ? -1 : blk * a.block + static_cast<int>(p % a.block);
}

}  // namespace mfb

extern "C" {
using namespace mfb;

// Picks the next token of every sequence and advances the decode state in place (see the file comment).
// params: 12 device words, see AdvanceArgs. Inverse temperature 0 selects the arg-max; otherwise a sample at that
// inverse temperature, reproducible from (seed, history index, row).
int mfb_decode_advance(const float* logits, int ld, int vocab, int batch, long long* tok, long long* pos, int* lens,
                       int* slots, const int* table, int width, int block, int* hist, int cap, int* count,
                       int* finished, const int* limit, const int* params, cudaStream_t stream) {
  if (batch < 1 || vocab < 1 || ld < vocab || block < 1 || width < 1 || cap < 1 || params == nullptr) {
    mfb_host::set_error("decode advance: batch %d vocab %d ld %d block %d width %d cap %d", batch, vocab, ld, block,
                        width, cap);
    return 1;
  }
  AdvanceArgs a;
  a.logits = logits; a.ld = ld; a.vocab = vocab; a.batch = batch; a.tok = tok; a.pos = pos; a.lens = lens;
  a.slots = slots; a.table = table; a.width = width; a.block = block; a.hist = hist; a.cap = cap; a.count = count;
  a.finished = finished; a.limit = limit; a.params = params;
  decode_advance_kernel<<<batch, kAdvThreads, 0, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

}  // extern "C"
