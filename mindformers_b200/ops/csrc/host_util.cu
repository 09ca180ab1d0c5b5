// Host-side utilities shared by all kernels: last-error string, tensor-map encoding.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace mfb_host {

static thread_local char g_err[512] = {0};

const char* last_error() { return g_err; }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, CUtensorMapDataType dt,
                 uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                 bool swizzle128) {
  // Driver entry points need a current context on the calling thread; worker threads (for
  // example an autograd backward thread) may have none yet. cudaFree(0) binds the primary one.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled entry point not available");
    return 1;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((ld * elem_bytes) & 15) != 0) {
    set_error("tensor map: base (%p) or row pitch (%llu B) not 16-byte aligned", base,
              (unsigned long long)(ld * elem_bytes));
    return 2;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed: %d (rows=%llu cols=%llu ld=%llu box=%ux%u eb=%d)", (int)r,
              (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows,
              box_cols, elem_bytes);
    return 3;
  }
  return 0;
}

}  // namespace mfb_host

extern "C" {

// Last error message of the calling thread ("" when none).
const char* mfb_last_error() { return mfb_host::last_error(); }

// ABI version of this library; bumped when an entry point changes its arguments.
int mfb_abi_version() { return 2; }

}  // extern "C"
