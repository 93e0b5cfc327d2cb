// Host-side helpers shared by the entry points: error text, argument checks,
// TMA tensor-map encoding (driver entry point resolved at run time, so the
// library links against the CUDA runtime only).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/castle_b200.h"
#include "../../include/castle_b200_diag.h"

namespace castle {

char* last_error_buf();  // thread-local, defined in api.cu

struct KernelEvents { cudaEvent_t start = nullptr, stop = nullptr; };
KernelEvents& kernel_events(int which);  // process-wide, defined in api.cu
inline void ev_start(int which, cudaStream_t st) { auto& e = kernel_events(which); if (e.start) cudaEventRecord(e.start, st); }
inline void ev_stop(int which, cudaStream_t st) { auto& e = kernel_events(which); if (e.stop) cudaEventRecord(e.stop, st); }

inline int reject(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return -1;
}

inline int cuda_fail(cudaError_t e, const char* what) {
  snprintf(last_error_buf(), 512, "%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}

inline int elem_size(int dtype) { return dtype == CASTLE_F32 ? 4 : 2; }

inline bool tensor_ok(const castle_tensor_t* t, int dtype, const char* name, int* rc) {
  if (!t || !t->ptr) { *rc = reject("%s: null tensor", name); return false; }
  int es = elem_size(dtype);
  if (((uintptr_t)t->ptr) % 16) { *rc = reject("%s: base pointer not 16-byte aligned", name); return false; }
  if ((t->stride_b * es) % 16 || (t->stride_h * es) % 16 || (t->stride_n * es) % 16) {
    *rc = reject("%s: strides must be multiples of 16 bytes", name);
    return false;
  }
  return true;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline encode_tiled_fn get_encode_fn() {
  static encode_tiled_fn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (encode_tiled_fn)p;
  }
  return fn;
}

// Tensor map over a 16-bit (batch, head, position, dim_head) tensor: dims (d, N, H, B),
// box (64, box_rows, 1, 1), 128-byte swizzle, out-of-range rows read as zero.
inline int make_tmap_16bit(CUtensorMap* m, const castle_tensor_t* t, int dtype, int B, int H, int N, int D,
                           int box_rows, const char* name) {
  encode_tiled_fn fn = get_encode_fn();
  if (!fn) return reject("cuTensorMapEncodeTiled is not available from this driver");
  // The encoder is a driver call and needs a current context on the calling thread; a thread
  // that has made no runtime call yet (an autograd worker, say) has none until one is made.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)B};
  // a size-1 dimension may carry any stride; give it a legal one
  cuuint64_t sn = (cuuint64_t)t->stride_n * 2, sh = (cuuint64_t)t->stride_h * 2, sb = (cuuint64_t)t->stride_b * 2;
  if (N == 1 || sn == 0) sn = (cuuint64_t)D * 2;
  if (H == 1 || sh == 0) sh = sn * (cuuint64_t)N;
  if (B == 1 || sb == 0) sb = sh * (cuuint64_t)H;
  cuuint64_t strides[3] = {sn, sh, sb};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(m, dtype == CASTLE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  t->ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return reject("%s: cuTensorMapEncodeTiled failed (CUresult %d)", name, (int)r);
  return 0;
}

// Tensor map over a contiguous fp32 [BH][N][D] buffer: dims (D, N, BH), box (32, 128, 1), 128-byte swizzle.
inline int make_tmap_f32_rows(CUtensorMap* m, float* base, int BH, int N, int D, const char* name) {
  encode_tiled_fn fn = get_encode_fn();
  if (!fn) return reject("cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)D * 4, (cuuint64_t)N * D * 4};
  cuuint32_t box[3] = {32, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return reject("%s: cuTensorMapEncodeTiled failed (CUresult %d)", name, (int)r);
  return 0;
}

}  // namespace castle
