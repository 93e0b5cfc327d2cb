// Element-type conversions around the parallel kernels, for callers whose tensors the kernels do not take as
// they are: bf16 tensors that are computed with fp16 operands (long sequences), in one pass each way.
// HBM-bound: 16 bytes in and 16 bytes out per thread and iteration, grid-stride.
#include "common.cuh"
#include "sm100.cuh"

namespace castle {

// bf16 -> fp16, saturating at +-65504 instead of overflowing to infinity; optional factor `*mul` (device scalar).
__global__ void __launch_bounds__(256) castle_bf16_to_f16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                 int64_t n8, const float* mul) {
  const float m = mul ? *mul : 1.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v = src[i];
    uint32_t* u = &v.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = Elem<__nv_bfloat16>::unpack2(u[j]);
      f.x = fminf(fmaxf(f.x * m, -65504.f), 65504.f);
      f.y = fminf(fmaxf(f.y * m, -65504.f), 65504.f);
      u[j] = Elem<__half>::pack2(f.x, f.y);
    }
    dst[i] = v;
  }
}

// fp16 -> bf16 times `*mul` (device scalar, may be null)
__global__ void __launch_bounds__(256) castle_f16_to_bf16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                                 int64_t n8, const float* mul) {
  const float m = mul ? *mul : 1.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v = src[i];
    uint32_t* u = &v.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = Elem<__half>::unpack2(u[j]);
      u[j] = Elem<__nv_bfloat16>::pack2(f.x * m, f.y * m);
    }
    dst[i] = v;
  }
}

}  // namespace castle

using namespace castle;

extern "C" int castle_convert_16bit(int32_t src_dtype, const void* src, void* dst, int64_t count, const float* mul,
                                    void* stream) {
  if (src_dtype != CASTLE_BF16 && src_dtype != CASTLE_F16) return reject("castle_convert_16bit: source must be bf16 or fp16");
  if (!src || !dst || count <= 0) return reject("castle_convert_16bit: null pointer or empty tensor");
  if (count % 8 || ((uintptr_t)src) % 16 || ((uintptr_t)dst) % 16)
    return reject("castle_convert_16bit: count must be a multiple of 8 and the pointers 16-byte aligned");
  const int64_t n8 = count / 8;
  const unsigned blocks = (unsigned)((n8 + 255) / 256 < 148 * 16 ? (n8 + 255) / 256 : 148 * 16);
  cudaStream_t st = (cudaStream_t)stream;
  if (src_dtype == CASTLE_BF16)
    castle_bf16_to_f16_kernel<<<blocks, 256, 0, st>>>((const uint4*)src, (uint4*)dst, n8, mul);
  else
    castle_f16_to_bf16_kernel<<<blocks, 256, 0, st>>>((const uint4*)src, (uint4*)dst, n8, mul);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_convert_16bit launch");
}
