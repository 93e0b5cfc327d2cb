// Self test of the tensor-core building blocks: one 128x128x128 product through
// every operand form the CASTLE kernels use (rows-contracted and
// columns-contracted shared-memory operands, staged by thread stores or by TMA,
// a preset accumulator and a negated operand), plus the two forms whose first operand sits in tensor
// memory as packed 16-bit pairs.
#include "common.cuh"
#include "sm100.cuh"

namespace castle {

constexpr uint32_t kPanel = 128 * 128;  // bytes of a [128 rows][64 x 16-bit] panel

__global__ void __launch_bounds__(128) castle_selftest_kernel(int mode, const __nv_bfloat16* x, const __nv_bfloat16* y,
                                                              float* d, int32_t* status,
                                                              const __grid_constant__ CUtensorMap mx,
                                                              const __grid_constant__ CUtensorMap my) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sx = smem;               // 2 panels
  uint8_t* sy = smem + 2 * kPanel;  // 2 panels
  __shared__ uint64_t bar_tma, bar_mma;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool a_in_tmem = mode == 9 || mode == 10;   // 9: X (tensor memory) @ Y^T, 10: X (tensor memory) @ Y
  const bool use_tma = mode >= 5 && mode <= 8;
  const int op = use_tma ? mode - 5 : mode;

  if (tid == 0) {
    mbar_init(&bar_tma, 1);
    mbar_init(&bar_mma, 1);
    mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  if (use_tma) {
    if (tid == 0) {
      mbar_expect_tx(&bar_tma, 4 * kPanel);
      tma_load_4d(sx, &mx, &bar_tma, 0, 0, 0, 0);
      tma_load_4d(sx + kPanel, &mx, &bar_tma, 64, 0, 0, 0);
      tma_load_4d(sy, &my, &bar_tma, 0, 0, 0, 0);
      tma_load_4d(sy + kPanel, &my, &bar_tma, 64, 0, 0, 0);
    }
    mbar_wait(&bar_tma, 0, &abort_flag);
  } else {
    for (int c = 0; c < 16; ++c) {
      uint4 vx = *reinterpret_cast<const uint4*>(x + tid * 128 + c * 8);
      uint4 vy = *reinterpret_cast<const uint4*>(y + tid * 128 + c * 8);
      *reinterpret_cast<uint4*>(sx + (c >> 3) * kPanel + swz_off(tid, c & 7)) = vx;
      *reinterpret_cast<uint4*>(sy + (c >> 3) * kPanel + swz_off(tid, c & 7)) = vy;
    }
    fence_async_smem();
  }
  if (a_in_tmem) {  // this thread's row of X as packed pairs into columns 128..191 of its lane
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float pk[32];
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        uint4 q = *reinterpret_cast<const uint4*>(x + tid * 128 + c * 64 + j * 2);
        pk[j] = __uint_as_float(q.x); pk[j + 1] = __uint_as_float(q.y);
        pk[j + 2] = __uint_as_float(q.z); pk[j + 3] = __uint_as_float(q.w);
      }
      tmem_st32(tmem + ((uint32_t)(warp * 32) << 16) + 128 + c * 32, pk);
    }
    tmem_st_wait();
  }
  if (op == 4) {  // preset the accumulator to 1.0
    float ones[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) ones[i] = 1.f;
    for (int c = 0; c < 4; ++c) tmem_st32(tmem + ((uint32_t)(warp * 32) << 16) + c * 32, ones);
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (tid == 0) {
    const uint32_t xa = smem_u32(sx), ya = smem_u32(sy);
    switch (op) {
      case 0: gemm_kk(tmem, xa, kPanel, ya, kPanel, 2, make_idesc(128, 128, 1, false, false, false), false); break;
      case 1: gemm_km(tmem, xa, kPanel, ya, kPanel, 8, make_idesc(128, 128, 1, false, true, false), false); break;
      case 2: gemm_mm(tmem, xa, kPanel, ya, kPanel, 8, make_idesc(128, 128, 1, true, true, false), false); break;
      case 3: gemm_mk(tmem, xa, kPanel, ya, kPanel, 8, make_idesc(128, 128, 1, true, false, false), false); break;
      case 9: gemm_tk_t<2>(tmem, tmem + 128, ya, make_idesc(128, 128, 1, false, false, false), false); break;
      case 10: gemm_tm_t<8>(tmem, tmem + 128, ya, make_idesc(128, 128, 1, false, true, false), false); break;
      default: gemm_kk(tmem, xa, kPanel, ya, kPanel, 2, make_idesc(128, 128, 1, false, false, true), true); break;
    }
    mma_commit(&bar_mma);
  }
  mbar_wait(&bar_mma, 0, &abort_flag);
  tc_fence_after();
  for (int c = 0; c < 4; ++c) {
    float v[32];
    tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + c * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) d[tid * 128 + c * 32 + i] = v[i];
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
  if (tid == 0 && abort_flag) atomicOr(status, CASTLE_STATUS_WAIT_TIMEOUT);
}

}  // namespace castle

using namespace castle;

extern "C" int castle_selftest_mma(int32_t mode, const void* x, const void* y, float* d, int32_t* status,
                                   void* stream) {
  if (mode < 0 || mode > 10) return reject("castle_selftest_mma: mode %d out of range", mode);
  if (!x || !y || !d || !status) return reject("castle_selftest_mma: null pointer");
  CUtensorMap mx, my;
  castle_tensor_t tx = {(void*)x, 128 * 128, 128 * 128, 128}, ty = {(void*)y, 128 * 128, 128 * 128, 128};
  int rc = make_tmap_16bit(&mx, &tx, CASTLE_BF16, 1, 1, 128, 128, 128, "x");
  if (rc) return rc;
  rc = make_tmap_16bit(&my, &ty, CASTLE_BF16, 1, 1, 128, 128, 128, "y");
  if (rc) return rc;
  size_t smem = 4 * kPanel + 1024;
  cudaError_t e = cudaFuncSetAttribute(castle_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "castle_selftest_mma attribute");
  castle_selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(mode, (const __nv_bfloat16*)x,
                                                                 (const __nv_bfloat16*)y, d, status, mx, my);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_selftest_mma launch");
}

// ---------------------------------------------------------------------------------------------
// Issue-to-completion cost of one tensor-core instruction per operand form and width: `reps`
// back-to-back products of shape 128 x n x 16 (operands are whatever the shared memory holds;
// only the timing matters), one commit, cycles from first issue to completion.
namespace castle {
__global__ void __launch_bounds__(128) castle_mma_rate_kernel(int form, int n, int reps, long long* cycles, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  // eight panels: A in 0..1 (128 rows or 128 columns), B in 2..5 (up to 256 rows, or 256 columns = 4 panels)
  for (int i = tid; i < 8 * (int)kPanel / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0x3c003c00u;  // finite values
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); abort_flag = 0; }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 256); tmem_relinquish(); }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  if (tid == 0) {
    const uint32_t xa = smem_u32(smem), ya = smem_u32(smem + 2 * kPanel);
    const bool a_mn = form == 2 || form == 3, b_mn = form == 1 || form == 2;
    const uint32_t idesc = make_idesc(128, n, 1, a_mn, b_mn, false);
    const uint64_t dx = a_mn ? desc_mnmajor(xa, kPanel) : desc_kmajor(xa);
    const uint64_t dy = b_mn ? desc_mnmajor(ya, kPanel) : desc_kmajor(ya);
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      const int k = r & 3;  // walk the four 16-element steps of a panel like the kernels do
      mma_ss(tmem, dx + (uint64_t)((a_mn ? 2048 * k : 32 * k) >> 4), dy + (uint64_t)((b_mn ? 2048 * k : 32 * k) >> 4), idesc, r > 0);
    }
    const long long t1 = clock64();
    mma_commit(&bar);
    mbar_wait(&bar, 0, &abort_flag);
    const long long t2 = clock64();
    cycles[0] = t1 - t0;  // issue only
    cycles[1] = t2 - t0;  // issue to completion
  }
  __syncthreads();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
  if (tid == 0 && abort_flag) atomicOr(status, CASTLE_STATUS_WAIT_TIMEOUT);
}
}  // namespace castle

extern "C" int castle_selftest_mma_rate(int32_t form, int32_t n, int32_t reps, long long* cycles, int32_t* status,
                                        void* stream) {
  if (form < 0 || form > 3 || (n != 64 && n != 128 && n != 192 && n != 256) || reps < 1 || reps > 4096)
    return reject("castle_selftest_mma_rate: bad arguments");
  if (!cycles || !status) return reject("castle_selftest_mma_rate: null pointer");
  size_t smem = 8 * kPanel + 1024;
  cudaError_t e = cudaFuncSetAttribute(castle_mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "castle_selftest_mma_rate attribute");
  castle_mma_rate_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(form, n, reps, cycles, status);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_selftest_mma_rate launch");
}

// ---------------------------------------------------------------------------------------------
// Failure path of the bounded waits, exercised without faulting anything: 128 threads allocate
// tensor memory like a production CTA, then ALL wait on an mbarrier nothing arrives on.  The first
// thread whose polls run out raises the abort flag; the others see it and return; a second wait
// must then return at once; the CTA frees its tensor memory and reports through the status word.
namespace castle {
__global__ void __launch_bounds__(128) castle_wait_timeout_kernel(uint32_t poll_limit, int32_t* polls, int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); abort_flag = 0; }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 32); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t n1 = mbar_wait(&bar, 0, &abort_flag, poll_limit);   // never completes: gives up after poll_limit polls
  const uint32_t n2 = mbar_wait(&bar, 0, &abort_flag, poll_limit);   // the flag is up: returns at the first poll
  if (tid == 0) { polls[0] = (int32_t)n1; polls[1] = (int32_t)n2; }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 32);
  if (tid == 0 && abort_flag) atomicOr(status, CASTLE_STATUS_WAIT_TIMEOUT);
}
}  // namespace castle

extern "C" int castle_selftest_wait_timeout(int32_t poll_limit, int32_t* polls, int32_t* status, void* stream) {
  if (poll_limit < 1 || poll_limit > 65536) return reject("castle_selftest_wait_timeout: poll_limit must be 1..65536");
  if (!polls || !status) return reject("castle_selftest_wait_timeout: null pointer");
  castle_wait_timeout_kernel<<<1, 128, 0, (cudaStream_t)stream>>>((uint32_t)poll_limit, polls, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_selftest_wait_timeout launch");
}
