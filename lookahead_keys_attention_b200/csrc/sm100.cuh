// Thin wrappers over the sm_100a instructions the CASTLE kernels are written in:
// mbarrier, TMA tile loads (cp.async.bulk.tensor), tensor memory (TMEM)
// allocation, tcgen05.mma with shared-memory operand descriptors, and
// tcgen05.ld/st between TMEM and registers.
//
// Every wait is bounded.  A wait that runs out of polls raises a CTA-wide
// abort flag in shared memory; from then on every wait in that CTA returns at
// once, the kernel falls through its (bounded) loops, frees its TMEM and
// records an error code in the status word the host reads back.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace castle {

constexpr uint32_t kWaitPollLimit = 1u << 22;  // polls of mbarrier.try_wait before giving up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  `abort_flag` lives in shared memory and is shared by the CTA.  Returns the number of
// polls made (the production kernels ignore it; the failure-path self test reports it).
__device__ __forceinline__ uint32_t mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              uint32_t poll_limit = kWaitPollLimit) {
  for (uint32_t i = 0; i < poll_limit; ++i) {
    if (mbar_try_wait(bar, parity)) return i;
    if (*abort_flag) return i;
  }
  *abort_flag = 1;
  return poll_limit;
}

// The same wait with the abort flag looked at on every 64th poll only.  With two CTAs per SM (the dim_head-64
// forward) the flag reads of one CTA's waiting threads share the shared-memory port with the other CTA's
// products and passes: 0.971 against 0.978 ms on the bench workload, same GPU.  (With one CTA per SM, in the backward,
// the same change measured slower: there the flag read paces the polls.)
__device__ __forceinline__ void mbar_wait_lazy_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitPollLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63u) == 63u && *abort_flag) return;
  }
  *abort_flag = 1;
}

// Barrier over the 128 threads (four warps) of one chunk group; ids 1..15 (0 is __syncthreads).
__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

// ---------------------------------------------------------------- fences
__device__ __forceinline__ void fence_async_smem() {  // generic-proxy smem writes -> async proxy (MMA/TMA) reads
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------- TMA
// 4-D tile load: coordinates are (c0 = element in row, c1 = row, c2 = head, c3 = batch).
__device__ __forceinline__ void tma_load_4d(void* dst, const void* tmap, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 3-D tile reduce-add from shared to global memory (fp32 atomic adds at L2, whole lines at a time);
// rows of the tile that fall outside the tensor are dropped.  Joins the thread's bulk async-group.
__device__ __forceinline__ void tma_reduce_add_3d(const void* tmap, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(tmap),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* tmap, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(tmap),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// 4-D tile store from a swizzled shared-memory tile (what tma_load_4d wrote) to global memory; rows of the
// tile that fall outside the tensor are dropped.  Joins the thread's bulk async-group.
__device__ __forceinline__ void tma_store_4d(const void* tmap, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tmap),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// Untiled bulk copies (16-byte aligned addresses, size a multiple of 16): a whole shared-memory tile, bytes as
// they lie (swizzle included), to or from a scratch area in global memory.
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* sdst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(sdst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory operand tiles are [rows][64 x 16-bit] with 128-byte rows and the
// 128-byte swizzle (16-byte chunk index XOR row%8), 1024-byte aligned: exactly
// what a TMA load with SWIZZLE_128B and a 64-element inner box writes.  Wider
// operands are several such "panels" laid one after another.
constexpr uint32_t kPanelRowBytes = 128;

__device__ __forceinline__ uint32_t swz_off(uint32_t row, uint32_t chunk16) {  // byte offset inside a panel
  return row * kPanelRowBytes + ((chunk16 ^ (row & 7u)) << 4);
}

// Descriptor for a panel read along its rows (the contraction index runs inside a
// row: "K-major").  8-row groups are 1024 bytes apart.  One MMA consumes 16
// elements = 32 bytes of every row; step k adds 32*k bytes to the start address.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                  // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                  // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
  return d;
}
// Descriptor for panels read down their columns (the contraction index is the ROW,
// the M/N index runs inside a row: "MN-major").  One MMA consumes 16 rows = two
// 8-row groups (stride byte offset 1024); M/N beyond 64 continues in the next
// panel, `panel_bytes` further on (leading byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t panel_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((panel_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation.
// fmt: 0 = fp16 operands, 1 = bf16 operands.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int fmt, bool a_mn, bool b_mn, bool neg_a) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((neg_a ? 1u : 0u) << 13) |
         ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// Both operands of one product must have the same format: an instruction descriptor with fp16 in one
// format field and bf16 in the other is rejected by the hardware (illegal instruction), so a tile the
// threads compute is always written in the type of the inputs it is multiplied with.

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accum)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows x 16 elements) sits in tensor memory, row m in
// lane m, elements 2j and 2j+1 packed in the low and high half of 32-bit column j (what a thread that owns
// row m writes with tcgen05.st of packed pairs).  Halves the shared-memory traffic of the product.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"((uint32_t)accum)
      : "memory");
}
// Make an mbarrier complete once every MMA this thread issued so far has finished.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------- TMEM <-> registers
// Warp w of a 128-thread group touches lanes 32*(w%4)..+31; each thread gets 32
// consecutive 32-bit columns of its own lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
      "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- 16-bit element helpers
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
  static constexpr int fmt = 1;
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
  }
  static __device__ __forceinline__ float2 unpack2(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
  static constexpr int fmt = 0;
  static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __half2 p = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
  }
  static __device__ __forceinline__ float2 unpack2(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

// 32 values of a row as 16 packed 16-bit pairs into 16 consecutive columns of the thread's lane: the
// layout a tensor-memory A operand wants (see mma_ts).
template <typename T>
__device__ __forceinline__ void tmem_st_packed32(uint32_t taddr, const float* v) {
  uint32_t r[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) r[j] = Elem<T>::pack2(v[2 * j], v[2 * j + 1]);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(taddr)
      : "memory");
}

// ---------------------------------------------------------------- fast transcendentals
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// sigmoid as one special-function op: 0.5 * tanh.approx(x / 2) + 0.5.  tanh.approx is good to about 2^-11,
// i.e. the result to ~2.4e-4: below bf16 rounding (2e-3) and at the level of fp16 rounding (2.4e-4) of the
// operand tiles the result is packed into.  (An exp-and-divide form costs two special-function ops.)
template <typename T>
__device__ __forceinline__ float sigmoid_t(float x) {
  return fmaf(0.5f, tanh_approx(0.5f * x), 0.5f);
}

// Write 32 consecutive elements (columns c0..c0+31, c0 a multiple of 32) of row `row`
// of a swizzled panel set whose panels are `panel_bytes` apart.
template <typename T>
__device__ __forceinline__ void store_row32(uint8_t* tile, uint32_t panel_bytes, uint32_t row, uint32_t c0,
                                            const float* v) {
  uint8_t* panel = tile + (c0 >> 6) * panel_bytes;
  uint32_t chunk0 = (c0 & 63u) >> 3;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q;
    q.x = Elem<T>::pack2(v[8 * c + 0], v[8 * c + 1]);
    q.y = Elem<T>::pack2(v[8 * c + 2], v[8 * c + 3]);
    q.z = Elem<T>::pack2(v[8 * c + 4], v[8 * c + 5]);
    q.w = Elem<T>::pack2(v[8 * c + 6], v[8 * c + 7]);
    *reinterpret_cast<uint4*>(panel + swz_off(row, chunk0 + c)) = q;
  }
}
// fp32 staging panel [128 rows][32 floats] with the same 128-byte swizzle: one row of 32 values
__device__ __forceinline__ void store_row32_f32(uint8_t* panel, uint32_t row, const float* v) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<float4*>(panel + swz_off(row, c)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}
template <typename T>
__device__ __forceinline__ void load_row32(const uint8_t* tile, uint32_t panel_bytes, uint32_t row, uint32_t c0,
                                           float* v) {
  const uint8_t* panel = tile + (c0 >> 6) * panel_bytes;
  uint32_t chunk0 = (c0 & 63u) >> 3;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q = *reinterpret_cast<const uint4*>(panel + swz_off(row, chunk0 + c));
    float2 a = Elem<T>::unpack2(q.x), b = Elem<T>::unpack2(q.y), e = Elem<T>::unpack2(q.z), f = Elem<T>::unpack2(q.w);
    v[8 * c + 0] = a.x; v[8 * c + 1] = a.y; v[8 * c + 2] = b.x; v[8 * c + 3] = b.y;
    v[8 * c + 4] = e.x; v[8 * c + 5] = e.y; v[8 * c + 6] = f.x; v[8 * c + 7] = f.y;
  }
}

// ---------------------------------------------------------------- whole-tile MMA helpers (one issuing thread)
// The issuing thread is a serial bottleneck (every product of a phase goes through it), so the
// step counts are compile-time, the loops are unrolled and each step's descriptor is the base
// descriptor plus a constant in its 16-byte-granular address field.
//
// C[128 x N] (+)= X[128 x Kc] * Y[N x Kc]^T, both operands read along rows; Kc = 64*NPANELS.
template <int NPANELS>
__device__ __forceinline__ void gemm_kk_t(uint32_t d_tmem, uint32_t x_addr, uint32_t y_addr, uint32_t idesc, bool accum) {
  const uint64_t dx = desc_kmajor(x_addr), dy = desc_kmajor(y_addr);
#pragma unroll
  for (int p = 0; p < NPANELS; ++p) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint64_t off = (uint64_t)((p * (128 * 128) + 32 * k) >> 4);
      mma_ss(d_tmem, dx + off, dy + off, idesc, accum || p > 0 || k > 0);
    }
  }
}
// C[128 x N] (+)= X[128 x Kc] * Y[Kc x N]: X read along rows, Y ([Kc rows][N], 64-column panels
// 16 KB apart) read down its columns.  Kc = 16*KSTEPS (rows of Y).
template <int KSTEPS>
__device__ __forceinline__ void gemm_km_t(uint32_t d_tmem, uint32_t x_addr, uint32_t y_addr, uint32_t idesc, bool accum) {
  const uint64_t dx = desc_kmajor(x_addr), dy = desc_mnmajor(y_addr, 128 * 128);
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
    const uint64_t xo = (uint64_t)(((k >> 2) * (128 * 128) + 32 * (k & 3)) >> 4);
    mma_ss(d_tmem, dx + xo, dy + (uint64_t)((2048 * k) >> 4), idesc, accum || k > 0);
  }
}
// C[128 x N] (+)= X * Y^T with X in tensor memory (packed 16-bit pairs, 8 columns per 16-element step) and
// Y [N rows][64*NPANELS] in shared memory read along its rows.
template <int NPANELS>
__device__ __forceinline__ void gemm_tk_t(uint32_t d_tmem, uint32_t x_tmem, uint32_t y_addr, uint32_t idesc, bool accum) {
  const uint64_t dy = desc_kmajor(y_addr);
#pragma unroll
  for (int p = 0; p < NPANELS; ++p) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint64_t off = (uint64_t)((p * (128 * 128) + 32 * k) >> 4);
      mma_ts(d_tmem, x_tmem + (p * 4 + k) * 8, dy + off, idesc, accum || p > 0 || k > 0);
    }
  }
}
// C[128 x N] (+)= X * Y with X in tensor memory and Y [Kc rows][N] in shared memory read down its columns.
template <int KSTEPS>
__device__ __forceinline__ void gemm_tm_t(uint32_t d_tmem, uint32_t x_tmem, uint32_t y_addr, uint32_t idesc, bool accum) {
  const uint64_t dy = desc_mnmajor(y_addr, 128 * 128);
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) mma_ts(d_tmem, x_tmem + k * 8, dy + (uint64_t)((2048 * k) >> 4), idesc, accum || k > 0);
}
// C[128 x N] (+)= X^T * Y with X [Kc rows][128] and Y [Kc rows][N], both read down their columns.
template <int KSTEPS>
__device__ __forceinline__ void gemm_mm_t(uint32_t d_tmem, uint32_t x_addr, uint32_t y_addr, uint32_t idesc, bool accum) {
  const uint64_t dx = desc_mnmajor(x_addr, 128 * 128), dy = desc_mnmajor(y_addr, 128 * 128);
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
    const uint64_t off = (uint64_t)((2048 * k) >> 4);
    mma_ss(d_tmem, dx + off, dy + off, idesc, accum || k > 0);
  }
}
// C[128 x N] (+)= X^T * Y^T with X [Kc rows][128] read down its columns and Y [N rows][Kc] read along rows.
template <int KSTEPS>
__device__ __forceinline__ void gemm_mk_t(uint32_t d_tmem, uint32_t x_addr, uint32_t y_addr, uint32_t idesc, bool accum) {
  const uint64_t dx = desc_mnmajor(x_addr, 128 * 128), dy = desc_kmajor(y_addr);
#pragma unroll
  for (int k = 0; k < KSTEPS; ++k) {
    const uint64_t yo = (uint64_t)(((k >> 2) * (128 * 128) + 32 * (k & 3)) >> 4);
    mma_ss(d_tmem, dx + (uint64_t)((2048 * k) >> 4), dy + yo, idesc, accum || k > 0);
  }
}

// Run-time-count forms (used by the self test).
__device__ __forceinline__ void gemm_kk(uint32_t d_tmem, uint32_t x_addr, uint32_t x_panel_bytes, uint32_t y_addr,
                                        uint32_t y_panel_bytes, int npanels, uint32_t idesc, bool accum) {
  (void)x_panel_bytes; (void)y_panel_bytes;
  if (npanels == 1) gemm_kk_t<1>(d_tmem, x_addr, y_addr, idesc, accum);
  else gemm_kk_t<2>(d_tmem, x_addr, y_addr, idesc, accum);
}
__device__ __forceinline__ void gemm_km(uint32_t d_tmem, uint32_t x_addr, uint32_t x_panel_bytes, uint32_t y_addr,
                                        uint32_t y_panel_bytes, int ksteps, uint32_t idesc, bool accum) {
  (void)x_panel_bytes; (void)y_panel_bytes; (void)ksteps;
  gemm_km_t<8>(d_tmem, x_addr, y_addr, idesc, accum);
}
__device__ __forceinline__ void gemm_mm(uint32_t d_tmem, uint32_t x_addr, uint32_t x_panel_bytes, uint32_t y_addr,
                                        uint32_t y_panel_bytes, int ksteps, uint32_t idesc, bool accum) {
  (void)x_panel_bytes; (void)y_panel_bytes; (void)ksteps;
  gemm_mm_t<8>(d_tmem, x_addr, y_addr, idesc, accum);
}
__device__ __forceinline__ void gemm_mk(uint32_t d_tmem, uint32_t x_addr, uint32_t x_panel_bytes, uint32_t y_addr,
                                        uint32_t y_panel_bytes, int ksteps, uint32_t idesc, bool accum) {
  (void)x_panel_bytes; (void)y_panel_bytes; (void)ksteps;
  gemm_mk_t<8>(d_tmem, x_addr, y_addr, idesc, accum);
}

}  // namespace castle
