// CASTLE parallel backward for dim_head 128.
//
// At d = 128 the five per-key-block accumulators of the d = 64 kernel (W, G, dkc, dvc, dqu) would
// need 640 TMEM columns, and seven 32 KB operand tiles already fill shared memory.  The pass is
// therefore split into two kernels, each walking the query blocks I downwards for one key block K:
//
//   castle_bwd128_kv_kernel   TMEM: W | dkc | dvc | scratch.  Recomputes the scores (Z, gate, peeled
//                             state W, T, Su, Sc) the way the d = 64 kernel does, accumulates dkc and
//                             dvc in TMEM, builds dqc[I] = dS@Kc + dSu@Wb + dT@Vu in the scratch and
//                             adds it to the fp32 workspace with a TMA reduce.  It also stores the gate A,
//                             dSu and the masked T of every (I, K) step to a global scratch, as the
//                             16-bit tiles lie in shared memory (3 x 32 KB per step).
//   castle_bwd128_la_kernel   TMEM: dqu | G | scratch | scratch.  Runs after it on the same stream,
//                             loads those three tiles and recomputes nothing: carries the reverse
//                             state G and dqu[K] in TMEM and reduces dvu[I], dku[I] per step.
//
// The scratch is bounded (see kTileScratchLimit): the (batch, head) pairs run in chunks, one launch
// of each kernel per chunk.
//
// Shared memory is seven 32 KB slots that are re-used as tiles die; each comment "-> sN" below
// says which slot a tile lands in.  512 threads: warp w owns TMEM lanes 32*(w%4).. and columns
// 32*(w/4).. of every 128-column accumulator.
#include "bwd_common.cuh"

namespace castle {

constexpr int kB128Threads = 512;
constexpr uint32_t kSlot = 2 * kPanelB;                      // 32 KB
constexpr size_t kB128Smem = 7 * kSlot + 1024;

// Timing experiments only (never in the shipped library): drop the reduces to see what they cost.
#ifdef CASTLE_TIMING_SKIP_REDUCE
#define tma_reduce_add_3d(...) do { } while (0)
#endif

// Optional phase timing (debug builds only): thread 0 of CTA (0,0) stores clock64() at phase boundaries of
// its first steps behind the fp32 workspace (key/value kernel at slot 0, lookahead kernel at slot 256).
#ifdef CASTLE_PHASE_TIMING
#define B128_MARK(base, i) do { if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && p.nblk - 1 - I < 8) p.timing[(base) + (p.nblk - 1 - I) * 32 + (i)] = clock64(); } while (0)
#else
#define B128_MARK(base, i) do { } while (0)
#endif

#define B128_MMA_WAIT()                  \
  mbar_wait(&bar_mma, ph_mma, abortp);   \
  ph_mma ^= 1;                           \
  tc_fence_after();
#define B128_SYNC()    \
  fence_async_smem();  \
  tc_fence_before();   \
  __syncthreads();

template <int NP>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int r0, int h, int b) {
#pragma unroll
  for (int pn = 0; pn < NP; ++pn) tma_load_4d(dst + pn * kPanelB, m, bar, pn * 64, r0, h, b);
}

// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kB128Threads, 1)
castle_bwd128_kv_kernel(const BwdParams p, const __grid_constant__ CUtensorMap m_qc, const __grid_constant__ CUtensorMap m_kc,
                        const __grid_constant__ CUtensorMap m_vc, const __grid_constant__ CUtensorMap m_qu,
                        const __grid_constant__ CUtensorMap m_ku, const __grid_constant__ CUtensorMap m_vu,
                        const __grid_constant__ CUtensorMap m_do, const __grid_constant__ CUtensorMap m_acc_dqc) {
  constexpr int D = 128;
  constexpr int FMT = Elem<T>::fmt;
  constexpr uint32_t ID_KK = make_idesc(128, 128, FMT, false, false, false);
  constexpr uint32_t ID_KM = make_idesc(128, 128, FMT, false, true, false);
  constexpr uint32_t ID_KM_NEG = make_idesc(128, 128, FMT, false, true, true);
  constexpr uint32_t ID_MM = make_idesc(128, 128, FMT, true, true, false);
  constexpr float kLog2e = 1.4426950408889634f;
  constexpr uint32_t C_W = 0, C_DKC = 128, C_DVC = 256, C_S = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* s0 = smem;              // Qu[K] -> Wb
  uint8_t* s1 = s0 + kSlot;        // Ku[I] -> gate A -> dT
  uint8_t* s2 = s1 + kSlot;        // Vu[I] -> masked T -> P -> Vu[I] again
  uint8_t* s3 = s2 + kSlot;        // Qc[I]
  uint8_t* s4 = s3 + kSlot;        // Kc[K]
  uint8_t* s5 = s4 + kSlot;        // Vc[K] -> dS -> dqc staging
  uint8_t* s6 = s5 + kSlot;        // dO[I] -> dSu -> dqc staging
  __shared__ uint64_t bar_a, bar_b, bar_vu2, bar_mma, bar_x1, bar_x2;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, cc = warp >> 2;
  const int row = quarter * 32 + lane, c0 = cc * 32;
  const int bh = p.bh0 + blockIdx.x, K = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int k0 = K * kBlkB, krow = k0 + row;
  const bool issuer = (quarter == 0 && lane == 0);   // threads 0, 128, 256, 384: one reduce each per step
  // One lane hands three tiles of every step to the lookahead kernel through global memory, bytes as they lie
  // in shared memory: the gate A, the masked T and dSu.  That kernel then recomputes nothing.
  const bool storer = (tid == 64);
  uint8_t* const tile_base = p.tiles + (int64_t)blockIdx.x * p.ntiles * 3 * kSlot;

  if (tid == 0) {
    mbar_init(&bar_a, 1); mbar_init(&bar_b, 1); mbar_init(&bar_vu2, 1); mbar_init(&bar_mma, 1);
    mbar_init(&bar_x1, 1); mbar_init(&bar_x2, 1);
    mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
  volatile int* abortp = &abort_flag;

  if (tid == 0) {
    const int il = (p.nblk - 1) * kBlkB;
    mbar_expect_tx(&bar_a, 5 * kSlot);
    load_tile<2>(s0, &m_qu, &bar_a, k0, h, b);
    load_tile<2>(s1, &m_ku, &bar_a, il, h, b);
    load_tile<2>(s2, &m_vu, &bar_a, il, h, b);
    load_tile<2>(s3, &m_qc, &bar_a, il, h, b);
    load_tile<2>(s4, &m_kc, &bar_a, k0, h, b);
  }
  {  // W_K starts as the forward's final state
    const float* src = p.w_state + ((int64_t)bh * p.N + krow) * D + c0;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      float4 q = (krow < p.N) ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
      v[j] = q.x; v[j + 1] = q.y; v[j + 2] = q.z; v[j + 3] = q.w;
    }
    tmem_st32(trow + C_W + c0, v);
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();

  uint32_t ph_a = 0, ph_b = 0, ph_vu2 = 0, ph_mma = 0, ph_x = 0;
  const uint32_t a0 = smem_u32(s0), a1 = smem_u32(s1), a2 = smem_u32(s2), a3 = smem_u32(s3), a4 = smem_u32(s4),
                 a5 = smem_u32(s5), a6 = smem_u32(s6);
  const float sl2 = p.scale * kLog2e;

  for (int I = p.nblk - 1; I >= K; --I) {
    const int i0 = I * kBlkB, irow = i0 + row;
    const bool diag = (I == K), first = (I == p.nblk - 1);
    const bool rvalid = irow < p.N;
    const float lse_b = rvalid ? p.lse[(int64_t)bh * p.N + irow] * kLog2e : 0.f;
    const float delta_i = rvalid ? p.delta[(int64_t)bh * p.N + irow] : 0.f;

    B128_MARK(0, 0);
    // ---- M0: Z = Qu[K] @ Ku[I]^T
    if (tid == 0) {
      mbar_wait(&bar_a, ph_a, abortp);
      B128_MARK(0, 1);
      tc_fence_after();
      gemm_kk_t<2>(tmem + C_S, a0, a1, ID_KK, false);
      mma_commit(&bar_mma);
    }
    ph_a ^= 1;
    B128_MMA_WAIT();
    B128_MARK(0, 2);
    {  // gate A -> s1 (over Ku)
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = sigmoid_t<T>(v[j] * p.scale);
      if (diag) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j > row) ? v[j] : 0.f;
      }
      store_row32<T>(s1, kPanelB, row, c0, v);
    }
    if (issuer) bulk_wait_read0();  // this lane's dqc panel of the step before (in s5|s6) has been read
    B128_SYNC();
    B128_MARK(0, 3);
    uint8_t* const tile = tile_base + ((int64_t)I * (I + 1) / 2 + K) * 3 * kSlot;
    if (storer) { bulk_s2g(tile, s1, kSlot); bulk_commit(); }   // gate A

    // ---- M1: peel W -= A @ Vu[I];  T = Qc[I] @ Vu[I]^T
    if (tid == 0) {
      tc_fence_after();
      gemm_km_t<8>(tmem + C_W, a1, a2, ID_KM_NEG, true);
      gemm_kk_t<2>(tmem + C_S, a3, a2, ID_KK, false);
      mma_commit(&bar_mma);
      mbar_expect_tx(&bar_b, 2 * kSlot);   // needed at the fifth phase; issued behind the products
      load_tile<2>(s5, &m_vc, &bar_b, k0, h, b);
      load_tile<2>(s6, &m_do, &bar_b, i0, h, b);
    }
    B128_MMA_WAIT();
    B128_MARK(0, 4);
    {  // masked T -> s2 (over Vu); 16-bit copy of the peeled state -> s0 (over Qu)
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      store_row32<T>(s2, kPanelB, row, c0, v);
      tmem_ld32(trow + C_W + c0, v);
      tmem_ld_wait();
      store_row32<T>(s0, kPanelB, row, c0, v);
    }
    B128_SYNC();
    B128_MARK(0, 5);
    if (storer) { bulk_s2g(tile + 2 * kSlot, s2, kSlot); bulk_commit(); }   // masked T

    // ---- M2: Su/scale = Qc[I] @ Wb^T + Tm @ A^T
    if (tid == 0) {
      tc_fence_after();
      if (!diag) gemm_kk_t<2>(tmem + C_S, a3, a0, ID_KK, false);
      gemm_kk_t<2>(tmem + C_S, a2, a1, ID_KK, !diag);
      mma_commit(&bar_mma);
    }
    B128_MMA_WAIT();
    B128_MARK(0, 6);
    uint32_t dpk[16], ppk[16];
    {
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float su0 = v[j] * p.scale, su1 = v[j + 1] * p.scale;
        float g0 = sigmoid_t<T>(su0), g1 = sigmoid_t<T>(su1);
        v[j] = -v[j] * g0;
        v[j + 1] = -v[j + 1] * g1;
        dpk[j / 2] = Elem<T>::pack2(g0 * (1.f + su0 * (1.f - g0)), g1 * (1.f + su1 * (1.f - g1)));
      }
      tmem_st32(trow + C_S + c0, v);
      tmem_st_wait();
    }
    if (storer) bulk_wait_read0();   // the copies of the gate and of the masked T have read their slots (P goes over T next)
    tc_fence_before();
    __syncthreads();
    B128_MARK(0, 7);

    // ---- M3: S/scale = penalty + Qc[I] @ Kc[K]^T
    if (tid == 0) {
      tc_fence_after();
      gemm_kk_t<2>(tmem + C_S, a3, a4, ID_KK, true);
      mma_commit(&bar_mma);
    }
    B128_MMA_WAIT();
    B128_MARK(0, 8);
    {  // P -> s2 (over the masked T)
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = ex2_approx(fmaf(v[j], sl2, -lse_b));
      if (diag) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      }
      if (!rvalid) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < 32; j += 2) ppk[j / 2] = Elem<T>::pack2(v[j], v[j + 1]);
      store_row32<T>(s2, kPanelB, row, c0, v);
    }
    B128_SYNC();
    B128_MARK(0, 9);

    // ---- M4: dvc += P^T @ dO[I];  dP = dO[I] @ Vc[K]^T
    if (tid == 0) {
      mbar_wait(&bar_b, ph_b, abortp);
      tc_fence_after();
      mbar_expect_tx(&bar_vu2, kSlot);   // armed here, the two loads are issued below by other lanes
      gemm_mm_t<8>(tmem + C_DVC, a2, a6, ID_MM, !first);
      gemm_kk_t<2>(tmem + C_S, a6, a5, ID_KK, false);
      mma_commit(&bar_mma);
    }
    ph_b ^= 1;
    B128_MMA_WAIT();
    B128_MARK(0, 10);
    // P is consumed: Vu[I] comes back into s2 for the last product (one panel per lane: a TMA
    // instruction costs its issuing thread ~150 cycles)
    if (lane == 0 && (warp == 5 || warp == 9)) tma_load_4d(s2 + (warp == 9) * kPanelB, &m_vu, &bar_vu2, (warp == 9) * 64, i0, h, b);
    {  // dS -> s5 (over Vc), dSu -> s6 (over dO)
      float v[32], w[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float2 pp = Elem<T>::unpack2(ppk[j / 2]);
        float2 dd = Elem<T>::unpack2(dpk[j / 2]);
        float ds0 = pp.x * (v[j] - delta_i), ds1 = pp.y * (v[j + 1] - delta_i);
        v[j] = ds0; v[j + 1] = ds1;
        w[j] = -ds0 * dd.x; w[j + 1] = -ds1 * dd.y;
      }
      store_row32<T>(s5, kPanelB, row, c0, v);
      store_row32<T>(s6, kPanelB, row, c0, w);
    }
    B128_SYNC();
    B128_MARK(0, 11);
    if (storer) { bulk_s2g(tile + kSlot, s6, kSlot); bulk_commit(); }   // dSu

    // ---- M5: dkc += dS^T @ Qc[I];  dT = dSu @ A
    if (tid == 0) {
      tc_fence_after();
      gemm_km_t<8>(tmem + C_S, a6, a1, ID_KM, false);
      mma_commit(&bar_mma);  // dT alone: masking it overlaps the dkc product, which the next commit covers
      gemm_mm_t<8>(tmem + C_DKC, a5, a3, ID_MM, !first);
    }
    B128_MMA_WAIT();
    B128_MARK(0, 12);
    {  // masked dT -> s1 (over the gate)
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      store_row32<T>(s1, kPanelB, row, c0, v);
    }
    if (storer) bulk_wait_read0();   // the copy of dSu has read its slot (the dqc staging goes there at the end of the step)
    B128_SYNC();
    B128_MARK(0, 13);

    // ---- M6: dqc[I] (unscaled) = dT @ Vu[I] + dSu @ Wb + dS @ Kc[K]
    // Three commits, in the order in which the products free the per-step slots, so that the next
    // block's tiles are fetched as early as possible (a tile takes 2-4 thousand cycles to arrive): behind
    // the first Ku, Vu and Qc (s1, s2; s3's last reader, the dkc product issued in the phase before, is
    // covered too), behind the second Qu (s0).  One 16 KB panel per lane of eight warps.
    if (tid == 0) {
      mbar_wait(&bar_vu2, ph_vu2, abortp);
      tc_fence_after();
      if (I > K) mbar_expect_tx(&bar_a, 4 * kSlot);   // armed here, the eight loads are issued by other lanes
      gemm_km_t<8>(tmem + C_S, a1, a2, ID_KM, false);
      mma_commit(&bar_x1);
      if (!diag) gemm_km_t<8>(tmem + C_S, a6, a0, ID_KM, true);
      mma_commit(&bar_x2);
      gemm_km_t<8>(tmem + C_S, a5, a4, ID_KM, true);
      mma_commit(&bar_mma);
    }
    ph_vu2 ^= 1;
    if (lane == 0 && warp < 8 && I > K) {
      const int in0 = (I - 1) * kBlkB;
      const int t = warp >> 1, pn = warp & 1;   // tile 0: Qu -> s0, 1: Ku -> s1, 2: Vu -> s2, 3: Qc -> s3
      const CUtensorMap* m = t == 0 ? &m_qu : (t == 1 ? &m_ku : (t == 2 ? &m_vu : &m_qc));
      mbar_wait(t == 0 ? &bar_x2 : &bar_x1, ph_x, abortp);
      tma_load_4d(smem + t * kSlot + pn * kPanelB, m, &bar_a, pn * 64, t == 0 ? k0 : in0, h, b);
    }
    ph_x ^= 1;
    B128_MMA_WAIT();
    B128_MARK(0, 14);
    {  // stage dqc[I] as four fp32 panels over s5|s6 and add it to the workspace by TMA reduce:
       // chunk group cc stages panel cc and one of its lanes issues that panel's reduce
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
      store_row32_f32(s5 + cc * kPanelB, row, v);
      fence_async_smem();
      group_sync(1 + cc);
      if (issuer) {
        tma_reduce_add_3d(&m_acc_dqc, s5 + cc * kPanelB, cc * 32, i0, bh);
        bulk_commit();
      }
    }
    tc_fence_before();
    __syncthreads();
    B128_MARK(0, 15);
  }
  if (issuer || storer) bulk_wait0();

  // ---- dkc (x scale) and dvc of the key block
  {
    tc_fence_after();
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const castle_tensor_t& dt = t == 0 ? p.dkc : p.dvc;
      const float mul = t == 0 ? p.scale : 1.f;
      T* dst = reinterpret_cast<T*>(dt.ptr) + b * dt.stride_b + h * dt.stride_h + (int64_t)krow * dt.stride_n + c0;
      float v[32];
      tmem_ld32(trow + (t == 0 ? C_DKC : C_DVC) + c0, v);
      tmem_ld_wait();
      if (krow < p.N) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 q;
          q.x = Elem<T>::pack2(v[8 * j] * mul, v[8 * j + 1] * mul);
          q.y = Elem<T>::pack2(v[8 * j + 2] * mul, v[8 * j + 3] * mul);
          q.z = Elem<T>::pack2(v[8 * j + 4] * mul, v[8 * j + 5] * mul);
          q.w = Elem<T>::pack2(v[8 * j + 6] * mul, v[8 * j + 7] * mul);
          *reinterpret_cast<uint4*>(dst + j * 8) = q;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && abort_flag) atomicOr(p.status, CASTLE_STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------------------------------------
// Lookahead-gradient kernel.  It recomputes nothing: the gate A, dSu and the masked T of every (I, K) step come
// from the key/value kernel through global memory (three 32 KB tiles per step, copied as they lay in shared
// memory).  TMEM: dqu | G | scratch | scratch: with the forward state gone from this kernel, dqu[K] accumulates
// in tensor memory over the walk and is written once at the end (no reduce, and deterministic).
template <typename T>
__global__ void __launch_bounds__(kB128Threads, 1)
castle_bwd128_la_kernel(const BwdParams p, const __grid_constant__ CUtensorMap m_qc, const __grid_constant__ CUtensorMap m_qu,
                        const __grid_constant__ CUtensorMap m_ku, const __grid_constant__ CUtensorMap m_vu,
                        const __grid_constant__ CUtensorMap m_acc_dvu, const __grid_constant__ CUtensorMap m_acc_dku) {
  constexpr int FMT = Elem<T>::fmt;
  constexpr uint32_t ID_KK = make_idesc(128, 128, FMT, false, false, false);
  constexpr uint32_t ID_KM = make_idesc(128, 128, FMT, false, true, false);
  constexpr uint32_t ID_MM = make_idesc(128, 128, FMT, true, true, false);
  constexpr uint32_t C_DQU = 0, C_G = 128, C_S = 256, C_X = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sG = smem;              // 16-bit copy of G (kept across steps)
  uint8_t* sA = sG + kSlot;        // gate A (from the key/value kernel) -> Qu[K]
  uint8_t* s0 = sA + kSlot;        // masked dT
  uint8_t* s1 = s0 + kSlot;        // Vu[I] -> Ku[I] -> dvu / dku staging
  uint8_t* s2 = s1 + kSlot;        // Qc[I] -> dvu / dku staging
  uint8_t* s3 = s2 + kSlot;        // masked T (from the key/value kernel) -> dZ
  uint8_t* s4 = s3 + kSlot;        // dSu (from the key/value kernel)
  __shared__ uint64_t bar_a, bar_v, bar_ku2, bar_qu2, bar_mma;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, cc = warp >> 2;
  const int row = quarter * 32 + lane, c0 = cc * 32;
  const int bh = p.bh0 + blockIdx.x, K = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int k0 = K * kBlkB, krow = k0 + row;
  // one lane per chunk group issues that group's reduces and, once they have read their staging panels,
  // refills the panels it owns; not thread 0, which must not be held up on its way to the next products
  const bool issuer = (quarter == 1 && lane == 0);   // threads 32, 160, 288, 416
  const uint8_t* const tile_base = p.tiles + (int64_t)blockIdx.x * p.ntiles * 3 * kSlot;

  if (tid == 0) {
    mbar_init(&bar_a, 1); mbar_init(&bar_v, 1); mbar_init(&bar_ku2, 1); mbar_init(&bar_qu2, 1); mbar_init(&bar_mma, 1);
    mbar_fence_init();
    abort_flag = 0;
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
  volatile int* abortp = &abort_flag;

  uint32_t ph_a = 0, ph_ku2 = 0, ph_qu2 = 0, ph_mma = 0;   // ph_a also serves bar_v
  const uint32_t aG = smem_u32(sG), aA = smem_u32(sA), a0 = smem_u32(s0), a1 = smem_u32(s1), a2 = smem_u32(s2),
                 a3 = smem_u32(s3), a4 = smem_u32(s4);

  auto tile_of = [&](int I) { return tile_base + ((int64_t)I * (I + 1) / 2 + K) * 3 * kSlot; };
  if (tid == 0) {  // the first block's tiles; later ones are fetched inside the step before (see the last phase)
    const int il = (p.nblk - 1) * kBlkB;
    const uint8_t* t = tile_of(p.nblk - 1);
    mbar_expect_tx(&bar_a, 3 * kSlot);
    bulk_g2s(sA, t, kSlot, &bar_a);
    bulk_g2s(s4, t + kSlot, kSlot, &bar_a);
    bulk_g2s(s3, t + 2 * kSlot, kSlot, &bar_a);
    mbar_expect_tx(&bar_v, 2 * kSlot);
    load_tile<2>(s1, &m_vu, &bar_v, il, h, b);
    load_tile<2>(s2, &m_qc, &bar_v, il, h, b);
  }
  for (int I = p.nblk - 1; I >= K; --I) {
    const int i0 = I * kBlkB;
    const bool first = (I == p.nblk - 1);
    // Vu[I] and Qc[I] go into the panels that held the dku staging of the step before: each issuing lane
    // waits until its reduce has read its panel and refills exactly that panel (nobody else touches it),
    // so no barrier is needed.  The three hand-over tiles were fetched during the step before.
    if (issuer && I < p.nblk - 1) {
      bulk_wait_read0();
      tma_load_4d((cc < 2 ? s1 : s2) + (cc & 1) * kPanelB, cc < 2 ? &m_vu : &m_qc, &bar_v, (cc & 1) * 64, i0, h, b);
    }

    // ---- dA/scale = Gb @ Vu[I]^T + dSu^T @ Tm;  dT = dSu @ A;  G += dSu^T @ Qc[I]
    if (tid == 0) {
      mbar_wait(&bar_a, ph_a, abortp);
      mbar_wait(&bar_v, ph_a, abortp);
      tc_fence_after();
      mbar_expect_tx(&bar_ku2, kSlot);   // armed here; the loads are issued below by two other lanes
      if (!first) gemm_kk_t<2>(tmem + C_S, aG, a1, ID_KK, false);
      gemm_mm_t<8>(tmem + C_S, a4, a3, ID_MM, !first);
      gemm_km_t<8>(tmem + C_X, a4, aA, ID_KM, false);
      mma_commit(&bar_mma);  // dA and dT: the pass below overlaps the G update, which the next commit covers
      gemm_mm_t<8>(tmem + C_G, a4, a2, ID_MM, !first);
    }
    ph_a ^= 1;
    B128_MARK(256, 0);
    B128_MMA_WAIT();
    B128_MARK(256, 1);
    // Vu[I] is consumed (dSu is not yet: the G update still reads it): Ku[I] -> s1 for the dqu product
    if (lane == 0 && (warp == 5 || warp == 9)) tma_load_4d(s1 + (warp == 9) * kPanelB, &m_ku, &bar_ku2, (warp == 9) * 64, i0, h, b);
    {  // dZ = dA A (1 - A) -> s3 (over the masked T); masked dT -> s0
      float v[32], a[32];
      tmem_ld32(trow + C_S + c0, v);
      load_row32<T>(sA, kPanelB, row, c0, a);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = v[j] * p.scale * a[j] * (1.f - a[j]);
      store_row32<T>(s3, kPanelB, row, c0, v);
      tmem_ld32(trow + C_X + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      store_row32<T>(s0, kPanelB, row, c0, v);
    }
    B128_SYNC();
    B128_MARK(256, 2);

    // ---- dvu[I] (unscaled) = A^T @ Gb + dT^T @ Qc[I];  dqu[K] += dZ @ Ku[I]
    if (tid == 0) {
      tc_fence_after();
      mbar_expect_tx(&bar_qu2, kSlot);   // armed here; the loads are issued below by two other lanes
      if (!first) gemm_mm_t<8>(tmem + C_X, aA, aG, ID_MM, false);
      gemm_mm_t<8>(tmem + C_X, a0, a2, ID_MM, !first);
      mbar_wait(&bar_ku2, ph_ku2, abortp);
      gemm_km_t<8>(tmem + C_DQU, a3, a1, ID_KM, !first);
      mma_commit(&bar_mma);
    }
    ph_ku2 ^= 1;
    B128_MMA_WAIT();
    B128_MARK(256, 3);
    // the gate is consumed: Qu[K] -> sA for the dku product
    if (lane == 0 && (warp == 5 || warp == 9)) tma_load_4d(sA + (warp == 9) * kPanelB, &m_qu, &bar_qu2, (warp == 9) * 64, k0, h, b);
    {  // stage dvu[I] over s1|s2 (four fp32 panels, one per chunk group)
      float v[32];
      tmem_ld32(trow + C_X + c0, v);
      tmem_ld_wait();
      store_row32_f32((cc < 2 ? s1 : s2) + (cc & 1) * kPanelB, row, v);
    }
    fence_async_smem();
    group_sync(1 + cc);
    if (issuer) {  // chunk group cc staged panel cc; its lane issues that panel's reduce
      tma_reduce_add_3d(&m_acc_dvu, (cc < 2 ? s1 : s2) + (cc & 1) * kPanelB, cc * 32, i0, bh);
      bulk_commit();
    }
    tc_fence_before();
    __syncthreads();
    B128_MARK(256, 4);

    // ---- dku[I] (unscaled) = dZ^T @ Qu[K]
    if (tid == 0) {
      mbar_wait(&bar_qu2, ph_qu2, abortp);
      tc_fence_after();
      gemm_mm_t<8>(tmem + C_X, a3, aA, ID_MM, false);
      mma_commit(&bar_mma);
      if (I > K) {  // the next step's tiles: three fetched below, two at the top of the next step
        mbar_expect_tx(&bar_a, 3 * kSlot);
        mbar_expect_tx(&bar_v, 2 * kSlot);
      }
    }
    ph_qu2 ^= 1;
    if (issuer) bulk_wait_read0();  // this lane's dvu panel has been read: its slot is free again
    B128_MMA_WAIT();
    __syncthreads();  // orders the issuing lanes' waits before everybody's staging stores
    B128_MARK(256, 5);
    // The dvu reduce has drained and the last product is done, so the slots of the
    // next step's hand-over tiles are all free: A -> sA, dSu -> s4, masked T -> s3, one 16 KB half per lane
    // of six warps; they arrive while dku is staged.
    if (lane == 0 && warp < 6 && I > K) {
      const int t = warp >> 1, pn = warp & 1;
      uint8_t* dst = (t == 0 ? sA : t == 1 ? s4 : s3) + pn * kPanelB;
      bulk_g2s(dst, tile_of(I - 1) + t * kSlot + pn * kPanelB, kPanelB, &bar_a);
    }
    {
      float v[32];
      tmem_ld32(trow + C_X + c0, v);
      tmem_ld_wait();
      store_row32_f32((cc < 2 ? s1 : s2) + (cc & 1) * kPanelB, row, v);
      // 16-bit copy of G including block I, for the next (lower) block
      tmem_ld32(trow + C_G + c0, v);
      tmem_ld_wait();
      store_row32<T>(sG, kPanelB, row, c0, v);
    }
    fence_async_smem();
    group_sync(1 + cc);
    if (issuer) {
      tma_reduce_add_3d(&m_acc_dku, (cc < 2 ? s1 : s2) + (cc & 1) * kPanelB, cc * 32, i0, bh);
      bulk_commit();
    }
    tc_fence_before();
    __syncthreads();
    B128_MARK(256, 6);
  }
  if (issuer) bulk_wait0();

  // ---- dqu (x scale) of the key block
  {
    tc_fence_after();
    T* dst = reinterpret_cast<T*>(p.dqu.ptr) + b * p.dqu.stride_b + h * p.dqu.stride_h + (int64_t)krow * p.dqu.stride_n + c0;
    float v[32];
    tmem_ld32(trow + C_DQU + c0, v);
    tmem_ld_wait();
    if (krow < p.N) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 q;
        q.x = Elem<T>::pack2(v[8 * j] * p.scale, v[8 * j + 1] * p.scale);
        q.y = Elem<T>::pack2(v[8 * j + 2] * p.scale, v[8 * j + 3] * p.scale);
        q.z = Elem<T>::pack2(v[8 * j + 4] * p.scale, v[8 * j + 5] * p.scale);
        q.w = Elem<T>::pack2(v[8 * j + 6] * p.scale, v[8 * j + 7] * p.scale);
        *reinterpret_cast<uint4*>(dst + j * 8) = q;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && abort_flag) atomicOr(p.status, CASTLE_STATUS_WAIT_TIMEOUT);
}

#undef B128_MMA_WAIT
#undef B128_SYNC

// Scratch of the tile hand-over: three 32 KB tiles per (query block, key block) step and (batch, head) pair.
// The pairs run in chunks so that it stays below 8 GiB per launch pair.
constexpr int64_t kTileScratchLimit = (int64_t)8 << 30;
size_t bwd128_pair_bytes(int nblk) { return (size_t)nblk * (nblk + 1) / 2 * 3 * kSlot; }
int bwd128_chunk_pairs(int BH, int nblk) {
  int64_t n = kTileScratchLimit / (int64_t)bwd128_pair_bytes(nblk);
  if (n < 1) n = 1;
  return (int)(n < BH ? n : BH);
}

template <typename T>
static int launch_bwd128_t(const BwdParams& p, const CUtensorMap* in, cudaStream_t st) {
  constexpr int D = 128;
  cudaError_t e = cudaFuncSetAttribute(castle_bwd128_kv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kB128Smem);
  if (e != cudaSuccess) return cuda_fail(e, "castle_bwd attribute");
  e = cudaFuncSetAttribute(castle_bwd128_la_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kB128Smem);
  if (e != cudaSuccess) return cuda_fail(e, "castle_bwd attribute");
  CUtensorMap acc[3];
  float* bases[3] = {p.acc_dqc, p.acc_dvu, p.acc_dku};
  for (int i = 0; i < 3; ++i) {
    int rc = make_tmap_f32_rows(&acc[i], bases[i], p.B * p.H, p.N, D, "gradient workspace");
    if (rc) return rc;
  }
  const int64_t rows = (int64_t)p.B * p.H * p.N;
  constexpr int RPB = 256 / (D / 8);
  e = cudaMemsetAsync(p.acc_dqc, 0, (size_t)rows * D * 3 * sizeof(float), st);
  if (e != cudaSuccess) return cuda_fail(e, "castle_bwd memset");
  castle_bwd_delta_kernel<T, D><<<(unsigned)((rows + RPB - 1) / RPB), 256, 0, st>>>(p);
  const int BH = p.B * p.H, chunk = p.chunk_pairs;
  ev_start(CASTLE_KERNEL_BWD, st);
  for (int bh0 = 0; bh0 < BH; bh0 += chunk) {
    BwdParams q = p;
    q.bh0 = bh0;
    q.ntiles = (int64_t)p.nblk * (p.nblk + 1) / 2;
    dim3 grid(BH - bh0 < chunk ? BH - bh0 : chunk, p.nblk);
    // in[]: qc, kc, vc, qu, ku, vu, dout
    castle_bwd128_kv_kernel<T><<<grid, kB128Threads, kB128Smem, st>>>(q, in[0], in[1], in[2], in[3], in[4], in[5], in[6], acc[0]);
    castle_bwd128_la_kernel<T><<<grid, kB128Threads, kB128Smem, st>>>(q, in[0], in[3], in[4], in[5], acc[1], acc[2]);
  }
  ev_stop(CASTLE_KERNEL_BWD, st);
  castle_bwd_finish_kernel<T, D, 3><<<(unsigned)((rows + RPB - 1) / RPB), 256, 0, st>>>(p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_bwd launch");
}

int launch_bwd128(const BwdParams& p, int dtype, const CUtensorMap* in_maps, cudaStream_t st) {
  return dtype == CASTLE_BF16 ? launch_bwd128_t<__nv_bfloat16>(p, in_maps, st) : launch_bwd128_t<__half>(p, in_maps, st);
}

}  // namespace castle
