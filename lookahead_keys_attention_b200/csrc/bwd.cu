// CASTLE parallel backward for sm_100a (dim_head 64).
//
// One CTA owns a block K of 128 keys and walks the query blocks I from the last
// one DOWN to K, recomputing the scores flash-style.  Two 128 x d fp32 states
// live in tensor memory for the whole walk:
//   W_K  the forward's lookahead state.  It starts as the forward's final state
//        (= U[K], saved unrounded) and block I is peeled off with a negated
//        product, W_K -= A[K,I] @ Vu[I], so that before the scores of block I
//        are rebuilt it equals what the forward saw there.
//   G_K  = sum_{I' > I} dSu[I',K]^T @ Qc[I']: everything later queries
//        contribute to d(loss)/d(W_K); it yields dA and dvu for block I.
// dkc, dvc and dqu of the key block accumulate in tensor memory as well and are
// written once at the end.  The gradients indexed by the query/position block
// (dqc, dvu, dku) are summed over key blocks with TMA reduce-adds (fp32) into a
// workspace that a last kernel scales and casts.  A thread owns 32 consecutive
// columns of one accumulator row; the soft-max statistics (lse, delta) of its
// row sit in registers.
//
// Shared memory (224 KB) is time-shared: the 128x128 16-bit operands the
// threads produce (gate A, masked T, P, dS, dSu, dZ, dT) rotate through four
// 32 KB slots, two of which overlay input tiles that are dead by then
// (slot 3 over Vc|dO holds dS then dT, slot 4 over Ku|spare holds P then dSu).
#include "bwd_common.cuh"

namespace castle {

constexpr int kBwdThreads = 512;
constexpr int kPrefetchTid = 384;

// Optional phase timing (debug builds only): thread 0 of CTA (0,0) stores clock64() at each phase
// boundary of its first steps behind the fp32 workspace, which the host dumps.
#ifdef CASTLE_PHASE_TIMING
#define BPHASE_MARK(i) do { if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && tstep < 8) p.timing[tstep * 32 + (i)] = clock64(); } while (0)
#else
#define BPHASE_MARK(i) do { } while (0)
#endif

// 512 threads: warp w works on TMEM lanes 32*(w%4).. and on the 32-column chunk w/4 of a
// 128-column accumulator, so thread (row, chunk) owns 32 values of every 128x128 tile.
// One 128 x 64 fp32 accumulator tile from tensor memory into two swizzled 128 x 32 staging panels.
__device__ __forceinline__ void stage_f32_tile(uint32_t taddr, uint8_t* panel0, uint8_t* panel1, uint32_t row) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    float v[32];
    tmem_ld32(taddr + c * 32, v);
    tmem_ld_wait();
    store_row32_f32(c == 0 ? panel0 : panel1, row, v);
  }
}
// Timing experiments only (never in the shipped library): drop the reduces to see what they cost.
#ifdef CASTLE_TIMING_SKIP_REDUCE
#define tma_reduce_add_3d(...) do { } while (0)
#endif

template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
castle_bwd_kernel(const BwdParams p, const __grid_constant__ CUtensorMap m_qc, const __grid_constant__ CUtensorMap m_kc,
                  const __grid_constant__ CUtensorMap m_vc, const __grid_constant__ CUtensorMap m_qu,
                  const __grid_constant__ CUtensorMap m_ku, const __grid_constant__ CUtensorMap m_vu,
                  const __grid_constant__ CUtensorMap m_do, const __grid_constant__ CUtensorMap m_acc_dqc,
                  const __grid_constant__ CUtensorMap m_acc_dvu, const __grid_constant__ CUtensorMap m_acc_dku) {
  static_assert(D == 64, "this kernel is laid out for dim_head 64");
  constexpr uint32_t OPB = kPanelB;          // one d-wide operand tile (16 KB)
  constexpr uint32_t SQB = 2 * kPanelB;      // one 128x128 tile (32 KB)
  constexpr int FMT = Elem<T>::fmt;
  constexpr uint32_t ID_SQ_KK = make_idesc(128, 128, FMT, false, false, false);
  constexpr uint32_t ID_SQ_KM = make_idesc(128, 128, FMT, false, true, false);
  constexpr uint32_t ID_SQ_MM = make_idesc(128, 128, FMT, true, true, false);
  constexpr uint32_t ID_D_KM = make_idesc(128, D, FMT, false, true, false);
  constexpr uint32_t ID_D_KM_NEG = make_idesc(128, D, FMT, false, true, true);
  constexpr uint32_t ID_D_MM = make_idesc(128, D, FMT, true, true, false);
  constexpr float kLog2e = 1.4426950408889634f;
  // tensor-memory columns
  constexpr uint32_t C_W = 0, C_G = 64, C_DKC = 128, C_DVC = 192, C_DQU = 256, C_S = 320, C_X = 448;
  constexpr uint32_t C_X2 = C_S, C_X3 = C_S + 64;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQu = smem;                 // resident
  uint8_t* sKc = sQu + OPB;            // resident
  uint8_t* sQc = sKc + OPB;            // per step
  uint8_t* sVu = sQc + OPB;            // per step
  uint8_t* sVD = sVu + OPB;            // [Vc | dO] per step, later slot 3: dS -> dSu -> dT
  uint8_t* sVc = sVD;
  uint8_t* sdO = sVD + OPB;
  uint8_t* sKP = sVD + SQB;            // [Ku | spare], later slot 4: P, then Ku again in the first half
  uint8_t* sWb = sKP + SQB;
  uint8_t* sGb = sWb + OPB;
  uint8_t* sA = sGb + OPB;             // slot 1: gate A
  uint8_t* sT = sA + SQB;              // slot 2: masked T, later dZ
  __shared__ uint64_t bar_res, bar_load, bar_vd, bar_ku, bar_mma, bar_x1, bar_x2, bar_kn;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, cc = warp >> 2;
  const int row = quarter * 32 + lane;
  const int c0 = cc * 32;
  const int bh = blockIdx.x, K = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int k0 = K * kBlkB, krow = k0 + row;

  if (tid == 0) {
    mbar_init(&bar_res, 1); mbar_init(&bar_load, 1); mbar_init(&bar_vd, 1); mbar_init(&bar_ku, 1); mbar_init(&bar_mma, 1);
    mbar_init(&bar_x1, 1); mbar_init(&bar_x2, 1); mbar_init(&bar_kn, 1);
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
    mbar_expect_tx(&bar_res, 2 * OPB);
    tma_load_4d(sQu, &m_qu, &bar_res, 0, k0, h, b);
    tma_load_4d(sKc, &m_kc, &bar_res, 0, k0, h, b);
    // first step's Qc, Vu, Ku; later steps prefetch theirs at the end of the step before
    mbar_expect_tx(&bar_kn, OPB);
    tma_load_4d(sKP, &m_ku, &bar_kn, 0, (p.nblk - 1) * kBlkB, h, b);
    mbar_expect_tx(&bar_load, 2 * OPB);
    tma_load_4d(sQc, &m_qc, &bar_load, 0, (p.nblk - 1) * kBlkB, h, b);
    tma_load_4d(sVu, &m_vu, &bar_load, 0, (p.nblk - 1) * kBlkB, h, b);
  }
  // W_K starts as the forward's final state
  if (c0 < D) {
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
  mbar_wait(&bar_res, 0, abortp);
  tc_fence_before();
  __syncthreads();

  uint32_t ph_load = 0, ph_vd = 0, ph_ku = 0, ph_mma = 0, ph_x = 0;
  const uint32_t aQu = smem_u32(sQu), aKc = smem_u32(sKc), aQc = smem_u32(sQc), aVu = smem_u32(sVu),
                 aVc = smem_u32(sVc), adO = smem_u32(sdO), aKP = smem_u32(sKP), aVD = smem_u32(sVD),
                 aWb = smem_u32(sWb), aGb = smem_u32(sGb), aA = smem_u32(sA), aT = smem_u32(sT);
  const float sl2 = p.scale * kLog2e;

#define MMA_WAIT()                       \
  mbar_wait(&bar_mma, ph_mma, abortp);   \
  ph_mma ^= 1;                           \
  tc_fence_after();
#define SMEM_TO_MMA_SYNC() \
  fence_async_smem();      \
  tc_fence_before();       \
  __syncthreads();

  float lse_nx = 0.f, delta_nx = 0.f;
  if ((p.nblk - 1) * kBlkB + row < p.N) {
    lse_nx = p.lse[(int64_t)bh * p.N + (p.nblk - 1) * kBlkB + row];
    delta_nx = p.delta[(int64_t)bh * p.N + (p.nblk - 1) * kBlkB + row];
  }
  for (int I = p.nblk - 1; I >= K; --I) {
    const int i0 = I * kBlkB, irow = i0 + row;
    const bool diag = (I == K), first = (I == p.nblk - 1);
    const bool rvalid = irow < p.N;
#ifdef CASTLE_PHASE_TIMING
    const int tstep = p.nblk - 1 - I;
#endif
    BPHASE_MARK(0);

    // the row statistics were fetched one step ahead (their latency hides behind the step before)
    const float lse_b = lse_nx * kLog2e, delta_i = delta_nx;
    if (I > K) {
      const int64_t nrow = (int64_t)bh * p.N + irow - kBlkB;   // rows of block I-1 always exist
      lse_nx = p.lse[nrow];
      delta_nx = p.delta[nrow];
    }
    // ---- M1: Z = Qu[K] @ Ku[I]^T   (Ku[I] was fetched during the last phase of the step before)
    if (tid == 0) {
      mbar_wait(&bar_kn, ph_load, abortp);
      BPHASE_MARK(1);
      tc_fence_after();
      gemm_kk_t<1>(tmem + C_S, aQu, aKP, ID_SQ_KK, false);
      mma_commit(&bar_mma);
    }
    MMA_WAIT();
    BPHASE_MARK(2);
    {  // gate A (rows k, columns j), zero unless j > k
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = sigmoid_t<T>(v[j] * p.scale);
      if (diag) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j > row) ? v[j] : 0.f;
      }
      store_row32<T>(sA, kPanelB, row, c0, v);
    }
    SMEM_TO_MMA_SYNC();
    BPHASE_MARK(3);

    // ---- M2: peel W_K -= A @ Vu[I];  T = Qc[I] @ Vu[I]^T
    if (tid == 0) {
      mbar_wait(&bar_load, ph_load, abortp);   // Qc[I], Vu[I]
      BPHASE_MARK(21);
      tc_fence_after();
      gemm_km_t<8>(tmem + C_W, aA, aVu, ID_D_KM_NEG, true);
      gemm_kk_t<1>(tmem + C_S, aQc, aVu, ID_SQ_KK, false);
      mma_commit(&bar_mma);
    }
    // The reduces of the step before must have finished reading their staging tiles before these are
    // written again.  A reduce takes a few thousand cycles to drain, so each issuing lane waits for its
    // own as late as the first overwrite allows: here for dqc and dku (Wb and slot 2 are written by the
    // pass below), after the next products are issued for dvu (Vc|dO is re-loaded there).
    if ((cc == 1 || cc == 2) && quarter == 0 && lane == 0) bulk_wait_read0();
    MMA_WAIT();
    BPHASE_MARK(22);
    __syncthreads();
    BPHASE_MARK(4);
    {  // masked T (rows i, columns j <= i), unscaled
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      store_row32<T>(sT, kPanelB, row, c0, v);
    }
    if (c0 < D) {  // 16-bit copy of the peeled state
      float v[32];
      tmem_ld32(trow + C_W + c0, v);
      tmem_ld_wait();
      store_row32<T>(sWb, kPanelB, row, c0, v);
    }
    SMEM_TO_MMA_SYNC();
    BPHASE_MARK(5);

    // ---- M3: Su/scale = Qc[I] @ Wb^T + Tm @ A^T
    if (tid == 0) {
      tc_fence_after();
      if (!diag) gemm_kk_t<1>(tmem + C_S, aQc, aWb, ID_SQ_KK, false);
      gemm_kk_t<2>(tmem + C_S, aT, aA, ID_SQ_KK, !diag);
      mma_commit(&bar_mma);
      bulk_wait_read0();   // this thread's dvu reduce of the step before has read Vc|dO's slot
      mbar_expect_tx(&bar_vd, 2 * OPB);
      tma_load_4d(sVc, &m_vc, &bar_vd, 0, k0, h, b);   // needed at the fifth phase
      tma_load_4d(sdO, &m_do, &bar_vd, 0, i0, h, b);
    }
    MMA_WAIT();
    BPHASE_MARK(6);
    uint32_t dpk[16];  // silu'(Su), later dSu, two 16-bit values per register
    uint32_t ppk[16];  // P
    {
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float su0 = v[j] * p.scale, su1 = v[j + 1] * p.scale;
        float g0 = sigmoid_t<T>(su0), g1 = sigmoid_t<T>(su1);
        v[j] = -v[j] * g0;          // -silu(su) / scale
        v[j + 1] = -v[j + 1] * g1;
        dpk[j / 2] = Elem<T>::pack2(g0 * (1.f + su0 * (1.f - g0)), g1 * (1.f + su1 * (1.f - g1)));
      }
      tmem_st32(trow + C_S + c0, v);
      tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    BPHASE_MARK(7);

    // ---- M4: S/scale = penalty + Qc[I] @ Kc[K]^T
    if (tid == 0) {
      tc_fence_after();
      gemm_kk_t<1>(tmem + C_S, aQc, aKc, ID_SQ_KK, true);
      mma_commit(&bar_mma);
    }
    MMA_WAIT();
    BPHASE_MARK(8);
    {  // P = exp(S - lse) (rows i, columns k); into slot 4 over Ku
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
      store_row32<T>(sKP, kPanelB, row, c0, v);
    }
    SMEM_TO_MMA_SYNC();
    BPHASE_MARK(9);

    // ---- M5: dvc += P^T @ dO[I];  dP = dO[I] @ Vc[K]^T
    if (tid == 0) {
      tc_fence_after();
      mbar_wait(&bar_vd, ph_vd, abortp);
      gemm_mm_t<8>(tmem + C_DVC, aKP, adO, ID_D_MM, !first);
      gemm_kk_t<1>(tmem + C_S, adO, aVc, ID_SQ_KK, false);
      mma_commit(&bar_mma);
    }
    MMA_WAIT();
    BPHASE_MARK(10);
    ph_vd ^= 1;
    {  // dS = P * (dP - delta) -> slot 3 (over Vc|dO); dSu = -dS * silu'(Su) -> slot 4 (over P)
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
      store_row32<T>(sVD, kPanelB, row, c0, v);
      store_row32<T>(sKP, kPanelB, row, c0, w);
    }
    SMEM_TO_MMA_SYNC();
    BPHASE_MARK(11);

    // ---- M6: dkc += dS^T @ Qc[I];  X = dS @ Kc[K] + dSu @ Wb;  dA/scale = Gb @ Vu[I]^T + dSu^T @ Tm
    if (tid == 0) {
      tc_fence_after();
      // dA first and committed alone: the pass that turns it into dZ only needs dA, so it overlaps the
      // products issued after the commit (dkc, X), which the next phase's commit covers
      if (!first) gemm_kk_t<1>(tmem + C_S, aGb, aVu, ID_SQ_KK, false);
      gemm_mm_t<8>(tmem + C_S, aKP, aT, ID_SQ_MM, !first);
      mma_commit(&bar_mma);
      gemm_mm_t<8>(tmem + C_DKC, aVD, aQc, ID_D_MM, !first);
      gemm_km_t<8>(tmem + C_X, aVD, aKc, ID_D_KM, false);
      if (!diag) gemm_km_t<8>(tmem + C_X, aKP, aWb, ID_D_KM, true);
    }
    MMA_WAIT();
    BPHASE_MARK(12);
    {  // dZ = dA * A * (1 - A) -> slot 2 (over Tm)
      float v[32], a[32];
      tmem_ld32(trow + C_S + c0, v);
      load_row32<T>(sA, kPanelB, row, c0, a);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = v[j] * p.scale * a[j] * (1.f - a[j]);
      store_row32<T>(sT, kPanelB, row, c0, v);
    }
    SMEM_TO_MMA_SYNC();
    BPHASE_MARK(13);

    // ---- M8: G += dSu^T @ Qc[I];  dT = dSu @ A
    if (tid == 0) {
      tc_fence_after();
      // dT first and committed alone: masking it overlaps the G update, which the next phase's first
      // commit covers (dSu stays in slot 4 until then)
      gemm_km_t<8>(tmem + C_S, aKP, aA, ID_SQ_KM, false);
      mma_commit(&bar_mma);
      gemm_mm_t<8>(tmem + C_G, aKP, aQc, ID_D_MM, !first);
    }
    MMA_WAIT();
    BPHASE_MARK(14);
    if (tid == 0) {  // Ku[I] comes back for the dqu product, into Wb's slot (its last reader is covered by the commit above)
      mbar_expect_tx(&bar_ku, OPB);
      tma_load_4d(sWb, &m_ku, &bar_ku, 0, i0, h, b);
    }
    {  // masked dT (rows i, columns j <= i) -> slot 3 (over dS)
      float v[32];
      tmem_ld32(trow + C_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      store_row32<T>(sVD, kPanelB, row, c0, v);
    }
    SMEM_TO_MMA_SYNC();
    BPHASE_MARK(15);

    // ---- M9: dqu += dZ @ Ku[I];  X2 = dT^T @ Qc[I] + A^T @ Gb;  X += dT @ Vu[I];  X3 = dZ^T @ Qu[K]
    // Three commits.  The first covers every product that reads a per-step input tile, so the next
    // step's Qc, Vu, Ku are fetched right behind it, ahead of the reduces in the TMA queue (a reduce
    // takes thousands of cycles to drain and loads issued behind one wait for it).  After each commit the
    // query-block gradient it completes is staged as fp32 panels in an operand slot that is dead by then
    // and handed to a TMA reduce (whole lines at L2 instead of scattered atomics): chunk group 1 takes
    // dqc (into Wb + the spare half of slot 4), group 2 dku (into slot 2, which held dZ), group 0 - the
    // issuing thread's, busy until the end - dvu (into Vc|dO, which held dT and is re-loaded last in the
    // next step); group 3 fetches the next tiles and refreshes the 16-bit copy of G.
    if (tid == 0) {
      tc_fence_after();
      gemm_mm_t<8>(tmem + C_X2, aVD, aQc, ID_D_MM, false);
      gemm_km_t<8>(tmem + C_X, aVD, aVu, ID_D_KM, true);
      mbar_wait(&bar_ku, ph_ku, abortp);
      gemm_km_t<8>(tmem + C_DQU, aT, aWb, ID_D_KM, !first);
      mma_commit(&bar_x1);
      gemm_mm_t<8>(tmem + C_X3, aT, aQu, ID_D_MM, false);
      mma_commit(&bar_x2);
      if (!first) gemm_mm_t<8>(tmem + C_X2, aA, aGb, ID_D_MM, true);
      mma_commit(&bar_mma);
    }
    ph_ku ^= 1;
    const bool issuer = (quarter == 0 && lane == 0);   // threads 0, 128, 256 issue the reduces
    if (cc == 1) {
      mbar_wait(&bar_x1, ph_x, abortp);
      tc_fence_after();
      stage_f32_tile(trow + C_X, sWb, sKP + kPanelB, row);
      fence_async_smem();
      group_sync(1);
      if (issuer) {
        tma_reduce_add_3d(&m_acc_dqc, sWb, 0, i0, bh);
        tma_reduce_add_3d(&m_acc_dqc, sKP + kPanelB, 32, i0, bh);
        bulk_commit();
      }
    } else if (cc == 2) {
      mbar_wait(&bar_x2, ph_x, abortp);
      tc_fence_after();
      stage_f32_tile(trow + C_X3, sT, sT + kPanelB, row);
      fence_async_smem();
      group_sync(2);
      if (issuer) {
        tma_reduce_add_3d(&m_acc_dku, sT, 0, i0, bh);
        tma_reduce_add_3d(&m_acc_dku, sT + kPanelB, 32, i0, bh);
        bulk_commit();
      }
    } else if (cc == 3) {
      mbar_wait(&bar_x1, ph_x, abortp);   // Qc[I], Vu[I], Ku[I] are consumed
      if (tid == kPrefetchTid && I > K) {
        const int in0 = i0 - kBlkB;
        mbar_expect_tx(&bar_kn, OPB);
        tma_load_4d(sKP, &m_ku, &bar_kn, 0, in0, h, b);
        mbar_expect_tx(&bar_load, 2 * OPB);
        tma_load_4d(sQc, &m_qc, &bar_load, 0, in0, h, b);
        tma_load_4d(sVu, &m_vu, &bar_load, 0, in0, h, b);
      }
    }
    ph_x ^= 1;
    ph_load ^= 1;
    BPHASE_MARK(16);
    MMA_WAIT();
    BPHASE_MARK(17);
    if (cc == 0) {
      stage_f32_tile(trow + C_X2, sVD, sVD + kPanelB, row);
      fence_async_smem();
      group_sync(3);
      if (issuer) {
        tma_reduce_add_3d(&m_acc_dvu, sVD, 0, i0, bh);
        tma_reduce_add_3d(&m_acc_dvu, sVD + kPanelB, 32, i0, bh);
        bulk_commit();
      }
    } else if (cc == 3) {  // 16-bit copy of G including block I, for the next (lower) block
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        float v[32];
        tmem_ld32(trow + C_G + c * 32, v);
        tmem_ld_wait();
        store_row32<T>(sGb, kPanelB, row, c * 32, v);
      }
    }
    BPHASE_MARK(18);
    BPHASE_MARK(19);
    SMEM_TO_MMA_SYNC();
    BPHASE_MARK(20);
  }
  if (cc < 3 && quarter == 0 && lane == 0) bulk_wait0();
#undef MMA_WAIT
#undef SMEM_TO_MMA_SYNC

  // ---- key-block gradients: dkc (x scale), dvc, dqu (x scale); one chunk group each
  if (cc < 3) {
    tc_fence_after();
    const uint32_t col = (cc == 0) ? C_DKC : (cc == 1 ? C_DVC : C_DQU);
    const castle_tensor_t& dt = (cc == 0) ? p.dkc : (cc == 1 ? p.dvc : p.dqu);
    const float mul = (cc == 1) ? 1.f : p.scale;
    T* dst = reinterpret_cast<T*>(dt.ptr) + b * dt.stride_b + h * dt.stride_h + (int64_t)krow * dt.stride_n;
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      float v[32];
      tmem_ld32(trow + col + c * 32, v);
      tmem_ld_wait();
      if (krow < p.N) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 q;
          q.x = Elem<T>::pack2(v[8 * j] * mul, v[8 * j + 1] * mul);
          q.y = Elem<T>::pack2(v[8 * j + 2] * mul, v[8 * j + 3] * mul);
          q.z = Elem<T>::pack2(v[8 * j + 4] * mul, v[8 * j + 5] * mul);
          q.w = Elem<T>::pack2(v[8 * j + 6] * mul, v[8 * j + 7] * mul);
          *reinterpret_cast<uint4*>(dst + c * 32 + j * 8) = q;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && abort_flag) atomicOr(p.status, CASTLE_STATUS_WAIT_TIMEOUT);
}

template <typename T, int D>
static int launch_bwd(const BwdParams& p, const CUtensorMap* maps, cudaStream_t st) {
  constexpr size_t smem = 7 * kPanelB + 4 * 2 * kPanelB - kPanelB + 1024;  // 224 KB + alignment slack
  {  // per device, so set on every call (cheap)
    cudaError_t e = cudaFuncSetAttribute(castle_bwd_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "castle_bwd attribute");
  }
  const int64_t rows = (int64_t)p.B * p.H * p.N;
  constexpr int RPB = 256 / (D / 8);
  cudaError_t e = cudaMemsetAsync(p.acc_dqc, 0, (size_t)rows * D * 3 * sizeof(float), st);
  if (e != cudaSuccess) return cuda_fail(e, "castle_bwd memset");
  castle_bwd_delta_kernel<T, D><<<(unsigned)((rows + RPB - 1) / RPB), 256, 0, st>>>(p);
  dim3 grid(p.B * p.H, p.nblk);
  ev_start(CASTLE_KERNEL_BWD, st);
  castle_bwd_kernel<T, D><<<grid, kBwdThreads, smem, st>>>(p, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], maps[6],
                                                         maps[7], maps[8], maps[9]);
  ev_stop(CASTLE_KERNEL_BWD, st);
  castle_bwd_finish_kernel<T, D, 3><<<(unsigned)((rows + RPB - 1) / RPB), 256, 0, st>>>(p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_bwd launch");
}

}  // namespace castle

using namespace castle;

// fp32 accumulators dqc, dvu, dku and delta; at dim_head 128 rounded up so that the tile scratch behind them
// stays 1 KB aligned
static size_t bwd_acc_bytes(const castle_problem_t* p) {
  int64_t rows = (int64_t)p->batch * p->heads * p->seq_len;
  size_t b = (size_t)(rows * (3 * p->dim_head + 1) * sizeof(float));
  return p->dim_head == 128 ? (b + 1023) & ~(size_t)1023 : b;
}

extern "C" size_t castle_bwd_workspace_bytes(const castle_problem_t* p) {
  if (!p || p->seq_len <= 0 || p->batch <= 0 || p->heads <= 0) return 0;
  const int nblk = (p->seq_len + kBlkB - 1) / kBlkB;
  size_t tiles = p->dim_head == 128 ? (size_t)bwd128_chunk_pairs(p->batch * p->heads, nblk) * bwd128_pair_bytes(nblk) : 0;
  return bwd_acc_bytes(p) + tiles;
}

extern "C" int castle_bwd(const castle_problem_t* p, const castle_tensor_t* qc, const castle_tensor_t* kc,
                          const castle_tensor_t* vc, const castle_tensor_t* qu, const castle_tensor_t* ku,
                          const castle_tensor_t* vu, const castle_tensor_t* out, const castle_tensor_t* dout,
                          const float* lse, const float* w_state, const castle_tensor_t* dqc,
                          const castle_tensor_t* dkc, const castle_tensor_t* dvc, const castle_tensor_t* dqu,
                          const castle_tensor_t* dku, const castle_tensor_t* dvu, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream) {
  if (!p) return reject("castle_bwd: null problem");
  if (p->batch <= 0 || p->heads <= 0 || p->seq_len <= 0) return reject("castle_bwd: empty problem");
  if (p->dim_head != 64 && p->dim_head != 128) return reject("castle_bwd: dim_head %d not supported (64 or 128)", p->dim_head);
  if (p->dtype != CASTLE_BF16 && p->dtype != CASTLE_F16) return reject("castle_bwd: dtype %d not supported (bf16, fp16)", p->dtype);
  int nblk = (p->seq_len + kBlkB - 1) / kBlkB;
  if (nblk > 65535) return reject("castle_bwd: sequence too long");
  int rc = 0;
  const castle_tensor_t* ts[14] = {qc, kc, vc, qu, ku, vu, dout, out, dqc, dkc, dvc, dqu, dku, dvu};
  const char* names[14] = {"qc", "kc", "vc", "qu", "ku", "vu", "dout", "out", "dqc", "dkc", "dvc", "dqu", "dku", "dvu"};
  for (int i = 0; i < 14; ++i)
    if (!tensor_ok(ts[i], p->dtype, names[i], &rc)) return rc;
  if (!lse || !w_state || !status) return reject("castle_bwd: lse, w_state and status must not be null");
  // dim_head 64: the accumulators.  dim_head 128: the accumulators and the tile hand-over scratch of at least
  // one (batch, head) pair; the pairs run in chunks of as many as the scratch the caller passed holds.
  const size_t need = castle_bwd_workspace_bytes(p), acc_bytes = bwd_acc_bytes(p);
  const size_t pair_bytes = p->dim_head == 128 ? bwd128_pair_bytes(nblk) : 0;
  const size_t least = p->dim_head == 128 ? acc_bytes + pair_bytes : need;
  if (!workspace || workspace_bytes < least)
    return reject("castle_bwd: workspace too small (%zu bytes; castle_bwd_workspace_bytes says %zu, the least that works is %zu)",
                  workspace_bytes, need, least);
  if (((uintptr_t)workspace) % 16) return reject("castle_bwd: workspace not 16-byte aligned");

  BwdParams bp;
  bp.B = p->batch; bp.H = p->heads; bp.N = p->seq_len; bp.nblk = nblk; bp.scale = p->scale;
  bp.lse = lse; bp.w_state = w_state;
  int64_t rows = (int64_t)p->batch * p->heads * p->seq_len;
  // dim_head 128: the tile hand-over scratch follows the accumulators
  bp.tiles = (uint8_t*)workspace + acc_bytes;
  bp.ntiles = 0; bp.bh0 = 0; bp.chunk_pairs = 0;
  if (p->dim_head == 128) {
    size_t fit = (workspace_bytes - acc_bytes) / pair_bytes;
    bp.chunk_pairs = (int)(fit < (size_t)(p->batch * p->heads) ? fit : (size_t)(p->batch * p->heads));
  }
  bp.acc_dqc = (float*)workspace;
  bp.acc_dvu = bp.acc_dqc + rows * p->dim_head;
  bp.acc_dku = bp.acc_dvu + rows * p->dim_head;
  bp.delta = bp.acc_dku + rows * p->dim_head;
  bp.out = *out; bp.dout = *dout;
  bp.dqc = *dqc; bp.dkc = *dkc; bp.dvc = *dvc; bp.dqu = *dqu; bp.dku = *dku; bp.dvu = *dvu;
  bp.status = status;
#ifdef CASTLE_PHASE_TIMING
  bp.timing = (long long*)((char*)workspace + need);  // the caller leaves 8 KB beyond what castle_bwd_workspace_bytes asks for
  if (bp.chunk_pairs > bwd128_chunk_pairs(p->batch * p->heads, nblk)) bp.chunk_pairs = bwd128_chunk_pairs(p->batch * p->heads, nblk);
#endif
  CUtensorMap maps[10];
  for (int i = 0; i < 7; ++i) {
    rc = make_tmap_16bit(&maps[i], ts[i], p->dtype, p->batch, p->heads, p->seq_len, p->dim_head, kBlkB, names[i]);
    if (rc) return rc;
  }
  float* accs[3] = {bp.acc_dqc, bp.acc_dvu, bp.acc_dku};
  for (int i = 0; i < 3; ++i) {
    rc = make_tmap_f32_rows(&maps[7 + i], accs[i], p->batch * p->heads, p->seq_len, p->dim_head, "gradient workspace");
    if (rc) return rc;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (p->dim_head == 128) return launch_bwd128(bp, p->dtype, maps, st);
  if (p->dtype == CASTLE_BF16) return launch_bwd<__nv_bfloat16, 64>(bp, maps, st);
  return launch_bwd<__half, 64>(bp, maps, st);
}
