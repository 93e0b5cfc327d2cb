// CASTLE parallel forward for sm_100a.
//
// The reference evaluates Su = T @ A^T as an (N x N) x (N x N) product, O(N^3)
// per head.  Here each CTA owns one block K of 128 keys and walks the query
// blocks I = K, K+1, ... keeping the running lookahead state
//     W_K = sum_{J < I} A[K,J] @ Vu[J]          (128 x d, fp32, in tensor memory)
// so that
//     Su[I,K] = Qc[I] @ W_K^T + tril(T[I,I]) @ A[K,I]^T
// costs O(N^2 d) in total.  Per (I,K) step the CTA issues seven tcgen05 products
// (Z, W update, T, Su main, Su in-block term, Sc, P@Vc), all with fp32
// accumulators in TMEM and 16-bit operands in 128-byte-swizzled shared memory,
// either loaded by TMA (inputs) or written by the threads (sigmoid gate A,
// masked T, the 16-bit copy of W, soft-max numerators P).  A thread owns 32
// consecutive columns of one accumulator row; row maxima and sums of the four
// threads sharing a row meet in shared memory.
//
// The soft-max over keys crosses CTAs, so each step emits an un-normalised
// partial (row max, row sum, P@Vc) and a second kernel merges the partials of a
// query block.  After the last step W_K is exactly U[K], the lookahead keys the
// decode cache stores, and (unrounded) the state the backward starts from.
#include "common.cuh"
#include "sm100.cuh"

namespace castle {

constexpr int kBlk = 128;                       // keys per CTA, queries per step
constexpr uint32_t kPanelBytes = kBlk * 128;    // [128 rows][64 x 16-bit]

struct FwdParams {
  int B, H, N, nblk;
  float scale;
  float* part_ml;   // [BH][ntiles][128][2]
  void* part_o;     // [BH][ntiles][128][D] in the operand type (un-normalised P@Vc of one tile)
  float* lse;       // [BH][N]
  float* w_state;   // [BH][N][D] or null
  castle_tensor_t u_out;  // ptr may be null
  int u_dtype;
  castle_tensor_t out;
  int32_t* status;
  int store_caches;   // also copy the Qu[K], Kc[K], Vc[K] tiles into the decode caches (prefill hand-off)
  int split_q8;       // dim_head 64: walks of 8+ query blocks are cut after split_q8/256 of their length (0 = never)
#ifdef CASTLE_PHASE_TIMING
  long long* timing;
#endif
};

__host__ __device__ inline int64_t tri(int64_t i) { return i * (i + 1) / 2; }

constexpr int kFwdThreads = 512;

// Optional phase timing (debug builds only): thread 0 of CTA (0,0) stores clock64() at each phase
// boundary of its first steps into the soft-max partial buffer's tail, which the host dumps.
#ifdef CASTLE_PHASE_TIMING
#define PHASE_MARK(i) do { if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0 && tstep < 8) p.timing[tstep * 16 + (i)] = clock64(); } while (0)
#else
#define PHASE_MARK(i) do { } while (0)
#endif

// 512 threads: warp w works on TMEM lanes 32*(w%4).. (the hardware's rule) and on the
// 32-column chunk w/4 of a 128-column accumulator, so thread (row, chunk) owns 32 values.
template <typename T, int D>
__global__ void __launch_bounds__(kFwdThreads, 1)
castle_fwd_kernel(const FwdParams p, const __grid_constant__ CUtensorMap m_qc, const __grid_constant__ CUtensorMap m_kc,
                  const __grid_constant__ CUtensorMap m_vc, const __grid_constant__ CUtensorMap m_qu,
                  const __grid_constant__ CUtensorMap m_ku, const __grid_constant__ CUtensorMap m_vu,
                  const __grid_constant__ CUtensorMap m_quc, const __grid_constant__ CUtensorMap m_kcc,
                  const __grid_constant__ CUtensorMap m_vcc) {
  constexpr int NP = D / 64;                         // panels per d-wide operand
  constexpr uint32_t OPB = NP * kPanelBytes;         // bytes of a d-wide operand tile
  constexpr uint32_t SQB = 2 * kPanelBytes;          // bytes of a 128x128 tile
  constexpr uint32_t TM_COLS = (D == 64) ? 256 : 512;
  static_assert(D == 128, "laid out for dim_head 128 (512 tensor-memory columns)");
  // accumulators W | S | O, then two 64-column areas for tiles the threads hand to the tensor cores as
  // packed 16-bit pairs (first operands read from tensor memory): the gate, later P; and the masked T
  constexpr uint32_t COL_W = 0, COL_S = D, COL_O = D + 128, COL_A = D + 256, COL_T = D + 320;
  constexpr int FMT = Elem<T>::fmt;
  constexpr uint32_t ID_SQ = make_idesc(128, 128, FMT, false, false, false);
  constexpr uint32_t ID_D = make_idesc(128, D, FMT, false, true, false);
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQu = smem;
  uint8_t* sKc = sQu + OPB;
  uint8_t* sVc = sKc + OPB;
  uint8_t* sQc = sVc + OPB;
  uint8_t* sWb = sQc + OPB;
  uint8_t* sKuA = sWb + OPB;   // Ku[I], then the gate A[K,I]; Ku[I+1] arrives once Su is done
  uint8_t* sVuT = sKuA + SQB;  // Vu[I]; Vu[I+1] arrives once Su (whose commit covers the state update) is done
  // row max / row sum exchange between the four threads of a row: 4 KB over Qc[I], which is dead
  // once the last product reading it (Sc) has completed and until the next step's TMA load
  float (*red_max)[kBlk] = reinterpret_cast<float (*)[kBlk]>(sQc);
  float (*red_sum)[kBlk] = reinterpret_cast<float (*)[kBlk]>(sQc + 4 * kBlk * sizeof(float));
  __shared__ uint64_t bar_res, bar_ku, bar_vu, bar_qc, bar_mma, bar_z;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, cc = warp >> 2;
  const int row = quarter * 32 + lane;   // accumulator row (TMEM lane) of this thread
  const int c0 = cc * 32;                // first of its 32 columns
  const int bh = blockIdx.x, K = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int k0 = K * kBlk;

  if (tid == 0) {
    mbar_init(&bar_res, 1);
    mbar_init(&bar_ku, 1);
    mbar_init(&bar_vu, 1);
    mbar_init(&bar_qc, 1);
    mbar_init(&bar_z, 1);
    mbar_init(&bar_mma, 1);
    mbar_fence_init();
    abort_flag = 0;
    tma_prefetch_desc(&m_qc); tma_prefetch_desc(&m_ku); tma_prefetch_desc(&m_vu);
  }
  if (warp == 0) { tmem_alloc(&tmem_base_s, TM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
  volatile int* abortp = &abort_flag;

  if (tid == 0) {
    mbar_expect_tx(&bar_res, 3 * OPB);
#pragma unroll
    for (int pn = 0; pn < NP; ++pn) {
      tma_load_4d(sQu + pn * kPanelBytes, &m_qu, &bar_res, pn * 64, k0, h, b);
      tma_load_4d(sKc + pn * kPanelBytes, &m_kc, &bar_res, pn * 64, k0, h, b);
      tma_load_4d(sVc + pn * kPanelBytes, &m_vc, &bar_res, pn * 64, k0, h, b);
    }
    // the first block's tiles; later blocks are fetched inside the step before, each as soon as its
    // slot dies (a tile takes 2-4 thousand cycles from issue to arrival)
    mbar_expect_tx(&bar_ku, OPB);
    mbar_expect_tx(&bar_vu, OPB);
    mbar_expect_tx(&bar_qc, OPB);
#pragma unroll
    for (int pn = 0; pn < NP; ++pn) {
      tma_load_4d(sKuA + pn * kPanelBytes, &m_ku, &bar_ku, pn * 64, k0, h, b);
      tma_load_4d(sVuT + pn * kPanelBytes, &m_vu, &bar_vu, pn * 64, k0, h, b);
      tma_load_4d(sQc + pn * kPanelBytes, &m_qc, &bar_qc, pn * 64, k0, h, b);
    }
  }
  mbar_wait(&bar_res, 0, abortp);
  // Prefill hand-off: the resident tiles of this key block are exactly the rows the decode caches hold for
  // it, so they go there straight from shared memory (the slots are never overwritten; the stores are
  // awaited before the CTA exits).
  if (p.store_caches && tid == 0 && !*abortp) {
#pragma unroll
    for (int pn = 0; pn < NP; ++pn) {
      tma_store_4d(&m_quc, sQu + pn * kPanelBytes, pn * 64, k0, h, b);
      tma_store_4d(&m_kcc, sKc + pn * kPanelBytes, pn * 64, k0, h, b);
      tma_store_4d(&m_vcc, sVc + pn * kPanelBytes, pn * 64, k0, h, b);
    }
    bulk_commit();
  }

  uint32_t ph_load = 0, ph_mma = 0, ph_z = 0;
  const uint32_t aQu = smem_u32(sQu), aKc = smem_u32(sKc), aVc = smem_u32(sVc), aQc = smem_u32(sQc),
                 aWb = smem_u32(sWb), aKuA = smem_u32(sKuA), aVuT = smem_u32(sVuT);
  const int krow = k0 + row;  // global key index of this thread's row when rows are keys
  const float sl2 = p.scale * kLog2e;

  for (int I = K; I < p.nblk; ++I) {
    const int i0 = I * kBlk;
    const bool diag = (I == K);
#ifdef CASTLE_PHASE_TIMING
    const int tstep = I - K;
#endif
    PHASE_MARK(0);
    const bool more = I + 1 < p.nblk;
    const int in0 = i0 + kBlk;
    // Qc[I] goes into its slot only now: that slot doubled as the soft-max exchange buffer until the end
    // of the step before.  It is needed at the second product phase.  One panel per lane of two warps
    // (a TMA instruction costs its issuing thread ~150 cycles); the barrier was armed in the step before.
    if (I > K && lane == 0 && warp >= 4 && warp < 4 + NP)
      tma_load_4d(sQc + (warp - 4) * kPanelBytes, &m_qc, &bar_qc, (warp - 4) * 64, i0, h, b);

    // ---- Z[K,I] = Qu[K] @ Ku[I]^T  (rows = keys k, columns = positions j)
    // After the first step this product was already issued behind P @ Vc of the step before (see there).
    if (diag) {
      if (tid == 0) {
        mbar_wait(&bar_ku, ph_load, abortp);
        PHASE_MARK(1);
        tc_fence_after();
        gemm_kk_t<NP>(tmem + COL_S, aQu, aKuA, ID_SQ, false);
        mma_commit(&bar_mma);
      }
      mbar_wait(&bar_mma, ph_mma, abortp);
      ph_mma ^= 1;
    } else {
      mbar_wait(&bar_z, ph_z, abortp);
      ph_z ^= 1;
    }
    tc_fence_after();
    PHASE_MARK(2);
    {  // gate A = sigmoid(scale * Z), kept for j > k; written over Ku[I]
      float v[32];
      tmem_ld32(trow + COL_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = sigmoid_t<T>(v[j] * p.scale);
      if (diag) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j > row) ? v[j] : 0.f;
      }
      store_row32<T>(sKuA, kPanelBytes, row, c0, v);   // operand of the Su correction (read along rows)
      tmem_st_packed32<T>(trow + COL_A + c0 / 2, v);   // first operand of the state update
    }
    tmem_st_wait();
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    PHASE_MARK(3);

    // ---- W_K += A @ Vu[I]   and   T[I,I] = Qc[I] @ Vu[I]^T
    if (tid == 0) {
      mbar_wait(&bar_vu, ph_load, abortp);
      mbar_wait(&bar_qc, ph_load, abortp);
      tc_fence_after();
      // T goes into O's columns (free until P @ Vc) and is committed alone: masking it overlaps the state
      // update and the part of Su that does not need the masked T, which the next commit covers
      gemm_kk_t<NP>(tmem + COL_O, aQc, aVuT, ID_SQ, false);
      mma_commit(&bar_mma);
      gemm_tm_t<8>(tmem + COL_W, tmem + COL_A, aVuT, ID_D, !diag);
      if (!diag) gemm_kk_t<NP>(tmem + COL_S, aQc, aWb, ID_SQ, false);
    }
    mbar_wait(&bar_mma, ph_mma, abortp);
    ph_mma ^= 1;
    tc_fence_after();
    PHASE_MARK(4);
    {  // masked T (j <= i), unscaled
      float v[32];
      tmem_ld32(trow + COL_O + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      tmem_st_packed32<T>(trow + COL_T + c0 / 2, v);   // first operand of the Su correction
    }
    tmem_st_wait();
    tc_fence_before();
    __syncthreads();
    PHASE_MARK(5);

    // ---- Su/scale = Qc[I] @ Wb^T + Tm @ A^T   (Wb = 16-bit copy of W before this step's update)
    if (tid == 0) {
      tc_fence_after();
      if (more) { mbar_expect_tx(&bar_ku, OPB); mbar_expect_tx(&bar_vu, OPB); }   // loads issued below by other lanes
      gemm_tk_t<2>(tmem + COL_S, tmem + COL_T, aKuA, ID_SQ, !diag);
      // the causal score Sc/scale = Qc[I] @ Kc[K]^T beside it, in O's columns (the masked T is consumed, P @ Vc
      // comes later): one pass then forms S = Sc - silu(Su) and the soft-max numerators
      gemm_kk_t<NP>(tmem + COL_O, aQc, aKc, ID_SQ, false);
      mma_commit(&bar_mma);
    }
    mbar_wait(&bar_mma, ph_mma, abortp);
    ph_mma ^= 1;
    tc_fence_after();
    PHASE_MARK(6);
    // the gate, and Vu[I] with the state update, are consumed: Ku[I+1] and Vu[I+1] -> their slots
    if (more && lane == 0 && warp >= 4 && warp < 4 + NP)
      tma_load_4d(sKuA + (warp - 4) * kPanelBytes, &m_ku, &bar_ku, (warp - 4) * 64, in0, h, b);
    if (more && lane == 0 && warp >= 8 && warp < 8 + NP)
      tma_load_4d(sVuT + (warp - 8) * kPanelBytes, &m_vu, &bar_vu, (warp - 8) * 64, in0, h, b);
    if (c0 < D) {  // refresh the 16-bit copy of W (now including block I) for the next step
      float v[32];
      tmem_ld32(trow + COL_W + c0, v);
      tmem_ld_wait();
      store_row32<T>(sWb, kPanelBytes, row, c0, v);
    }
    // S/scale = Sc/scale - silu(Su)/scale, row max over the four column chunks, then P = exp(S - max)
    // (rows = queries i, columns = keys k)
    const int irow = i0 + row;
    float mrow;
    {
      float v[32], w[32];
      tmem_ld32(trow + COL_S + c0, w);
      tmem_ld32(trow + COL_O + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = fmaf(-w[j], sigmoid_t<T>(w[j] * p.scale), v[j]);
      if (diag) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : -INFINITY;
      }
      float mx = v[0];
#pragma unroll
      for (int j = 1; j < 32; ++j) mx = fmaxf(mx, v[j]);
      red_max[cc][row] = mx;
      __syncthreads();
      mx = fmaxf(fmaxf(red_max[0][row], red_max[1][row]), fmaxf(red_max[2][row], red_max[3][row]));
      mrow = mx * p.scale;   // column 0 is never masked, so the maximum is finite
      const float mb = mx * sl2;
      float lsum = 0.f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float pe = ex2_approx(fmaf(v[j], sl2, -mb));   // exp(scale*v - max); masked entries give 0
        lsum += pe;
        v[j] = pe;
      }
      red_sum[cc][row] = lsum;
      tmem_st_packed32<T>(trow + COL_A + c0 / 2, v);   // P over the gate's packed copy, first operand of P @ Vc
    }
    tmem_st_wait();
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    PHASE_MARK(9);

    // ---- O_partial = P @ Vc[K]
    if (tid == 0) {
      tc_fence_after();
      if (more) mbar_expect_tx(&bar_qc, OPB);   // the load is issued at the top of the next step
      gemm_tm_t<8>(tmem + COL_O, tmem + COL_A, aVc, ID_D, false);
      mma_commit(&bar_mma);
      if (more) {  // S is consumed and Ku[I+1] was fetched after the Su product: the next step's Z runs under the
                   // store of this step's partial
        mbar_wait(&bar_ku, ph_load ^ 1, abortp);
        gemm_kk_t<NP>(tmem + COL_S, aQu, aKuA, ID_SQ, false);
        mma_commit(&bar_z);
      }
    }
    const int64_t tile = (int64_t)bh * tri(p.nblk) + tri(I) + K;
    if (cc == 0 && irow < p.N) {
      float lrow = red_sum[0][row] + red_sum[1][row] + red_sum[2][row] + red_sum[3][row];
      float2* ml = reinterpret_cast<float2*>(p.part_ml) + tile * kBlk + row;
      *ml = make_float2(mrow, lrow);
    }
    mbar_wait(&bar_mma, ph_mma, abortp);
    ph_mma ^= 1;
    tc_fence_after();
    PHASE_MARK(10);
    if (c0 < D) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.part_o) + (tile * kBlk + row) * D + c0);
      float v[32];
      tmem_ld32(trow + COL_O + c0, v);
      tmem_ld_wait();
      if (irow < p.N) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          dst[j] = make_uint4(Elem<T>::pack2(v[8 * j], v[8 * j + 1]), Elem<T>::pack2(v[8 * j + 2], v[8 * j + 3]),
                              Elem<T>::pack2(v[8 * j + 4], v[8 * j + 5]), Elem<T>::pack2(v[8 * j + 6], v[8 * j + 7]));
      }
    }
    fence_async_smem();  // the exchange buffer over Qc[I] was read by threads; TMA writes it next
    tc_fence_before();
    __syncthreads();
    ph_load ^= 1;
    PHASE_MARK(11);
  }

  // ---- W_K is now U[K]: the cache's lookahead keys and the backward's starting state
  if ((p.u_out.ptr != nullptr || p.w_state != nullptr) && c0 < D) {
    tc_fence_after();
    float v[32];
    tmem_ld32(trow + COL_W + c0, v);
    tmem_ld_wait();
    if (krow < p.N) {
      if (p.w_state != nullptr) {
        float* dst = p.w_state + ((int64_t)bh * p.N + krow) * D + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
      if (p.u_out.ptr != nullptr) {
        int64_t off = b * p.u_out.stride_b + h * p.u_out.stride_h + (int64_t)krow * p.u_out.stride_n + c0;
        if (p.u_dtype == CASTLE_F32) {
          float* dst = reinterpret_cast<float*>(p.u_out.ptr) + off;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else if (p.u_dtype == CASTLE_BF16) {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.u_out.ptr) + off);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_uint4(Elem<__nv_bfloat16>::pack2(v[8 * j], v[8 * j + 1]),
                                Elem<__nv_bfloat16>::pack2(v[8 * j + 2], v[8 * j + 3]),
                                Elem<__nv_bfloat16>::pack2(v[8 * j + 4], v[8 * j + 5]),
                                Elem<__nv_bfloat16>::pack2(v[8 * j + 6], v[8 * j + 7]));
        } else {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.u_out.ptr) + off);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_uint4(Elem<__half>::pack2(v[8 * j], v[8 * j + 1]),
                                Elem<__half>::pack2(v[8 * j + 2], v[8 * j + 3]),
                                Elem<__half>::pack2(v[8 * j + 4], v[8 * j + 5]),
                                Elem<__half>::pack2(v[8 * j + 6], v[8 * j + 7]));
        }
      }
    }
  }
  if (p.store_caches && tid == 0) bulk_wait0();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
  if (tid == 0 && abort_flag) atomicOr(p.status, CASTLE_STATUS_WAIT_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// dim_head 64: a leaner CTA (256 threads, 112 KB of shared memory, 256 TMEM columns) so that TWO
// CTAs share an SM.  Each CTA's step is a serial chain of products and elementwise passes; with two
// resident chains one CTA's transcendental work fills the time the other spends waiting on the
// tensor pipe or on a barrier.  To fit, only Qu[K] stays resident: Kc[K] and Vc[K] are re-fetched by
// TMA each step into slots that have just died (Kc over Vu[I] once Su is done, Vc over Qc[I] once Sc
// is done); both fetches hide behind the elementwise pass that follows their issue.
// The three products whose first operand is a tile the threads have just computed (gate A for the state
// update, the masked T for the Su correction, P for P @ Vc) read it from TENSOR MEMORY, where the
// threads put it as packed 16-bit pairs with tcgen05.st: that halves the shared-memory traffic of those
// products (the port, not the tensor pipe, bounds a product with both operands in shared memory) and
// saves the shared-memory copies of the masked T and of P.  The 64 packed columns alias accumulators
// that are dead at that moment: gate and masked T over O, P over the first half of S.
// Warp w owns TMEM lanes 32*(w%4).. and the column group w/4 of a 128-column accumulator: with G = 2
// groups (256 threads) a thread works on 64 values of every 128x128 tile, with G = 4 (512 threads, 64
// registers each) on 32 (measured slower, see below).
constexpr uint32_t kFwd2Smem = 7 * kPanelBytes + 256;   // 112 KB of tiles + barriers
#ifndef CASTLE_FWD_GROUPS
#define CASTLE_FWD_GROUPS 2   // measured: 4 groups (512 threads, 63 registers) run the bench forward in 1.10 ms, 2 in 1.01 ms
#endif
constexpr int kFwd2Groups = CASTLE_FWD_GROUPS;

// Tensor maps of the three decode caches a prefill launch stores into; the plain launch carries an empty
// struct instead.  AUX = the kernel with the two rarely needed paths (cache stores, cut walks) compiled in:
// as run-time branches of the one kernel they cost the plain path 2.3 % (1.001 against 0.979 ms on the bench
// workload), so the plain instantiation has none of their code or parameters.
template <bool AUX> struct CacheMaps {};
template <> struct CacheMaps<true> { CUtensorMap qu, kc, vc; };

template <typename T, int G, bool AUX>
__global__ void __launch_bounds__(G * 128, 2)
castle_fwd_kernel_d64(const FwdParams p, const __grid_constant__ CUtensorMap m_qc, const __grid_constant__ CUtensorMap m_kc,
                      const __grid_constant__ CUtensorMap m_vc, const __grid_constant__ CUtensorMap m_qu,
                      const __grid_constant__ CUtensorMap m_ku, const __grid_constant__ CUtensorMap m_vu,
                      const __grid_constant__ CacheMaps<AUX> m_cache) {
  constexpr int D = 64;
  constexpr int NCH = 4 / G;   // 32-column chunks of a 128-column tile per thread
  constexpr uint32_t OPB = kPanelBytes;
  constexpr uint32_t TM_COLS = 256;
  constexpr uint32_t COL_W = 0, COL_S = 64, COL_O = 192;
  constexpr int FMT = Elem<T>::fmt;
  constexpr uint32_t ID_SQ = make_idesc(128, 128, FMT, false, false, false);
  constexpr uint32_t ID_D = make_idesc(128, D, FMT, false, true, false);
  constexpr float kLog2e = 1.4426950408889634f;

  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQu = smem;                 // resident
  uint8_t* sQV = sQu + OPB;            // Qc[I], then Vc[K]
  uint8_t* sWb = sQV + OPB;
  uint8_t* sKuA = sWb + OPB;           // Ku[I] -> gate A (32 KB; P lives in tensor memory)
  uint8_t* sVuT = sKuA + 2 * OPB;      // Vu[I] -> Kc[K] in the first half (the masked T lives in tensor memory)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sVuT + 2 * OPB);
  uint64_t *bar_qu = bars, *bar_qc = bars + 1, *bar_ku = bars + 2, *bar_vu = bars + 3, *bar_kc = bars + 4,
           *bar_vc = bars + 5, *bar_mma = bars + 6;
  uint32_t* tmem_base_s = reinterpret_cast<uint32_t*>(bars + 8);
  int* abort_flag = reinterpret_cast<int*>(bars + 9);
  // row max / row sum exchange between the two threads of a row: over the second half of the T slot,
  // dead from the end of the Su product until the next step's masked T is written
  float (*red_max)[kBlk] = reinterpret_cast<float (*)[kBlk]>(sVuT + OPB);
  float (*red_sum)[kBlk] = reinterpret_cast<float (*)[kBlk]>(sVuT + OPB + G * kBlk * sizeof(float));

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int quarter = warp & 3, grp = warp >> 2;
  const int cbase = grp * NCH * 32;
  const int row = quarter * 32 + lane;
  const int bh = blockIdx.x, K = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int k0 = K * kBlk;
  // Walk segments.  With few (batch, head) pairs the grid is a single wave whose makespan is the longest
  // walk (key block 0: every query block), so long walks are cut in two, one CTA each.  The CTA that takes
  // the later part first rebuilds the state it would have inherited with a short pre-loop over the earlier
  // blocks (Z, gate and W += A @ Vu only, no scores).  blockIdx.z = 0 is the LATER part: those CTAs are the heaviest, and the grid is handed
  // out in blockIdx order, so they start first.
  const int seg = AUX ? (int)gridDim.z - 1 - (int)blockIdx.z : 0;
  const int walk = p.nblk - K;
  const int cut = (AUX && p.split_q8 > 0 && walk >= 8) ? K + (walk * p.split_q8 + 128) / 256 : p.nblk;
  const bool store_caches = AUX && p.store_caches;
  const CUtensorMap *m_cache_qu = nullptr, *m_cache_kc = nullptr, *m_cache_vc = nullptr;
  if constexpr (AUX) { m_cache_qu = &m_cache.qu; m_cache_kc = &m_cache.kc; m_cache_vc = &m_cache.vc; }
  const int I_begin = seg == 0 ? K : cut;              // first block whose scores this CTA computes
  const int I_end = seg == 0 ? cut : p.nblk;           // one past its last
  if (I_begin >= I_end) return;                        // a short walk is not cut: its later part is empty
  const bool owns_state = (I_end == p.nblk);                                      // the last segment ends with W_K = U[K]

  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need 1024-byte alignment
    if (tid == 0) atomicOr(p.status, CASTLE_STATUS_BAD_LAUNCH);
    return;
  }
  if (tid == 0) {
    for (int i = 0; i < 7; ++i) mbar_init(bars + i, 1);
    mbar_fence_init();
    *abort_flag = 0;
    tma_prefetch_desc(&m_qc); tma_prefetch_desc(&m_ku); tma_prefetch_desc(&m_vu);
    tma_prefetch_desc(&m_kc); tma_prefetch_desc(&m_vc);
  }
  if (warp == 0) { tmem_alloc(tmem_base_s, TM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_base_s;
  const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
  volatile int* abortp = abort_flag;

  if (tid == 0) {
    mbar_expect_tx(bar_qu, OPB);
    tma_load_4d(sQu, &m_qu, bar_qu, 0, k0, h, b);
    if (I_begin == K) {   // the pre-loop needs no Qc; the last pre-loop step fetches the first real one
      mbar_expect_tx(bar_qc, OPB);
      tma_load_4d(sQV, &m_qc, bar_qc, 0, k0, h, b);
    }
    mbar_expect_tx(bar_ku, OPB);
    tma_load_4d(sKuA, &m_ku, bar_ku, 0, k0, h, b);
    mbar_expect_tx(bar_vu, OPB);
    tma_load_4d(sVuT, &m_vu, bar_vu, 0, k0, h, b);
    mbar_wait(bar_qu, 0, abortp);
    // Prefill hand-off: Qu[K] is the block's rows of the decode cache; Kc[K] and Vc[K] follow in the
    // first step, each when its fetch has landed (see there).
    if (store_caches && seg == 0 && !*abortp) tma_store_4d(m_cache_qu, sQu, 0, k0, h, b);
  }

  uint32_t ph_ld = 0, ph_mma = 0;   // Ku/Vu barriers flip once per step (pre-loop steps included) ...
  uint32_t ph_main = 0;             // ... the Qc/Kc/Vc barriers once per step that computes scores
  const uint32_t aQu = smem_u32(sQu), aQV = smem_u32(sQV), aWb = smem_u32(sWb), aKuA = smem_u32(sKuA),
                 aVuT = smem_u32(sVuT);
  const int krow = k0 + row;
  const float sl2 = p.scale * kLog2e;

#define F2_MMA_WAIT()                              \
  mbar_wait_lazy_abort(bar_mma, ph_mma, abortp);   \
  ph_mma ^= 1;                          \
  tc_fence_after();
#define F2_SYNC()      \
  fence_async_smem();  \
  tc_fence_before();   \
  __syncthreads();

  for (int I = K; I < I_end; ++I) {
    const int i0 = I * kBlk;
    const bool diag = (I == K), last = (I == I_end - 1);
    const bool pre = AUX && I < I_begin;   // state-only step of the pre-loop
#ifdef CASTLE_PHASE_TIMING
    const int tstep = I - K;
#endif
    PHASE_MARK(0);

    // ---- Z[K,I] = Qu[K] @ Ku[I]^T
    if (tid == 0) {
      mbar_wait(bar_ku, ph_ld, abortp);
      tc_fence_after();
      gemm_kk_t<1>(tmem + COL_S, aQu, aKuA, ID_SQ, false);
      mma_commit(bar_mma);
    }
    F2_MMA_WAIT();
    PHASE_MARK(1);
    if (pre && tid == 0) {
      // Pre-loop steps are short, so their loads are issued as early as the slots allow: Ku[I] is consumed
      // by Z (and the gate's shared-memory copy is not needed without scores), so the next Ku goes now,
      // together with Qc when the next step is the first one that computes scores.
      const int in0 = i0 + kBlk;   // a pre-loop step is never the last step of its CTA
      if (I + 1 == I_begin) {
        mbar_expect_tx(bar_qc, OPB);
        tma_load_4d(sQV, &m_qc, bar_qc, 0, in0, h, b);
      }
      mbar_expect_tx(bar_ku, OPB);
      tma_load_4d(sKuA, &m_ku, bar_ku, 0, in0, h, b);
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {  // gate A = sigmoid(scale * Z), kept for j > k; over Ku[I]
      const int c0 = cbase + c * 32;
      float v[32];
      tmem_ld32(trow + COL_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = sigmoid_t<T>(v[j] * p.scale);
      if (diag) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = (c0 + j > row) ? v[j] : 0.f;
      }
      if (!pre) store_row32<T>(sKuA, kPanelBytes, row, c0, v);   // operand of the Su correction (read along rows)
      tmem_st_packed32<T>(trow + COL_O + c0 / 2, v);             // first operand of the state update
    }
    tmem_st_wait();
    F2_SYNC();
    PHASE_MARK(2);

    // ---- W_K += A @ Vu[I]   and   T[I,I] = Qc[I] @ Vu[I]^T
    if (tid == 0) {
      mbar_wait(bar_vu, ph_ld, abortp);
      if (!pre) mbar_wait(bar_qc, ph_main, abortp);
      tc_fence_after();
      gemm_tm_t<8>(tmem + COL_W, tmem + COL_O, aVuT, ID_D, !diag);
      if (!pre) gemm_kk_t<1>(tmem + COL_S, aQV, aVuT, ID_SQ, false);
      mma_commit(bar_mma);
    }
    F2_MMA_WAIT();
    PHASE_MARK(3);
    if (pre) {
      // The state now includes block I.  Before the first step that computes scores, make its 16-bit copy
      // (the later steps refresh it themselves); then fetch the next block's tiles and go on.
      const bool next_real = (I + 1 == I_begin);
      if (next_real && grp < 2) {
        float v[32];
        tmem_ld32(trow + COL_W + grp * 32, v);
        tmem_ld_wait();
        store_row32<T>(sWb, kPanelBytes, row, grp * 32, v);
      }
      F2_SYNC();
      if (tid == 0) {   // Vu[I] is consumed by the state update: the next one goes now
        mbar_expect_tx(bar_vu, OPB);
        tma_load_4d(sVuT, &m_vu, bar_vu, 0, i0 + kBlk, h, b);
      }
      ph_ld ^= 1;
      continue;
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {  // masked T (j <= i), unscaled; over Vu[I]
      const int c0 = cbase + c * 32;
      float v[32];
      tmem_ld32(trow + COL_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = (c0 + j <= row) ? v[j] : 0.f;
      tmem_st_packed32<T>(trow + COL_O + c0 / 2, v);   // over the gate's packed copy, which the update has consumed
    }
    tmem_st_wait();
    tc_fence_before();
    __syncthreads();
    PHASE_MARK(4);

    // ---- Su/scale = Qc[I] @ Wb^T + Tm @ A^T
    if (tid == 0) {
      tc_fence_after();
      if (!diag) gemm_kk_t<1>(tmem + COL_S, aQV, aWb, ID_SQ, false);
      gemm_tk_t<2>(tmem + COL_S, tmem + COL_O, aKuA, ID_SQ, !diag);
      mma_commit(bar_mma);
    }
    F2_MMA_WAIT();
    PHASE_MARK(5);
    if (tid == 0) {  // Vu[I] is long consumed: fetch Kc[K] into its slot
      mbar_expect_tx(bar_kc, OPB);
      tma_load_4d(sVuT, &m_kc, bar_kc, 0, k0, h, b);
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {  // penalty -silu(Su)/scale back into the accumulator
      const int c0 = cbase + c * 32;
      float v[32];
      tmem_ld32(trow + COL_S + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = -v[j] * sigmoid_t<T>(v[j] * p.scale);
      tmem_st32(trow + COL_S + c0, v);
    }
    if (grp < 2) {  // refresh the 16-bit copy of W (now including block I)
      float v[32];
      tmem_ld32(trow + COL_W + grp * 32, v);
      tmem_ld_wait();
      store_row32<T>(sWb, kPanelBytes, row, grp * 32, v);
    }
    tmem_st_wait();
    F2_SYNC();
    PHASE_MARK(6);

    // ---- S/scale = penalty + Qc[I] @ Kc[K]^T
    if (tid == 0) {
      mbar_wait(bar_kc, ph_main, abortp);
      tc_fence_after();
      gemm_kk_t<1>(tmem + COL_S, aQV, aVuT, ID_SQ, true);
      mma_commit(bar_mma);
      if (diag && store_caches && !*abortp) tma_store_4d(m_cache_kc, sVuT, 0, k0, h, b);
    }
    F2_MMA_WAIT();
    PHASE_MARK(7);
    if (tid == 0) {  // Qc[I] and Kc[K] are consumed: fetch Vc[K] over Qc, and the next Vu over Kc
      mbar_expect_tx(bar_vc, OPB);
      tma_load_4d(sQV, &m_vc, bar_vc, 0, k0, h, b);
    }
    const int irow = i0 + row;
    float mrow, lsum = 0.f;
    {
      float v[NCH][32];
#pragma unroll
      for (int c = 0; c < NCH; ++c) tmem_ld32(trow + COL_S + cbase + c * 32, v[c]);
      tmem_ld_wait();
      if (diag) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
          for (int j = 0; j < 32; ++j) v[c][j] = (cbase + c * 32 + j <= row) ? v[c][j] : -INFINITY;
      }
      float mx = v[0][0];
#pragma unroll
      for (int c = 0; c < NCH; ++c)
#pragma unroll
        for (int j = 0; j < 32; ++j) mx = fmaxf(mx, v[c][j]);
      red_max[grp][row] = mx;
      __syncthreads();
#pragma unroll
      for (int g = 0; g < G; ++g) mx = fmaxf(mx, red_max[g][row]);
      mrow = mx * p.scale;
      const float mb = mx * sl2;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          v[c][j] = ex2_approx(fmaf(v[c][j], sl2, -mb));
          lsum += v[c][j];
        }
      }
      red_sum[grp][row] = lsum;
      // P as packed pairs over the first 64 columns of S: every thread of the row has its values in
      // registers since the barrier above, so the accumulator may be overwritten
#pragma unroll
      for (int c = 0; c < NCH; ++c) tmem_st_packed32<T>(trow + COL_S + (cbase + c * 32) / 2, v[c]);
    }
    tmem_st_wait();
    tc_fence_before();
    __syncthreads();
    PHASE_MARK(8);

    // ---- O_partial = P @ Vc[K]
    if (tid == 0) {
      mbar_wait(bar_vc, ph_main, abortp);
      tc_fence_after();
      gemm_tm_t<8>(tmem + COL_O, tmem + COL_S, aQV, ID_D, false);
      mma_commit(bar_mma);
      if (diag && store_caches) {
        if (!*abortp) tma_store_4d(m_cache_vc, sQV, 0, k0, h, b);
        bulk_commit();
      }
    }
    const int64_t tile = (int64_t)bh * tri(p.nblk) + tri(I) + K;
    if (grp == 0 && irow < p.N) {
      float2* ml = reinterpret_cast<float2*>(p.part_ml) + tile * kBlk + row;
      float l = red_sum[0][row];
#pragma unroll
      for (int g = 1; g < G; ++g) l += red_sum[g][row];
      *ml = make_float2(mrow, l);
    }
    fence_async_smem();  // the exchange buffer is read here and written by TMA (next Vu) below
    F2_MMA_WAIT();
    PHASE_MARK(9);
    if (tid == 0 && !last) {  // every slot of this step is dead: fetch the next step's Qc, Ku, Vu
      const int in0 = i0 + kBlk;
      if (diag && store_caches) bulk_wait_read0();   // the cache stores have read the Kc and Vc slots
      mbar_expect_tx(bar_qc, OPB);
      tma_load_4d(sQV, &m_qc, bar_qc, 0, in0, h, b);
      mbar_expect_tx(bar_ku, OPB);
      tma_load_4d(sKuA, &m_ku, bar_ku, 0, in0, h, b);
      mbar_expect_tx(bar_vu, OPB);
      tma_load_4d(sVuT, &m_vu, bar_vu, 0, in0, h, b);
    }
    if (grp < 2) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.part_o) + (tile * kBlk + row) * D + grp * 32);
      float v[32];
      tmem_ld32(trow + COL_O + grp * 32, v);
      tmem_ld_wait();
      if (irow < p.N) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          dst[j] = make_uint4(Elem<T>::pack2(v[8 * j], v[8 * j + 1]), Elem<T>::pack2(v[8 * j + 2], v[8 * j + 3]),
                              Elem<T>::pack2(v[8 * j + 4], v[8 * j + 5]), Elem<T>::pack2(v[8 * j + 6], v[8 * j + 7]));
      }
    }
    ph_ld ^= 1;
    ph_main ^= 1;
    tc_fence_before();
    __syncthreads();
    PHASE_MARK(10);
  }
#undef F2_MMA_WAIT
#undef F2_SYNC

  // ---- W_K is now U[K] (in the CTA that walked to the last query block)
  if (owns_state && grp < 2 && (p.u_out.ptr != nullptr || p.w_state != nullptr)) {
    tc_fence_after();
    const int c0 = grp * 32;
    float v[32];
    tmem_ld32(trow + COL_W + c0, v);
    tmem_ld_wait();
    if (krow < p.N) {
      if (p.w_state != nullptr) {
        float* dst = p.w_state + ((int64_t)bh * p.N + krow) * D + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
      if (p.u_out.ptr != nullptr) {
        int64_t off = b * p.u_out.stride_b + h * p.u_out.stride_h + (int64_t)krow * p.u_out.stride_n + c0;
        if (p.u_dtype == CASTLE_F32) {
          float* dst = reinterpret_cast<float*>(p.u_out.ptr) + off;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else if (p.u_dtype == CASTLE_BF16) {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.u_out.ptr) + off);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_uint4(Elem<__nv_bfloat16>::pack2(v[8 * j], v[8 * j + 1]),
                                Elem<__nv_bfloat16>::pack2(v[8 * j + 2], v[8 * j + 3]),
                                Elem<__nv_bfloat16>::pack2(v[8 * j + 4], v[8 * j + 5]),
                                Elem<__nv_bfloat16>::pack2(v[8 * j + 6], v[8 * j + 7]));
        } else {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.u_out.ptr) + off);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_uint4(Elem<__half>::pack2(v[8 * j], v[8 * j + 1]),
                                Elem<__half>::pack2(v[8 * j + 2], v[8 * j + 3]),
                                Elem<__half>::pack2(v[8 * j + 4], v[8 * j + 5]),
                                Elem<__half>::pack2(v[8 * j + 6], v[8 * j + 7]));
        }
      }
    }
  }
  if (store_caches && tid == 0) bulk_wait0();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, TM_COLS);
  if (tid == 0 && *abort_flag) atomicOr(p.status, CASTLE_STATUS_WAIT_TIMEOUT);
}

// Merge the per-key-block partials of one query block: out = sum_K e^{m_K - m} O_K / sum_K e^{m_K - m} l_K.
// D/8 threads per row, each owning eight consecutive elements (one 16-byte load per partial).
template <typename T, int D>
__global__ void __launch_bounds__(256) castle_fwd_merge_kernel(const FwdParams p) {
  constexpr int TPR = D / 8, ROWS = 256 / TPR;
  const int bh = blockIdx.y, I = blockIdx.x / (kBlk / ROWS), sub = blockIdx.x % (kBlk / ROWS);
  const int r = sub * ROWS + threadIdx.x / TPR, c8 = threadIdx.x % TPR;
  const int i = I * kBlk + r;
  if (i >= p.N) return;
  const int64_t tile0 = (int64_t)bh * tri(p.nblk) + tri(I);
  const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + tile0 * kBlk + r;
  float m = -INFINITY;
  for (int K = 0; K <= I; ++K) m = fmaxf(m, ml[(int64_t)K * kBlk].x);
  float l = 0.f, acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  const uint4* po = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.part_o) + (tile0 * kBlk + r) * D) + c8;
  for (int K = 0; K <= I; ++K) {
    float2 v = ml[(int64_t)K * kBlk];
    float w = __expf(v.x - m);
    l += v.y * w;
    uint4 o = po[(int64_t)K * kBlk * D / 8];
    float2 a = Elem<T>::unpack2(o.x), b2 = Elem<T>::unpack2(o.y), c = Elem<T>::unpack2(o.z), d2 = Elem<T>::unpack2(o.w);
    acc[0] += a.x * w; acc[1] += a.y * w; acc[2] += b2.x * w; acc[3] += b2.y * w;
    acc[4] += c.x * w; acc[5] += c.y * w; acc[6] += d2.x * w; acc[7] += d2.y * w;
  }
  const float inv = 1.f / l;
  const int b = bh / p.H, h = bh % p.H;
  T* dst = reinterpret_cast<T*>(p.out.ptr) + b * p.out.stride_b + h * p.out.stride_h + (int64_t)i * p.out.stride_n + c8 * 8;
  uint4 q;
  q.x = Elem<T>::pack2(acc[0] * inv, acc[1] * inv);
  q.y = Elem<T>::pack2(acc[2] * inv, acc[3] * inv);
  q.z = Elem<T>::pack2(acc[4] * inv, acc[5] * inv);
  q.w = Elem<T>::pack2(acc[6] * inv, acc[7] * inv);
  *reinterpret_cast<uint4*>(dst) = q;
  if (c8 == 0) p.lse[(int64_t)bh * p.N + i] = m + __logf(l);
}

template <typename T>
static int launch_fwd_d64(const FwdParams& p, const CUtensorMap* maps, cudaStream_t st) {
  constexpr int G = kFwd2Groups;
  {  // per device, so set on every call (cheap)
    cudaError_t e = cudaFuncSetAttribute(castle_fwd_kernel_d64<T, G, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwd2Smem);
    if (e != cudaSuccess) return cuda_fail(e, "castle_fwd attribute");
  }
  // Few (batch, head) pairs: cut the long walks so that the grid is several waves of short CTAs instead of
  // one wave bounded by the walk of key block 0 (296 CTAs are resident at a time: 2 per SM on 148 SMs).
  FwdParams q = p;
  q.split_q8 = 0;
  if ((int64_t)p.B * p.H * p.nblk < 384 && p.nblk >= 8)   // beyond ~1.3 waves the pre-loops cost more than the balance gains
    q.split_q8 = 128;   // the middle measured best (0.169 ms at 8 pairs x 32 blocks; 0.240 ms uncut; later cuts slower)
  const bool aux = q.split_q8 > 0 || p.store_caches;
  dim3 grid(p.B * p.H, p.nblk, q.split_q8 > 0 ? 2 : 1);
  ev_start(CASTLE_KERNEL_FWD, st);
  if (aux) {
    cudaError_t e = cudaFuncSetAttribute(castle_fwd_kernel_d64<T, G, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwd2Smem);
    if (e != cudaSuccess) return cuda_fail(e, "castle_fwd attribute");
    CacheMaps<true> cm;
    cm.qu = maps[6]; cm.kc = maps[7]; cm.vc = maps[8];
    castle_fwd_kernel_d64<T, G, true><<<grid, G * 128, kFwd2Smem, st>>>(q, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], cm);
  } else {
    castle_fwd_kernel_d64<T, G, false><<<grid, G * 128, kFwd2Smem, st>>>(q, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5],
                                                                        CacheMaps<false>{});
  }
  ev_stop(CASTLE_KERNEL_FWD, st);
  constexpr int ROWS = 256 / (64 / 8);
  dim3 g2(p.nblk * (kBlk / ROWS), p.B * p.H);
  castle_fwd_merge_kernel<T, 64><<<g2, 256, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_fwd launch");
}

template <typename T, int D>
static int launch_fwd(const FwdParams& p, const CUtensorMap* maps, cudaStream_t st) {
  constexpr size_t smem = 5 * (D / 64) * kPanelBytes + 2 * 2 * kPanelBytes + 1024;
  {  // per device, so set on every call (cheap)
    cudaError_t e = cudaFuncSetAttribute(castle_fwd_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "castle_fwd attribute");
  }
  dim3 grid(p.B * p.H, p.nblk);
  ev_start(CASTLE_KERNEL_FWD, st);
  castle_fwd_kernel<T, D><<<grid, kFwdThreads, smem, st>>>(p, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5],
                                                            maps[6], maps[7], maps[8]);
  ev_stop(CASTLE_KERNEL_FWD, st);
  constexpr int ROWS = 256 / (D / 8);
  dim3 g2(p.nblk * (kBlk / ROWS), p.B * p.H);
  castle_fwd_merge_kernel<T, D><<<g2, 256, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_fwd launch");
}

static int check_parallel_problem(const castle_problem_t* p, const char* who) {
  if (!p) return reject("%s: null problem", who);
  if (p->batch <= 0 || p->heads <= 0 || p->seq_len <= 0) return reject("%s: empty problem", who);
  if (p->dim_head != 64 && p->dim_head != 128) return reject("%s: dim_head %d not supported (64 or 128)", who, p->dim_head);
  if (p->dtype != CASTLE_BF16 && p->dtype != CASTLE_F16) return reject("%s: dtype %d not supported (bf16, fp16)", who, p->dtype);
  if ((int64_t)p->batch * p->heads > 2147483647LL || (p->seq_len + kBlk - 1) / kBlk > 65535)
    return reject("%s: grid too large", who);
  return 0;
}

}  // namespace castle

using namespace castle;

extern "C" size_t castle_fwd_workspace_bytes(const castle_problem_t* p) {
  if (!p || p->seq_len <= 0) return 0;
  int64_t nb = (p->seq_len + kBlk - 1) / kBlk;
  int64_t tiles = (int64_t)p->batch * p->heads * tri(nb);
  return (size_t)(tiles * kBlk * (2 * sizeof(float) + p->dim_head * 2));  // (max, sum) fp32 + a 16-bit row
}

static int fwd_impl(const char* who, const castle_problem_t* p, const castle_tensor_t* qc, const castle_tensor_t* kc,
                    const castle_tensor_t* vc, const castle_tensor_t* qu, const castle_tensor_t* ku,
                    const castle_tensor_t* vu, const castle_tensor_t* out, float* lse, const castle_tensor_t* u_out,
                    int32_t u_dtype, float* w_state, const castle_tensor_t* const* caches, void* workspace,
                    size_t workspace_bytes, int32_t* status, void* stream) {
  int rc = check_parallel_problem(p, who);
  if (rc) return rc;
  const castle_tensor_t* ins[6] = {qc, kc, vc, qu, ku, vu};
  const char* names[6] = {"qc", "kc", "vc", "qu", "ku", "vu"};
  for (int i = 0; i < 6; ++i)
    if (!tensor_ok(ins[i], p->dtype, names[i], &rc)) return rc;
  if (!tensor_ok(out, p->dtype, "out", &rc)) return rc;
  if (!lse || !status) return reject("%s: lse and status must not be null", who);
  if (u_out && u_out->ptr) {
    if (u_dtype != CASTLE_BF16 && u_dtype != CASTLE_F16 && u_dtype != CASTLE_F32) return reject("%s: bad u_dtype", who);
    if (!tensor_ok(u_out, u_dtype, "u_out", &rc)) return rc;
  }
  const char* cnames[3] = {"qu_cache", "kc_cache", "vc_cache"};
  if (caches)
    for (int i = 0; i < 3; ++i)
      if (!tensor_ok(caches[i], p->dtype, cnames[i], &rc)) return rc;
  size_t need = castle_fwd_workspace_bytes(p);
  if (!workspace || workspace_bytes < need)
    return reject("%s: workspace too small (%zu < %zu bytes)", who, workspace_bytes, need);
  if (((uintptr_t)workspace) % 16) return reject("%s: workspace not 16-byte aligned", who);

  FwdParams fp;
  fp.B = p->batch; fp.H = p->heads; fp.N = p->seq_len; fp.nblk = (p->seq_len + kBlk - 1) / kBlk;
  fp.scale = p->scale;
  int64_t tiles = (int64_t)p->batch * p->heads * tri(fp.nblk);
  fp.part_ml = (float*)workspace;
  fp.part_o = fp.part_ml + tiles * kBlk * 2;  // 16-bit rows behind the fp32 (max, sum) pairs
  fp.lse = lse; fp.w_state = w_state;
  fp.u_out = (u_out && u_out->ptr) ? *u_out : castle_tensor_t{nullptr, 0, 0, 0};
  fp.u_dtype = u_dtype;
  fp.out = *out; fp.status = status;
  fp.store_caches = caches ? 1 : 0;
  fp.split_q8 = 0;
#ifdef CASTLE_PHASE_TIMING
  fp.timing = (long long*)((char*)workspace + need);  // the caller leaves 1 KB beyond the partials
#endif

  CUtensorMap maps[9];
  for (int i = 0; i < 6; ++i) {
    rc = make_tmap_16bit(&maps[i], ins[i], p->dtype, p->batch, p->heads, p->seq_len, p->dim_head, kBlk, names[i]);
    if (rc) return rc;
  }
  for (int i = 0; i < 3; ++i) {
    // without caches the three maps are never used by the kernel; give them a valid encoding anyway
    const castle_tensor_t* t = caches ? caches[i] : ins[3];
    rc = make_tmap_16bit(&maps[6 + i], t, p->dtype, p->batch, p->heads, p->seq_len, p->dim_head, kBlk, cnames[i]);
    if (rc) return rc;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (p->dtype == CASTLE_BF16)
    return p->dim_head == 64 ? launch_fwd_d64<__nv_bfloat16>(fp, maps, st) : launch_fwd<__nv_bfloat16, 128>(fp, maps, st);
  return p->dim_head == 64 ? launch_fwd_d64<__half>(fp, maps, st) : launch_fwd<__half, 128>(fp, maps, st);
}

extern "C" int castle_fwd(const castle_problem_t* p, const castle_tensor_t* qc, const castle_tensor_t* kc,
                          const castle_tensor_t* vc, const castle_tensor_t* qu, const castle_tensor_t* ku,
                          const castle_tensor_t* vu, const castle_tensor_t* out, float* lse,
                          const castle_tensor_t* u_out, int32_t u_dtype, float* w_state, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream) {
  return fwd_impl("castle_fwd", p, qc, kc, vc, qu, ku, vu, out, lse, u_out, u_dtype, w_state, nullptr, workspace,
                  workspace_bytes, status, stream);
}

extern "C" int castle_fwd_prefill(const castle_problem_t* p, const castle_tensor_t* qc, const castle_tensor_t* kc,
                                  const castle_tensor_t* vc, const castle_tensor_t* qu, const castle_tensor_t* ku,
                                  const castle_tensor_t* vu, const castle_tensor_t* out, float* lse,
                                  const castle_tensor_t* u_cache, const castle_tensor_t* qu_cache,
                                  const castle_tensor_t* kc_cache, const castle_tensor_t* vc_cache, float* w_state,
                                  void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  if (!u_cache || !u_cache->ptr || !qu_cache || !kc_cache || !vc_cache)
    return reject("castle_fwd_prefill: the four cache tensors must not be null");
  const castle_tensor_t* caches[3] = {qu_cache, kc_cache, vc_cache};
  return fwd_impl("castle_fwd_prefill", p, qc, kc, vc, qu, ku, vu, out, lse, u_cache, p ? p->dtype : 0, w_state, caches,
                  workspace, workspace_bytes, status, stream);
}
