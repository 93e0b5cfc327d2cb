// Cached single-token CASTLE step (HBM-bound).
//
// Per (batch, head) the step streams four caches of `t` rows once: it reads
// qu_cache, U, kc_cache and vc_cache and writes U back, i.e. 5*t*d elements,
// which is the algorithmic traffic of the step.  Each row is handled by d/VEC
// adjacent lanes (VEC = 16 bytes of elements per lane), so every global access
// is a 128-bit load/store and a warp touches whole 128-byte lines; the three
// dot products of a row are reduced with xor-shuffles inside that lane group.
// Rows are split over `nsplit` CTAs per (batch, head); each CTA keeps a running
// (max, sum, weighted value sum) and writes one partial, which a small second
// kernel merges.
#include <mutex>
#include "common.cuh"
#include "sm100.cuh"

namespace castle {

struct DecodeParams {
  castle_tensor_t qc, kc, vc, qu, ku, vu;          // new rows
  castle_tensor_t U, quc, kcc, vcc;                // caches
  castle_tensor_t out;
  float* part;                                     // [BH][nsplit][2 + D]
  int H, t, nsplit, rows_per_split;
  float scale;
  int32_t* status;
};

template <typename T> struct Vec;  // 16 bytes of T <-> floats
template <> struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  static __device__ __forceinline__ void round(float*) {}
};
template <typename T> struct Vec16 {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const T* p, float* v) {
    uint4 q = *reinterpret_cast<const uint4*>(p);
    float2 a = Elem<T>::unpack2(q.x), b = Elem<T>::unpack2(q.y), c = Elem<T>::unpack2(q.z), d = Elem<T>::unpack2(q.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static __device__ __forceinline__ void store(T* p, const float* v) {
    uint4 q;
    q.x = Elem<T>::pack2(v[0], v[1]); q.y = Elem<T>::pack2(v[2], v[3]);
    q.z = Elem<T>::pack2(v[4], v[5]); q.w = Elem<T>::pack2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = q;
  }
  // round to the storage type, so the value used for the score equals the value stored
  static __device__ __forceinline__ void round(float* v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = Elem<T>::to_f(Elem<T>::from_f(v[i]));
  }
};
template <> struct Vec<__nv_bfloat16> : Vec16<__nv_bfloat16> {};
template <> struct Vec<__half> : Vec16<__half> {};

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

#ifndef CASTLE_DECODE_THREADS
#define CASTLE_DECODE_THREADS 128
#endif
#ifndef CASTLE_DECODE_UNROLL
#define CASTLE_DECODE_UNROLL 1
#endif
#ifndef CASTLE_DECODE_MIN_CTAS
#define CASTLE_DECODE_MIN_CTAS 8
#endif
constexpr int kDecodeThreads = CASTLE_DECODE_THREADS;
constexpr int kDecodeUnroll = CASTLE_DECODE_UNROLL;

template <typename T, int D>
__global__ void __launch_bounds__(kDecodeThreads, CASTLE_DECODE_MIN_CTAS) castle_decode_kernel(const DecodeParams p) {
  constexpr int VEC = Vec<T>::N;
  constexpr int LPR = D / VEC;                 // lanes per row
  constexpr int RPW = 32 / LPR;                // rows per warp per pass
  constexpr int NW = kDecodeThreads / 32;
  const int bh = blockIdx.x, split = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPR, grp = lane / LPR;
  const int64_t col = (int64_t)sub * VEC;

  auto row_ptr = [&](const castle_tensor_t& t, int64_t r) {
    return reinterpret_cast<T*>(t.ptr) + b * t.stride_b + h * t.stride_h + r * t.stride_n + col;
  };

  float qcv[VEC], kuv[VEC], vuv[VEC];
  Vec<T>::load(row_ptr(p.qc, 0), qcv);
  Vec<T>::load(row_ptr(p.ku, 0), kuv);
  Vec<T>::load(row_ptr(p.vu, 0), vuv);
#pragma unroll
  for (int i = 0; i < VEC; ++i) { qcv[i] *= p.scale; kuv[i] *= p.scale; }  // scale*(qu.ku) == qu.(scale*ku)

  float m = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;

  const int r_begin = split * p.rows_per_split;
  const int r_end = min(p.t, r_begin + p.rows_per_split);

  // rows of this CTA, RPW*NW*UNROLL per pass
  // (the loop bound is warp-uniform: the shuffles below need every lane of the warp)
  for (int base = r_begin + warp * RPW; base < r_end; base += RPW * NW * kDecodeUnroll) {
    float quv[kDecodeUnroll][VEC], uv[kDecodeUnroll][VEC], kv[kDecodeUnroll][VEC], vv[kDecodeUnroll][VEC];
    bool live[kDecodeUnroll];
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      int r = base + grp + u * RPW * NW;
      live[u] = r < r_end;
      if (live[u]) {
        Vec<T>::load(row_ptr(p.quc, r), quv[u]);
        Vec<T>::load(row_ptr(p.U, r), uv[u]);
        Vec<T>::load(row_ptr(p.kcc, r), kv[u]);
        Vec<T>::load(row_ptr(p.vcc, r), vv[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      int r = base + grp + u * RPW * NW;
      float z = 0.f, sc = 0.f, su = 0.f;
      if (live[u]) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) z += quv[u][i] * kuv[i];
      }
      z = group_sum<LPR>(z);
      float a = sigmoid_f(z);
      if (live[u]) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) uv[u][i] += a * vuv[i];
        Vec<T>::round(uv[u]);
        Vec<T>::store(row_ptr(p.U, r), uv[u]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) { sc += qcv[i] * kv[u][i]; su += qcv[i] * uv[u][i]; }
      }
      sc = group_sum<LPR>(sc);
      su = group_sum<LPR>(su);
      if (live[u]) {
        float s = sc - su * sigmoid_f(su);
        float mn = fmaxf(m, s);
        float corr = __expf(m - mn), pe = __expf(s - mn);
        l = l * corr + pe;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = acc[i] * corr + pe * vv[u][i];
        m = mn;
      }
    }
  }

  // the appended row: U[t] = 0 so its score is just qc.kc_new; done by the last split
  if (split == p.nsplit - 1 && warp == 0) {  // whole warp runs the shuffle; lane group 0 keeps the result
    float kn[VEC], vn[VEC], qn[VEC], zero[VEC];
    Vec<T>::load(row_ptr(p.kc, 0), kn);
    Vec<T>::load(row_ptr(p.vc, 0), vn);
    Vec<T>::load(row_ptr(p.qu, 0), qn);
#pragma unroll
    for (int i = 0; i < VEC; ++i) zero[i] = 0.f;
    if (grp == 0) {
      Vec<T>::store(row_ptr(p.kcc, p.t), kn);
      Vec<T>::store(row_ptr(p.vcc, p.t), vn);
      Vec<T>::store(row_ptr(p.quc, p.t), qn);
      Vec<T>::store(row_ptr(p.U, p.t), zero);
    }
    float sc = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) sc += qcv[i] * kn[i];
    sc = group_sum<LPR>(sc);
    if (grp == 0) {
      float mn = fmaxf(m, sc);
      float corr = __expf(m - mn), pe = __expf(sc - mn);
      l = l * corr + pe;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = acc[i] * corr + pe * vn[i];
      m = mn;
    }
  }

  // merge the RPW lane groups of a warp, then the warps of the CTA
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
    float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    float mn = fmaxf(m, m2);
    float c1 = (m == -INFINITY) ? 0.f : __expf(m - mn), c2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
    l = l * c1 + l2 * c2;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float a2 = __shfl_xor_sync(0xffffffffu, acc[i], o);
      acc[i] = acc[i] * c1 + a2 * c2;
    }
    m = mn;
  }
  __shared__ float s_m[NW], s_l[NW], s_acc[NW][D];
  if (grp == 0) {
    if (sub == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < VEC; ++i) s_acc[warp][sub * VEC + i] = acc[i];
  }
  __syncthreads();
  if (threadIdx.x < D) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, s_m[w]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      float c = (s_m[w] == -INFINITY) ? 0.f : __expf(s_m[w] - mm);
      ll += s_l[w] * c;
      aa += s_acc[w][threadIdx.x] * c;
    }
    if (p.nsplit == 1) {
      T* o = reinterpret_cast<T*>(p.out.ptr) + b * p.out.stride_b + h * p.out.stride_h;
      if constexpr (sizeof(T) == 4) o[threadIdx.x] = aa / ll;
      else o[threadIdx.x] = Elem<T>::from_f(aa / ll);
    } else {
      float* dst = p.part + ((int64_t)bh * p.nsplit + split) * (2 + D);
      if (threadIdx.x == 0) { dst[0] = mm; dst[1] = ll; }
      dst[2 + threadIdx.x] = aa;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Same step, with the four caches brought in by bulk asynchronous copies (the TMA engine) into a
// ring of shared-memory stages instead of per-thread loads: the bytes in flight no longer depend
// on how many warps are resident or on how many registers a thread can spare.  One thread issues,
// per stage, four contiguous copies (the rows of a tile are adjacent in each cache, which is why
// this variant needs position stride == dim_head); the warps consume a stage row group by row
// group, write U back from registers, and the stage is refilled after a block-wide barrier.
constexpr int kRingRows = 16;     // rows per stage
constexpr int kRingStages = 3;

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <typename T, int D>
__global__ void __launch_bounds__(kDecodeThreads, 4) castle_decode_ring_kernel(const DecodeParams p) {
  constexpr int VEC = Vec<T>::N;
  constexpr int LPR = D / VEC;
  constexpr int RPW = 32 / LPR;
  constexpr int NW = kDecodeThreads / 32;
  constexpr int PASSES = (kRingRows + RPW * NW - 1) / (RPW * NW);
  constexpr uint32_t ROWB = D * sizeof(T);
  constexpr uint32_t TENB = kRingRows * ROWB;            // one tensor's tile
  extern __shared__ __align__(128) uint8_t ring[];       // [stage][tensor: qu, U, kc, vc][row][D]
  __shared__ uint64_t full[kRingStages];
  __shared__ int abort_flag;
  __shared__ float s_m[NW], s_l[NW], s_acc[NW][D];

  const int bh = blockIdx.x, split = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPR, grp = lane / LPR;
  const int64_t col = (int64_t)sub * VEC;
  volatile int* abortp = &abort_flag;

  auto row_ptr = [&](const castle_tensor_t& t, int64_t r) {
    return reinterpret_cast<T*>(t.ptr) + b * t.stride_b + h * t.stride_h + r * t.stride_n + col;
  };
  const int r_begin = split * p.rows_per_split;
  const int r_end = min(p.t, r_begin + p.rows_per_split);
  const int ntiles = (max(r_end - r_begin, 0) + kRingRows - 1) / kRingRows;

  auto issue = [&](int tile) {  // thread 0 only
    const int st = tile % kRingStages;
    const int r0 = r_begin + tile * kRingRows;
    const uint32_t bytes = (uint32_t)min(kRingRows, r_end - r0) * ROWB;
    uint8_t* dst = ring + (size_t)st * 4 * TENB;
    mbar_expect_tx(&full[st], 4 * bytes);
    bulk_load(dst, row_ptr(p.quc, r0) - col, bytes, &full[st]);
    bulk_load(dst + TENB, row_ptr(p.U, r0) - col, bytes, &full[st]);
    bulk_load(dst + 2 * TENB, row_ptr(p.kcc, r0) - col, bytes, &full[st]);
    bulk_load(dst + 3 * TENB, row_ptr(p.vcc, r0) - col, bytes, &full[st]);
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRingStages; ++s) mbar_init(&full[s], 1);
    mbar_fence_init();
    abort_flag = 0;
  }
  __syncthreads();
  if (threadIdx.x == 0)
    for (int t0 = 0; t0 < kRingStages && t0 < ntiles; ++t0) issue(t0);

  float qcv[VEC], kuv[VEC], vuv[VEC];
  Vec<T>::load(row_ptr(p.qc, 0), qcv);
  Vec<T>::load(row_ptr(p.ku, 0), kuv);
  Vec<T>::load(row_ptr(p.vu, 0), vuv);
#pragma unroll
  for (int i = 0; i < VEC; ++i) { qcv[i] *= p.scale; kuv[i] *= p.scale; }

  float m = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int st = tile % kRingStages;
    mbar_wait(&full[st], (uint32_t)((tile / kRingStages) & 1), abortp);
    // A wait that ran out means this stage never arrived: the U cache is persistent state, so
    // nothing computed from such a stage may be stored.  (No early exit: the barrier below must
    // still be reached by every thread.)
    const bool arrived = (*abortp == 0);
    const uint8_t* src = ring + (size_t)st * 4 * TENB;
    const int r0 = r_begin + tile * kRingRows;
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps) {
      const int rr = ps * RPW * NW + warp * RPW + grp;   // row inside the tile
      const int r = r0 + rr;
      const bool live = arrived && rr < kRingRows && r < r_end;
      float quv[VEC], uv[VEC], kv[VEC], vv[VEC];
      if (live) {
        const T* base = reinterpret_cast<const T*>(src) + (size_t)rr * D + col;
        Vec<T>::load(base, quv);
        Vec<T>::load(base + kRingRows * D, uv);
        Vec<T>::load(base + 2 * kRingRows * D, kv);
        Vec<T>::load(base + 3 * kRingRows * D, vv);
      }
      float z = 0.f, sc = 0.f, su = 0.f;
      if (live) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) z += quv[i] * kuv[i];
      }
      z = group_sum<LPR>(z);
      const float a = sigmoid_f(z);
      if (live) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) uv[i] += a * vuv[i];
        Vec<T>::round(uv);
        Vec<T>::store(row_ptr(p.U, r), uv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) { sc += qcv[i] * kv[i]; su += qcv[i] * uv[i]; }
      }
      sc = group_sum<LPR>(sc);
      su = group_sum<LPR>(su);
      if (live) {
        const float s = sc - su * sigmoid_f(su);
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn), pe = __expf(s - mn);
        l = l * corr + pe;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = acc[i] * corr + pe * vv[i];
        m = mn;
      }
    }
    __syncthreads();  // every warp is done with this stage
    if (threadIdx.x == 0 && tile + kRingStages < ntiles) issue(tile + kRingStages);
  }

  // the appended row: U[t] = 0 so its score is just qc.kc_new; done by the last split
  if (split == p.nsplit - 1 && warp == 0) {
    float kn[VEC], vn[VEC], qn[VEC], zero[VEC];
    Vec<T>::load(row_ptr(p.kc, 0), kn);
    Vec<T>::load(row_ptr(p.vc, 0), vn);
    Vec<T>::load(row_ptr(p.qu, 0), qn);
#pragma unroll
    for (int i = 0; i < VEC; ++i) zero[i] = 0.f;
    if (grp == 0 && *abortp == 0) {   // a timed-out step leaves the caches as they were
      Vec<T>::store(row_ptr(p.kcc, p.t), kn);
      Vec<T>::store(row_ptr(p.vcc, p.t), vn);
      Vec<T>::store(row_ptr(p.quc, p.t), qn);
      Vec<T>::store(row_ptr(p.U, p.t), zero);
    }
    float sc = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) sc += qcv[i] * kn[i];
    sc = group_sum<LPR>(sc);
    if (grp == 0) {
      const float mn = fmaxf(m, sc);
      const float corr = __expf(m - mn), pe = __expf(sc - mn);
      l = l * corr + pe;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = acc[i] * corr + pe * vn[i];
      m = mn;
    }
  }

  // merge the lane groups of a warp, then the warps of the CTA
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float mn = fmaxf(m, m2);
    const float c1 = (m == -INFINITY) ? 0.f : __expf(m - mn), c2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
    l = l * c1 + l2 * c2;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float a2 = __shfl_xor_sync(0xffffffffu, acc[i], o);
      acc[i] = acc[i] * c1 + a2 * c2;
    }
    m = mn;
  }
  if (grp == 0) {
    if (sub == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < VEC; ++i) s_acc[warp][sub * VEC + i] = acc[i];
  }
  __syncthreads();
  if (threadIdx.x < D) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, s_m[w]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float c = (s_m[w] == -INFINITY) ? 0.f : __expf(s_m[w] - mm);
      ll += s_l[w] * c;
      aa += s_acc[w][threadIdx.x] * c;
    }
    if (p.nsplit == 1) {
      T* o = reinterpret_cast<T*>(p.out.ptr) + b * p.out.stride_b + h * p.out.stride_h;
      if constexpr (sizeof(T) == 4) o[threadIdx.x] = aa / ll;
      else o[threadIdx.x] = Elem<T>::from_f(aa / ll);
    } else {
      float* dst = p.part + ((int64_t)bh * p.nsplit + split) * (2 + D);
      if (threadIdx.x == 0) { dst[0] = mm; dst[1] = ll; }
      dst[2 + threadIdx.x] = aa;
    }
  }
  if (threadIdx.x == 0 && abort_flag) atomicOr(p.status, CASTLE_STATUS_WAIT_TIMEOUT);
}

template <typename T, int D>
__global__ void castle_decode_merge_kernel(const DecodeParams p) {
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H, c = threadIdx.x;
  const float* src = p.part + (int64_t)bh * p.nsplit * (2 + D);
  float mm = -INFINITY;
  for (int s = 0; s < p.nsplit; ++s) mm = fmaxf(mm, src[s * (2 + D)]);
  float ll = 0.f, aa = 0.f;
  for (int s = 0; s < p.nsplit; ++s) {
    float ms = src[s * (2 + D)];
    float w = (ms == -INFINITY) ? 0.f : __expf(ms - mm);
    ll += src[s * (2 + D) + 1] * w;
    aa += src[s * (2 + D) + 2 + c] * w;
  }
  T* o = reinterpret_cast<T*>(p.out.ptr) + b * p.out.stride_b + h * p.out.stride_h;
  if constexpr (sizeof(T) == 4) o[c] = aa / ll;
  else o[c] = Elem<T>::from_f(aa / ll);
}

// How many CTAs share the rows of one (batch, head) pair.  The kernel is bandwidth bound and runs
// CASTLE_DECODE_MIN_CTAS CTAs per SM, so what matters is that the grid fills whole "waves" of
// resident CTAs: pick the smallest split (at least 128 rows each, at most 64) whose last wave is
// nearly full.
static int decode_nsplit(int BH, int t, int ctas_per_sm = CASTLE_DECODE_MIN_CTAS) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      sms = n;
    else
      sms = 148;
  }
  const int slots = sms * ctas_per_sm;
  int max_ns = t / 128;
  if (max_ns > 64) max_ns = 64;
  if (max_ns < 1) max_ns = 1;
  int best = 1;
  double best_eff = 0.0;
  for (int ns = 1; ns <= max_ns; ++ns) {
    const long long total = (long long)BH * ns;
    const long long waves = (total + slots - 1) / slots;
    const double eff = (double)total / (double)(waves * slots);
    if (eff > best_eff + 0.02) { best_eff = eff; best = ns; }
  }
  return best;
}

constexpr int kRingCtasPerSm = 4;

// The bulk-copy variant needs rows that are adjacent in memory and at least 128 bytes long.
static bool decode_use_ring(int D, int dtype, const castle_tensor_t* const* caches) {
  if (kDecodeThreads != 128 || D * elem_size(dtype) < 128) return false;
  for (int i = 0; i < 4; ++i)
    if (caches[i]->stride_n != D) return false;
  return true;
}

template <typename T, int D>
static int launch_decode(const DecodeParams& p, int BH, bool ring, cudaStream_t st) {
  dim3 grid(BH, p.nsplit);
  if constexpr (D * sizeof(T) >= 128) {
    if (ring) {
      constexpr size_t smem = (size_t)kRingStages * 4 * kRingRows * D * sizeof(T);
      cudaError_t e = cudaFuncSetAttribute(castle_decode_ring_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cuda_fail(e, "castle_decode_step attribute");
      ev_start(CASTLE_KERNEL_DECODE, st);
      castle_decode_ring_kernel<T, D><<<grid, kDecodeThreads, smem, st>>>(p);
      ev_stop(CASTLE_KERNEL_DECODE, st);
      if (p.nsplit > 1) castle_decode_merge_kernel<T, D><<<BH, D, 0, st>>>(p);
      e = cudaGetLastError();
      return e == cudaSuccess ? 0 : cuda_fail(e, "castle_decode_step launch");
    }
  }
  ev_start(CASTLE_KERNEL_DECODE, st);
  castle_decode_kernel<T, D><<<grid, kDecodeThreads, 0, st>>>(p);
  ev_stop(CASTLE_KERNEL_DECODE, st);
  if (p.nsplit > 1) castle_decode_merge_kernel<T, D><<<BH, D, 0, st>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : cuda_fail(e, "castle_decode_step launch");
}

template <typename T>
static int launch_decode_d(const DecodeParams& p, int BH, int D, bool ring, cudaStream_t st) {
  switch (D) {
    case 16: return launch_decode<T, 16>(p, BH, ring, st);
    case 32: return launch_decode<T, 32>(p, BH, ring, st);
    case 64: return launch_decode<T, 64>(p, BH, ring, st);
    case 128: return launch_decode<T, 128>(p, BH, ring, st);
  }
  return reject("castle_decode_step: dim_head %d not supported (16, 32, 64, 128)", D);
}

}  // namespace castle

using namespace castle;

extern "C" size_t castle_decode_workspace_bytes(const castle_problem_t* p, int32_t cache_len) {
  if (!p) return 0;
  int BH = p->batch * p->heads;
  int ns = decode_nsplit(BH, cache_len), ns_ring = decode_nsplit(BH, cache_len, kRingCtasPerSm);
  return (size_t)BH * (ns > ns_ring ? ns : ns_ring) * (2 + p->dim_head) * sizeof(float);
}

extern "C" int castle_decode_step(const castle_problem_t* p, int32_t cache_len, int32_t capacity,
                                  const castle_tensor_t* qc_new, const castle_tensor_t* kc_new,
                                  const castle_tensor_t* vc_new, const castle_tensor_t* qu_new,
                                  const castle_tensor_t* ku_new, const castle_tensor_t* vu_new,
                                  const castle_tensor_t* u_cache, const castle_tensor_t* qu_cache,
                                  const castle_tensor_t* kc_cache, const castle_tensor_t* vc_cache,
                                  const castle_tensor_t* out, void* workspace, size_t workspace_bytes,
                                  int32_t* status, void* stream) {
  if (!p) return reject("castle_decode_step: null problem");
  if (p->batch <= 0 || p->heads <= 0) return reject("castle_decode_step: empty batch/heads");
  if (cache_len < 0 || cache_len >= capacity)
    return reject("castle_decode_step: cache_len %d must be in [0, capacity %d)", cache_len, capacity);
  if (p->dtype != CASTLE_BF16 && p->dtype != CASTLE_F16 && p->dtype != CASTLE_F32)
    return reject("castle_decode_step: unknown dtype %d", p->dtype);
  int rc = 0;
  const castle_tensor_t* ts[11] = {qc_new, kc_new, vc_new, qu_new, ku_new, vu_new, u_cache, qu_cache, kc_cache, vc_cache, out};
  const char* names[11] = {"qc_new", "kc_new", "vc_new", "qu_new", "ku_new", "vu_new", "u_cache", "qu_cache", "kc_cache", "vc_cache", "out"};
  for (int i = 0; i < 11; ++i)
    if (!tensor_ok(ts[i], p->dtype, names[i], &rc)) return rc;
  DecodeParams dp;
  dp.qc = *qc_new; dp.kc = *kc_new; dp.vc = *vc_new; dp.qu = *qu_new; dp.ku = *ku_new; dp.vu = *vu_new;
  dp.U = *u_cache; dp.quc = *qu_cache; dp.kcc = *kc_cache; dp.vcc = *vc_cache; dp.out = *out;
  int BH = p->batch * p->heads;
  dp.H = p->heads; dp.t = cache_len; dp.scale = p->scale; dp.status = status;
  const castle_tensor_t* caches[4] = {u_cache, qu_cache, kc_cache, vc_cache};
  const bool ring = status != nullptr && decode_use_ring(p->dim_head, p->dtype, caches);
  dp.nsplit = decode_nsplit(BH, cache_len, ring ? kRingCtasPerSm : CASTLE_DECODE_MIN_CTAS);
  dp.rows_per_split = (cache_len + dp.nsplit - 1) / dp.nsplit;
  if (dp.rows_per_split < 1) dp.rows_per_split = 1;
  dp.part = (float*)workspace;
  if (dp.nsplit > 1) {
    size_t need = (size_t)BH * dp.nsplit * (2 + p->dim_head) * sizeof(float);
    if (!workspace || workspace_bytes < need)
      return reject("castle_decode_step: workspace too small (%zu < %zu bytes)", workspace_bytes, need);
  }
  cudaStream_t st = (cudaStream_t)stream;
  switch (p->dtype) {
    case CASTLE_BF16: return launch_decode_d<__nv_bfloat16>(dp, BH, p->dim_head, ring, st);
    case CASTLE_F16: return launch_decode_d<__half>(dp, BH, p->dim_head, ring, st);
    default: return launch_decode_d<float>(dp, BH, p->dim_head, ring, st);
  }
}

// ---------------------------------------------------------------------------
// Decode step for hosts that may not allocate device memory on the token path.
//
// Some callers of this library cannot hand over a scratch buffer: a serving
// loop whose own arena took all device memory at start-up (so a cudaMalloc on
// the token path would fail, and would stall the device even if it did not), or
// a small non-torch host that binds only this C ABI and has no device allocator
// of its own.  For them the split partials of the decode step live in a fixed
// array inside the library image.  Every GPU that loads the library carries
// this array (520 KiB) until the process exits.
namespace castle {

constexpr int kStaticMaxSlots = 1024;          // batch * heads * row-splits
constexpr int kStaticSlotFloats = 2 + 128;     // (max, sum) + dim_head values, dim_head <= 128
static __device__ __align__(256) float g_decode_static_scratch[kStaticMaxSlots * kStaticSlotFloats];

// In host code the array's name is only a handle for the runtime, not an address a kernel may
// use; the device address is looked up once per device and kept here.
constexpr int kMaxDevices = 64;
static float* g_decode_static_ptr[kMaxDevices] = {nullptr};
static std::mutex g_decode_static_mu;   // host threads may make their first call on a device at the same time

}  // namespace castle

extern "C" int castle_decode_step_static(const castle_problem_t* p, int32_t cache_len, int32_t capacity,
                                         const castle_tensor_t* qc_new, const castle_tensor_t* kc_new,
                                         const castle_tensor_t* vc_new, const castle_tensor_t* qu_new,
                                         const castle_tensor_t* ku_new, const castle_tensor_t* vu_new,
                                         const castle_tensor_t* u_cache, const castle_tensor_t* qu_cache,
                                         const castle_tensor_t* kc_cache, const castle_tensor_t* vc_cache,
                                         const castle_tensor_t* out, int32_t* status, void* stream) {
  if (!p) return reject("castle_decode_step_static: null problem");
  if (p->batch <= 0 || p->heads <= 0) return reject("castle_decode_step_static: empty batch/heads");
  if (cache_len < 0 || cache_len >= capacity)
    return reject("castle_decode_step_static: cache_len %d must be in [0, capacity %d)", cache_len, capacity);
  if (p->dtype != CASTLE_BF16 && p->dtype != CASTLE_F16 && p->dtype != CASTLE_F32)
    return reject("castle_decode_step_static: unknown dtype %d", p->dtype);
  int rc = 0;
  const castle_tensor_t* ts[11] = {qc_new, kc_new, vc_new, qu_new, ku_new, vu_new, u_cache, qu_cache, kc_cache, vc_cache, out};
  const char* names[11] = {"qc_new", "kc_new", "vc_new", "qu_new", "ku_new", "vu_new", "u_cache", "qu_cache", "kc_cache", "vc_cache", "out"};
  for (int i = 0; i < 11; ++i)
    if (!tensor_ok(ts[i], p->dtype, names[i], &rc)) return rc;
  const int BH = p->batch * p->heads;
  const int nsplit = decode_nsplit(BH, cache_len);
  if (p->dim_head > 128 || (int64_t)BH * nsplit > kStaticMaxSlots)
    return reject("castle_decode_step_static: batch*heads*splits = %lld exceeds the built-in scratch of %d partials "
                  "(dim_head <= 128); use castle_decode_step with a caller-owned workspace",
                  (long long)BH * nsplit, kStaticMaxSlots);
  // set-up, once per device, with that device current
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "castle_decode_step_static cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return reject("castle_decode_step_static: device ordinal %d not supported", dev);
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_decode_static_mu);
    if (g_decode_static_ptr[dev] == nullptr) {
      float* ptr = nullptr;
      e = cudaGetSymbolAddress((void**)&ptr, g_decode_static_scratch);
      if (e != cudaSuccess) return cuda_fail(e, "castle_decode_step_static cudaGetSymbolAddress");
      g_decode_static_ptr[dev] = ptr;
    }
    scratch = g_decode_static_ptr[dev];
  }
  DecodeParams dp;
  dp.qc = *qc_new; dp.kc = *kc_new; dp.vc = *vc_new; dp.qu = *qu_new; dp.ku = *ku_new; dp.vu = *vu_new;
  dp.U = *u_cache; dp.quc = *qu_cache; dp.kcc = *kc_cache; dp.vcc = *vc_cache; dp.out = *out;
  dp.H = p->heads; dp.t = cache_len; dp.scale = p->scale; dp.status = status;
  dp.nsplit = nsplit;
  dp.rows_per_split = (cache_len + nsplit - 1) / nsplit;
  if (dp.rows_per_split < 1) dp.rows_per_split = 1;
  // Every partial slot the merge kernel reads is written by this same call first, so the
  // array needs no clearing between calls even though it keeps the previous call's contents.
  dp.part = scratch;
  cudaStream_t st = (cudaStream_t)stream;
  switch (p->dtype) {
    case CASTLE_BF16: return launch_decode_d<__nv_bfloat16>(dp, BH, p->dim_head, false, st);
    case CASTLE_F16: return launch_decode_d<__half>(dp, BH, p->dim_head, false, st);
    default: return launch_decode_d<float>(dp, BH, p->dim_head, false, st);
  }
}
