// Shared by the backward kernels (dim_head 64 in bwd.cu, dim_head 128 in bwd128.cu): launch
// parameters, the delta pre-pass and the kernel that turns fp32 accumulators into gradients.
#pragma once
#include "common.cuh"
#include "sm100.cuh"

namespace castle {

constexpr int kBlkB = 128;
constexpr uint32_t kPanelB = kBlkB * 128;

struct BwdParams {
  int B, H, N, nblk;
  float scale;
  const float* lse;      // [BH][N]
  const float* w_state;  // [BH][N][D]
  float* delta;          // [BH][N]
  float* acc_dqc;        // [BH][N][D] fp32, zeroed
  float* acc_dvu;
  float* acc_dku;
  uint8_t* tiles;        // dim_head 128: per (pair, query block, key block) the 32 KB tiles A | dSu | Tm that the
                         // key/value kernel hands to the lookahead kernel
  int64_t ntiles;        // query-block x key-block pairs per (batch, head) pair
  int bh0;               // dim_head 128: first (batch, head) pair of this launch (the pairs run in chunks)
  int chunk_pairs;       // dim_head 128: pairs per chunk (what the caller's scratch holds)
  castle_tensor_t out, dout;
  castle_tensor_t dqc, dkc, dvc, dqu, dku, dvu;
  int32_t* status;
#ifdef CASTLE_PHASE_TIMING
  long long* timing;
#endif
};

// delta[b,h,i] = sum_d out * dout  (lookahead_keys_attention_triton.py:175-214 in the reference)
template <typename T, int D>
__global__ void castle_bwd_delta_kernel(const BwdParams p) {
  constexpr int LPR = D / 8;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x / LPR) + threadIdx.x / LPR;
  const int sub = threadIdx.x % LPR;
  const int64_t total = (int64_t)p.B * p.H * p.N;
  float s = 0.f;
  if (row < total) {
    int bh = row / p.N, i = row % p.N, b = bh / p.H, h = bh % p.H;
    const T* po = reinterpret_cast<const T*>(p.out.ptr) + b * p.out.stride_b + h * p.out.stride_h + (int64_t)i * p.out.stride_n + sub * 8;
    const T* pd = reinterpret_cast<const T*>(p.dout.ptr) + b * p.dout.stride_b + h * p.dout.stride_h + (int64_t)i * p.dout.stride_n + sub * 8;
    uint4 a = *reinterpret_cast<const uint4*>(po), c = *reinterpret_cast<const uint4*>(pd);
    const uint32_t* ua = &a.x; const uint32_t* uc = &c.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = Elem<T>::unpack2(ua[j]), y = Elem<T>::unpack2(uc[j]);
      s += x.x * y.x + x.y * y.y;
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (row < total && sub == 0) p.delta[row] = s;
}

// fp32 accumulators -> scaled 16-bit gradients in the caller's (strided) tensors.
// NACC = 3: dqc, dvu, dku (dqu is written by the kernel that owns the key block).
template <typename T, int D, int NACC>
__global__ void castle_bwd_finish_kernel(const BwdParams p) {
  constexpr int LPR = D / 8;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x / LPR) + threadIdx.x / LPR;
  const int sub = threadIdx.x % LPR;
  if (row >= (int64_t)p.B * p.H * p.N) return;
  int bh = row / p.N, i = row % p.N, b = bh / p.H, h = bh % p.H;
  const float* srcs[3] = {p.acc_dqc, p.acc_dvu, p.acc_dku};
  const castle_tensor_t* dsts[3] = {&p.dqc, &p.dvu, &p.dku};
#pragma unroll
  for (int t = 0; t < NACC; ++t) {
    const float4* s4 = reinterpret_cast<const float4*>(srcs[t] + row * D + sub * 8);
    float4 x = s4[0], y = s4[1];
    uint4 q;
    q.x = Elem<T>::pack2(x.x * p.scale, x.y * p.scale); q.y = Elem<T>::pack2(x.z * p.scale, x.w * p.scale);
    q.z = Elem<T>::pack2(y.x * p.scale, y.y * p.scale); q.w = Elem<T>::pack2(y.z * p.scale, y.w * p.scale);
    T* d = reinterpret_cast<T*>(dsts[t]->ptr) + b * dsts[t]->stride_b + h * dsts[t]->stride_h + (int64_t)i * dsts[t]->stride_n + sub * 8;
    *reinterpret_cast<uint4*>(d) = q;
  }
}

// dim_head 128 backward (bwd128.cu)
size_t bwd128_pair_bytes(int nblk);           // tile hand-over scratch of one (batch, head) pair
int bwd128_chunk_pairs(int BH, int nblk);     // pairs per launch pair that keep the scratch under its limit
int launch_bwd128(const BwdParams& p, int dtype, const CUtensorMap* in_maps, cudaStream_t st);

}  // namespace castle
