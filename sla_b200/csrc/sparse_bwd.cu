// Backward of the block-sparse branch on warp-level MMA (legacy tensor path).
// Mathematics: sparse_linear_attention/kernel.py:85-237.
//   delta = rowsum(o_s * do)                      (kernel.py:102-105)
//   P = exp2(S * scale * log2e - lse), 0 for keys >= L
//   dP = dO V^T, dS = P * (dP - delta)
//   dQ = dS K * scale                             (query-block stationary, walks the LUT row)
//   dV = P^T dO, dK = dS^T Q * scale              (KV-block stationary)
// Unlike the reference's dK/dV kernel, which scans every query slice of the sequence and tests a
// mask byte (kernel.py:208-210), the KV-stationary kernel here walks the per-KV-block column list
// built together with the LUT, so its work is proportional to the number of selected pairs.
#include "common.cuh"
#include "kernels.h"

namespace sla {

__device__ inline float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------------------------
// dQ (and delta): one CTA per query block.
// ---------------------------------------------------------------------------------------------
template <typename T, int D, int BM>
__global__ void __launch_bounds__(BM / 16 * 32) sparse_bwd_dq_kernel(BwdParams p) {
  constexpr int NT = BM / 16 * 32;
  constexpr int KS = D / 16;
  constexpr int TILE_KV = 64 * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;
  unsigned char* sdO = sQ + BM * D * 2;
  unsigned char* sK = sdO + BM * D * 2;
  unsigned char* sV = sK + 2 * TILE_KV;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ib = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* qg = static_cast<const T*>(p.q) + head_off;
  const T* kg = static_cast<const T*>(p.k) + head_off;
  const T* vg = static_cast<const T*>(p.v) + head_off;
  const T* og = static_cast<const T*>(p.o_s) + head_off;
  const T* dog = static_cast<const T*>(p.d_o) + head_off;
  const int32_t* lut = p.lut + (static_cast<size_t>(bh) * p.mb + ib) * p.topk;
  const int q_row0 = ib * BM, m0 = warp * 16;
  const uint32_t sQ_a = smem_u32(sQ), sdO_a = smem_u32(sdO), sK_a = smem_u32(sK), sV_a = smem_u32(sV);

  load_tile_async<D, BM>(sQ_a, qg, q_row0, L, tid, NT);
  load_tile_async<D, BM>(sdO_a, dog, q_row0, L, tid, NT);
  int idx_n = lut[0];
  load_tile_async<D, 64>(sK_a, kg, idx_n * 64, L, tid, NT);
  load_tile_async<D, 64>(sV_a, vg, idx_n * 64, L, tid, NT);
  cp_async_commit();

  // delta for this warp's 16 rows, straight from global memory (kernel.py:102-105)
  float* delta_g = p.delta + static_cast<size_t>(bh) * L;
  const float* lse_g = p.lse + static_cast<size_t>(bh) * L;
  float my_delta0 = 0.f, my_delta1 = 0.f;
  {
    constexpr int EPL = D / 32;
    for (int r = 0; r < 16; ++r) {
      int gr = q_row0 + m0 + r;
      float s = 0.f;
      if (gr < L) {
        const T* a = og + static_cast<size_t>(gr) * D + lane * EPL;
        const T* b = dog + static_cast<size_t>(gr) * D + lane * EPL;
#pragma unroll
        for (int e = 0; e < EPL; e += 2) {
          float2 x = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(a + e));
          float2 y = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(b + e));
          s += x.x * y.x + x.y * y.y;
        }
      }
      s = warp_sum(s);
      if (lane == 0 && gr < L) delta_g[gr] = s;
      if (r == g) my_delta0 = s;
      if (r == g + 8) my_delta1 = s;
    }
  }
  const int r0 = q_row0 + m0 + g, r1 = r0 + 8;
  const float lse0 = r0 < L ? lse_g[r0] : INFINITY;  // rows past the end give P = 0 (kernel.py:144)
  const float lse1 = r1 < L ? lse_g[r1] : INFINITY;

  uint32_t qf[KS][4];
  float dq[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) dq[j][0] = dq[j][1] = dq[j][2] = dq[j][3] = 0.f;
  const float sc = p.scale_log2;

  for (int it = 0; it < p.topk; ++it) {
    const int stage = it & 1;
    int next_n = 0;
    if (it + 1 < p.topk) {
      next_n = lut[it + 1];
      load_tile_async<D, 64>(sK_a + (stage ^ 1) * TILE_KV, kg, next_n * 64, L, tid, NT);
      load_tile_async<D, 64>(sV_a + (stage ^ 1) * TILE_KV, vg, next_n * 64, L, tid, NT);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (it == 0) load_a_frags<D, KS>(qf, sQ_a, m0, 0, lane);

    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    gemm_b_nk<T, D, 8, KS>(s, qf, sK_a + stage * TILE_KV, 0, 0, lane);
    const int valid = L - idx_n * 64;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float pv = bwd_exp2(s[j][c] * sc - ((c & 2) ? lse1 : lse0));
        if (valid < 64 && (8 * j + 2 * t + (c & 1)) >= valid) pv = 0.f;  // kernel.py:157
        s[j][c] = pv;
      }
    }
    float dp[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) dp[j][0] = dp[j][1] = dp[j][2] = dp[j][3] = 0.f;
    gemm_at_b_nk<T, D, 8, KS>(dp, sdO_a, m0, sV_a + stage * TILE_KV, lane);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j][0] *= dp[j][0] - my_delta0;
      s[j][1] *= dp[j][1] - my_delta0;
      s[j][2] *= dp[j][2] - my_delta1;
      s[j][3] *= dp[j][3] - my_delta1;
    }
    uint32_t dsf[4][4];
    acc_to_a_frags<T, 4>(dsf, s);
    gemm_b_kn<T, D, D / 8, 4>(dq, dsf, sK_a + stage * TILE_KV, 0, 0, lane);
    __syncthreads();
    idx_n = next_n;
  }
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    dq[j][0] *= p.scale; dq[j][1] *= p.scale; dq[j][2] *= p.scale; dq[j][3] *= p.scale;  // kernel.py:164
  }
  store_acc_to_tile<T, D, D / 8>(sQ, dq, m0, lane);
  flush16<T, D>(sQ, m0, static_cast<T*>(p.dq) + head_off, q_row0 + m0, L, lane, p.accumulate != 0);
}

// ---------------------------------------------------------------------------------------------
// dK, dV: one CTA (4 warps x 16 keys) per KV block, walking the block's column list.
// ---------------------------------------------------------------------------------------------
template <typename T, int D, int BM>
__global__ void __launch_bounds__(128) sparse_bwd_dkdv_kernel(BwdParams p) {
  constexpr int NT = 128;
  constexpr int KS = D / 16;
  constexpr int TILE = 64 * D * 2;
  constexpr int SL = BM / 64;  // 64-row slices per query block (kernel.py:179)
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sK = smem;
  unsigned char* sV = sK + TILE;
  unsigned char* sQ = sV + TILE;        // [2][64][D]
  unsigned char* sdO = sQ + 2 * TILE;   // [2][64][D]
  float* sLse = reinterpret_cast<float*>(sdO + 2 * TILE);  // [2][64]
  float* sDelta = sLse + 128;                              // [2][64]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int jb = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* qg = static_cast<const T*>(p.q) + head_off;
  const T* kg = static_cast<const T*>(p.k) + head_off;
  const T* vg = static_cast<const T*>(p.v) + head_off;
  const T* dog = static_cast<const T*>(p.d_o) + head_off;
  const float* lse_g = p.lse + static_cast<size_t>(bh) * L;
  const float* delta_g = p.delta + static_cast<size_t>(bh) * L;
  const int32_t* offs = p.col_offsets + static_cast<size_t>(bh) * (p.nb + 1);
  const int c_begin = offs[jb], c_end = offs[jb + 1];
  const int32_t* cols = p.col_index + static_cast<size_t>(bh) * p.mb * p.topk + c_begin;
  const int nslices = (c_end - c_begin) * SL;
  const int m0 = warp * 16;
  const uint32_t sK_a = smem_u32(sK), sV_a = smem_u32(sV), sQ_a = smem_u32(sQ), sdO_a = smem_u32(sdO);

  auto slice_row0 = [&](int s) { return cols[s / SL] * BM + (s % SL) * 64; };
  auto prefetch = [&](int s, int stage) {
    int row0 = slice_row0(s);
    load_tile_async<D, 64>(sQ_a + stage * TILE, qg, row0, L, tid, NT);
    load_tile_async<D, 64>(sdO_a + stage * TILE, dog, row0, L, tid, NT);
    if (tid < 64) {
      int r = row0 + tid;
      sLse[stage * 64 + tid] = r < L ? lse_g[r] : INFINITY;
      sDelta[stage * 64 + tid] = r < L ? delta_g[r] : 0.f;
    }
  };

  load_tile_async<D, 64>(sK_a, kg, jb * 64, L, tid, NT);
  load_tile_async<D, 64>(sV_a, vg, jb * 64, L, tid, NT);
  if (nslices > 0) prefetch(0, 0);
  cp_async_commit();

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    dk[j][0] = dk[j][1] = dk[j][2] = dk[j][3] = 0.f;
    dv[j][0] = dv[j][1] = dv[j][2] = dv[j][3] = 0.f;
  }
  const float sc = p.scale_log2;
  const bool key_ok0 = jb * 64 + m0 + g < L, key_ok1 = jb * 64 + m0 + g + 8 < L;

  for (int s = 0; s < nslices; ++s) {
    const int stage = s & 1;
    if (s + 1 < nslices) {
      prefetch(s + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* lse_s = sLse + stage * 64;
    const float* del_s = sDelta + stage * 64;

    float st[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f;
    gemm_at_b_nk<T, D, 8, KS>(st, sK_a, m0, sQ_a + stage * TILE, lane);  // K Q^T (kernel.py:214)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2 ls = *reinterpret_cast<const float2*>(lse_s + 8 * j + 2 * t);
      st[j][0] = key_ok0 ? bwd_exp2(st[j][0] * sc - ls.x) : 0.f;  // kernel.py:215-216
      st[j][1] = key_ok0 ? bwd_exp2(st[j][1] * sc - ls.y) : 0.f;
      st[j][2] = key_ok1 ? bwd_exp2(st[j][2] * sc - ls.x) : 0.f;
      st[j][3] = key_ok1 ? bwd_exp2(st[j][3] * sc - ls.y) : 0.f;
    }
    uint32_t pf[4][4];
    acc_to_a_frags<T, 4>(pf, st);
    gemm_b_kn<T, D, D / 8, 4>(dv, pf, sdO_a + stage * TILE, 0, 0, lane);  // dV += P^T dO (kernel.py:220)
    float dpt[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) dpt[j][0] = dpt[j][1] = dpt[j][2] = dpt[j][3] = 0.f;
    gemm_at_b_nk<T, D, 8, KS>(dpt, sV_a, m0, sdO_a + stage * TILE, lane);  // V dO^T (kernel.py:223)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float2 de = *reinterpret_cast<const float2*>(del_s + 8 * j + 2 * t);
      st[j][0] *= dpt[j][0] - de.x;
      st[j][1] *= dpt[j][1] - de.y;
      st[j][2] *= dpt[j][2] - de.x;
      st[j][3] *= dpt[j][3] - de.y;
    }
    acc_to_a_frags<T, 4>(pf, st);
    gemm_b_kn<T, D, D / 8, 4>(dk, pf, sQ_a + stage * TILE, 0, 0, lane);  // dK += dS^T Q (kernel.py:225)
    __syncthreads();
  }
  if (nslices == 0) {
    cp_async_wait<0>();
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    dk[j][0] *= p.scale; dk[j][1] *= p.scale; dk[j][2] *= p.scale; dk[j][3] *= p.scale;  // kernel.py:236
  }
  // stage through the (now idle) Q ring: each warp only touches its own 16 rows
  store_acc_to_tile<T, D, D / 8>(sQ, dk, m0, lane);
  flush16<T, D>(sQ, m0, static_cast<T*>(p.dk) + head_off, jb * 64 + m0, L, lane, p.accumulate != 0);
  store_acc_to_tile<T, D, D / 8>(sQ, dv, m0, lane);
  flush16<T, D>(sQ, m0, static_cast<T*>(p.dv) + head_off, jb * 64 + m0, L, lane, p.accumulate != 0);
}

template <typename T, int D, int BM>
static int launch_bwd(const BwdParams& p, int bh, cudaStream_t st) {
  {
    auto kern = sparse_bwd_dq_kernel<T, D, BM>;
    int smem = 2 * BM * D * 2 + 4 * 64 * D * 2;
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<dim3(p.mb, bh), BM / 16 * 32, smem, st>>>(p);
    SLA_LAUNCH_OK();
  }
  {
    auto kern = sparse_bwd_dkdv_kernel<T, D, BM>;
    int smem = 6 * 64 * D * 2 + 4 * 64 * 4;
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<dim3(p.nb, bh), 128, smem, st>>>(p);
    SLA_LAUNCH_OK();
  }
  return SLA_OK;
}

template <typename T>
static int dispatch_bwd(const sla_shape* s, const BwdParams& p, cudaStream_t st) {
  int bh = s->B * s->H;
  if (s->D == 64) return s->BLKQ == 64 ? launch_bwd<T, 64, 64>(p, bh, st) : launch_bwd<T, 64, 128>(p, bh, st);
  return s->BLKQ == 64 ? launch_bwd<T, 128, 64>(p, bh, st) : launch_bwd<T, 128, 128>(p, bh, st);
}

int run_sparse_bwd_mma(const sla_shape* s, const BwdParams& p, cudaStream_t st) {
  if (s->dtype == SLA_BF16) return dispatch_bwd<__nv_bfloat16>(s, p, st);
  return dispatch_bwd<__half>(s, p, st);
}

}  // namespace sla
