// Linear branch restricted to the KV blocks a query block did NOT select (the scope drawn in the
// reference's assets/overview_of_SLA.png; the reference's code, sparse_linear_attention/core.py:92-96,
// sums over all tokens). For query block i
//   H_i = sum_{j not in sel(i)} phi(K_j)^T V_j = H_all - sum_{j in sel(i)} phi(K_j)^T V_j
//   z_i = z_all - sum_{j in sel(i)} sum_rows phi(K_j)
// so with C_num = sum_{j in sel(i)} (phi(Q_i) phi(K_j)^T) V_j and C_den = its row sums without V -- a
// block-sparse "attention" without softmax over the same LUT, computed by the tcgen05 forward kernel in its
// plain mode --
//   o_l = (phi(q) H_all - C_num) / (1e-5 + phi(q) . z_all - C_den),   o = o_s + round(o_l W^T + b).
// The complement form costs two extra GEMMs per selected pair instead of reading 25 D x D block states per
// query block. Its rounding error is about 2^-8 * (selected mass / unselected mass) of o_l: meant for small
// top-k ratios; when every block is selected o_l is defined as 0.
#include "common.cuh"
#include "kernels.h"

namespace sla {

// out = phi(x) rounded to T, row by row (core.py:90-91). One warp per row.
template <typename T, int D, int FEAT>
__global__ void __launch_bounds__(256) feature_map_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                          long long rows) {
  constexpr int EPL = D / 32;
  const long long r = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  float v[EPL];
  const T* src = x + r * D + lane * EPL;
#pragma unroll
  for (int e = 0; e < EPL; e += 2) {
    float2 f = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(src + e));
    v[e] = f.x; v[e + 1] = f.y;
  }
  if (FEAT == SLA_PHI_SOFTMAX) {
    float mx = v[0];
#pragma unroll
    for (int e = 1; e < EPL; ++e) mx = fmaxf(mx, v[e]);
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) { v[e] = __expf(v[e] - mx); s += v[e]; }
    s = 1.f / warp_sum(s);
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] *= s;
  } else if (FEAT == SLA_PHI_RELU) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = fmaxf(v[e], 0.f);
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[e] = v[e] > 0.f ? v[e] + 1.f : __expf(v[e]);
  }
  T* dst = out + r * D + lane * EPL;
#pragma unroll
  for (int e = 0; e < EPL; e += 2) *reinterpret_cast<uint32_t*>(dst + e) = Elem<T>::pack2(v[e], v[e + 1]);
}

template <typename T, int D>
static int feature_map_typed(const sla_shape* s, const T* x, T* out, cudaStream_t st) {
  const long long rows = static_cast<long long>(s->B) * s->H * s->L;
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  switch (s->feature_map) {
    case SLA_PHI_SOFTMAX: feature_map_kernel<T, D, SLA_PHI_SOFTMAX><<<grid, 256, 0, st>>>(x, out, rows); break;
    case SLA_PHI_RELU: feature_map_kernel<T, D, SLA_PHI_RELU><<<grid, 256, 0, st>>>(x, out, rows); break;
    default: feature_map_kernel<T, D, SLA_PHI_ELU><<<grid, 256, 0, st>>>(x, out, rows); break;
  }
  SLA_LAUNCH_OK();
  return SLA_OK;
}

int run_feature_map(const sla_shape* s, const void* x, void* out, cudaStream_t st) {
  if (s->dtype == SLA_BF16) {
    using T = __nv_bfloat16;
    return s->D == 64 ? feature_map_typed<T, 64>(s, (const T*)x, (T*)out, st) : feature_map_typed<T, 128>(s, (const T*)x, (T*)out, st);
  }
  using T = __half;
  return s->D == 64 ? feature_map_typed<T, 64>(s, (const T*)x, (T*)out, st) : feature_map_typed<T, 128>(s, (const T*)x, (T*)out, st);
}

// 64 query rows per CTA, one warp per 16 rows: phi(q) rows (already mapped, `p.q`), H, C_num, C_den in;
// o = o_s + round(round((phi(q) H - C_num) / den) W^T + b) out. o_s may alias o.
template <typename T, int D>
__global__ void __launch_bounds__(128) linear_readout_unselected_kernel(FwdParams p, const T* __restrict__ cnum,
                                                                        const float* __restrict__ cden,
                                                                        int all_selected) {
  constexpr int NT = 128, KS = D / 16, T64 = 64 * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;             // [64][D] phi(q), reused as output staging
  unsigned char* sO = sQ + T64;         // [64][D] o_s
  unsigned char* sC = sO + T64;         // [64][D] C_num
  unsigned char* sH = sC + T64;         // [D][D] H, [i][j]
  unsigned char* sW = sH + D * D * 2;   // [D][D] W, [n][k]
  __shared__ float s_z[D];
  __shared__ float s_bias[D];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int bh = blockIdx.y, row0 = blockIdx.x * 64, m0 = warp * 16;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* hs = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);
  const T* wb = static_cast<const T*>(p.wbits);
  const uint32_t sQ_a = smem_u32(sQ), sO_a = smem_u32(sO), sC_a = smem_u32(sC), sH_a = smem_u32(sH), sW_a = smem_u32(sW);
  load_tile_async<D, 64>(sQ_a, static_cast<const T*>(p.q) + head_off, row0, L, tid, NT);
  load_tile_async<D, 64>(sO_a, static_cast<const T*>(p.o_s) + head_off, row0, L, tid, NT);
  load_tile_async<D, 64>(sC_a, cnum + head_off, row0, L, tid, NT);
  load_tile_async<D, D>(sH_a, hs, 0, D, tid, NT);
  load_tile_async<D, D>(sW_a, wb, 0, D, tid, NT);
  cp_async_commit();
  for (int i = tid; i < D; i += NT) {
    s_z[i] = Elem<T>::to_f(hs[D * D + i]);
    s_bias[i] = Elem<T>::to_f(wb[D * D + i]);
  }
  cp_async_wait<0>();
  __syncthreads();

  uint32_t pq[KS][4];
  load_a_frags<D, KS>(pq, sQ_a, m0, 0, lane);
  float num[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) num[j][0] = num[j][1] = num[j][2] = num[j][3] = 0.f;
  gemm_b_kn<T, D, D / 8, KS>(num, pq, sH_a, 0, 0, lane);  // phi(q) H_all
  float d0 = 0.f, d1 = 0.f;                               // phi(q) . z_all
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float2 ph = Elem<T>::unpack2(pq[kk][r]);
      int col = 16 * kk + (r >> 1) * 8 + 2 * t;
      float a = ph.x * s_z[col] + ph.y * s_z[col + 1];
      if (r & 1) d1 += a; else d0 += a;
    }
  }
  const int gr0 = row0 + m0 + g, gr1 = gr0 + 8;
  const float c0 = gr0 < L ? cden[static_cast<size_t>(bh) * L + gr0] : 0.f;
  const float c1 = gr1 < L ? cden[static_cast<size_t>(bh) * L + gr1] : 0.f;
  d0 = 1.f / (1e-5f + (quad_sum(d0) - c0));
  d1 = 1.f / (1e-5f + (quad_sum(d1) - c1));
  if (all_selected) d0 = d1 = 0.f;                        // nothing is left for the linear branch
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    float2 a = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sC + tile_off<D>(m0 + g, j) + t * 4));
    float2 b = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sC + tile_off<D>(m0 + g + 8, j) + t * 4));
    num[j][0] = (num[j][0] - a.x) * d0;
    num[j][1] = (num[j][1] - a.y) * d0;
    num[j][2] = (num[j][2] - b.x) * d1;
    num[j][3] = (num[j][3] - b.y) * d1;
  }
  uint32_t ol[KS][4];
  acc_to_a_frags<T, KS>(ol, num);  // o_l in T
#pragma unroll
  for (int j = 0; j < D / 8; ++j) num[j][0] = num[j][1] = num[j][2] = num[j][3] = 0.f;
  gemm_b_nk<T, D, D / 8, KS>(num, ol, sW_a, 0, 0, lane);  // o_l W^T (core.py:99)
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    int col = 8 * j + 2 * t;
    float2 a = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sO + tile_off<D>(m0 + g, j) + t * 4));
    float2 b = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sO + tile_off<D>(m0 + g + 8, j) + t * 4));
    num[j][0] = a.x + round_to<T>(num[j][0] + s_bias[col]);
    num[j][1] = a.y + round_to<T>(num[j][1] + s_bias[col + 1]);
    num[j][2] = b.x + round_to<T>(num[j][2] + s_bias[col]);
    num[j][3] = b.y + round_to<T>(num[j][3] + s_bias[col + 1]);
  }
  store_acc_to_tile<T, D, D / 8>(sQ, num, m0, lane);
  flush16<T, D>(sQ, m0, static_cast<T*>(p.o) + head_off, row0 + m0, L, lane, false);
}

template <typename T, int D>
static int readout_unselected_typed(const sla_shape* s, const FwdParams& p, const void* cnum, const float* cden,
                                    cudaStream_t st) {
  auto kern = linear_readout_unselected_kernel<T, D>;
  const int smem = 3 * 64 * D * 2 + 2 * D * D * 2;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int nb = ceil_div(s->L, s->BLKK);
  kern<<<dim3(ceil_div(s->L, 64), s->B * s->H), 128, smem, st>>>(p, static_cast<const T*>(cnum), cden,
                                                                s->topk >= nb ? 1 : 0);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

// p.q must hold phi(q) (run_feature_map), p.o_s the sparse branch's output, p.lin_state H and z.
int run_linear_readout_unselected(const sla_shape* s, const FwdParams& p, const void* cnum, const float* cden,
                                  cudaStream_t st) {
  if (s->dtype == SLA_BF16)
    return s->D == 64 ? readout_unselected_typed<__nv_bfloat16, 64>(s, p, cnum, cden, st)
                      : readout_unselected_typed<__nv_bfloat16, 128>(s, p, cnum, cden, st);
  return s->D == 64 ? readout_unselected_typed<__half, 64>(s, p, cnum, cden, st)
                    : readout_unselected_typed<__half, 128>(s, p, cnum, cden, st);
}

}  // namespace sla
