// Linear-branch read-out, proj_l and the final sum as a streaming kernel (core.py:90,95-100):
//   o = o_s + round( (phi(q) H / (1e-5 + phi(q).z)) W^T + b ) = o_s + round( phi(q) (H W^T) / den + b )
// H W^T is one D x D matrix per head, prepared by a tiny kernel, so a row tile needs a single GEMM.
// Used after the tcgen05 sparse forward; o_s may alias o (each CTA reads its 64 rows before writing
// them). HBM-bound: reads q and o_s, writes o (3 * L * D * 2 bytes per head); H W^T stays in L2.
#include "common.cuh"
#include "kernels.h"

namespace sla {

// HW[bh][i][n] = sum_k H[bh][i][k] W[n][k], rounded to T: one CTA per head, one warp per 16 rows.
// Both operands are staged in shared memory with coalesced copies; the result is written behind H and
// z in the head's state record (the backward reuses it: (W H^T)[n][i] = HW[i][n]).
template <typename T, int D>
__global__ void __launch_bounds__(D / 16 * 32) state_proj_kernel(T* __restrict__ lin_state,
                                                                 const T* __restrict__ wbits) {
  constexpr int NT = D / 16 * 32, KS = D / 16;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sA = smem;               // H [i][k]
  unsigned char* sB = smem + D * D * 2;   // W [n][k]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T* rec = lin_state + static_cast<size_t>(blockIdx.x) * (2 * D * D + D);
  const uint32_t sA_a = smem_u32(sA), sB_a = smem_u32(sB);
  load_tile_async<D, D>(sA_a, rec, 0, D, tid, NT);
  load_tile_async<D, D>(sB_a, wbits, 0, D, tid, NT);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t a[KS][4];
  load_a_frags<D, KS>(a, sA_a, warp * 16, 0, lane);
  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  gemm_b_nk<T, D, D / 8, KS>(acc, a, sB_a, 0, 0, lane);
  __syncthreads();   // every warp has its A fragments: the H tile can be overwritten with the result
  store_acc_to_tile<T, D, D / 8>(sA, acc, warp * 16, lane);
  flush16<T, D>(sA, warp * 16, rec + D * D + D, warp * 16, D, lane, false);
}

template <typename T, int D, int FEAT>
__global__ void __launch_bounds__(128) linear_readout_kernel(FwdParams p) {
  constexpr int NT = 128, KS = D / 16;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;                 // [64][D], reused as output staging
  unsigned char* sO = sQ + 64 * D * 2;      // [64][D] o_s
  unsigned char* sH = sO + 64 * D * 2;      // [D][D] H W^T, [i][n]
  __shared__ float s_z[D];
  __shared__ float s_bias[D];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int bh = blockIdx.y, row0 = blockIdx.x * 64, m0 = warp * 16;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* qg = static_cast<const T*>(p.q) + head_off;
  const T* osg = static_cast<const T*>(p.o_s) + head_off;
  const T* hs = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);
  const T* wb = static_cast<const T*>(p.wbits);
  const T* hw = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D) + D * D + D;
  const uint32_t sQ_a = smem_u32(sQ), sO_a = smem_u32(sO), sH_a = smem_u32(sH);
  load_tile_async<D, 64>(sQ_a, qg, row0, L, tid, NT);
  load_tile_async<D, 64>(sO_a, osg, row0, L, tid, NT);
  load_tile_async<D, D>(sH_a, hw, 0, D, tid, NT);
  cp_async_commit();
  for (int i = tid; i < D; i += NT) {
    s_z[i] = Elem<T>::to_f(hs[D * D + i]);
    s_bias[i] = Elem<T>::to_f(wb[D * D + i]);
  }
  cp_async_wait<0>();
  __syncthreads();

  uint32_t pq[KS][4];
  {
    uint32_t qf[KS][4];
    load_a_frags<D, KS>(qf, sQ_a, m0, 0, lane);
    feature_map_frags<T, KS, FEAT>(pq, qf);
  }
  float num[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) num[j][0] = num[j][1] = num[j][2] = num[j][3] = 0.f;
  gemm_b_kn<T, D, D / 8, KS>(num, pq, sH_a, 0, 0, lane);  // phi(q) (H W^T)
  float d0 = 0.f, d1 = 0.f;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float2 ph = Elem<T>::unpack2(pq[kk][r]);
      int col = 16 * kk + (r >> 1) * 8 + 2 * t;
      float a = round_to<T>(ph.x * s_z[col]) + round_to<T>(ph.y * s_z[col + 1]);
      if (r & 1) d1 += a; else d0 += a;
    }
  }
  d0 = 1.f / round_to<T>(1e-5f + round_to<T>(quad_sum(d0)));
  d1 = 1.f / round_to<T>(1e-5f + round_to<T>(quad_sum(d1)));
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    int col = 8 * j + 2 * t;
    float2 a = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sO + tile_off<D>(m0 + g, j) + t * 4));
    float2 b = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sO + tile_off<D>(m0 + g + 8, j) + t * 4));
    num[j][0] = a.x + round_to<T>(num[j][0] * d0 + s_bias[col]);
    num[j][1] = a.y + round_to<T>(num[j][1] * d0 + s_bias[col + 1]);
    num[j][2] = b.x + round_to<T>(num[j][2] * d1 + s_bias[col]);
    num[j][3] = b.y + round_to<T>(num[j][3] * d1 + s_bias[col + 1]);
  }
  store_acc_to_tile<T, D, D / 8>(sQ, num, m0, lane);
  flush16<T, D>(sQ, m0, static_cast<T*>(p.o) + head_off, row0 + m0, L, lane, false);
}

template <typename T, int D, int FEAT>
static int launch_readout(const sla_shape* s, const FwdParams& p, cudaStream_t st) {
  auto kern = linear_readout_kernel<T, D, FEAT>;
  int smem = 2 * 64 * D * 2 + D * D * 2;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<dim3(ceil_div(s->L, 64), s->B * s->H), 128, smem, st>>>(p);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

template <typename T, int D>
static int readout_feat(const sla_shape* s, const FwdParams& p, cudaStream_t st) {
  switch (s->feature_map) {
    case SLA_PHI_SOFTMAX: return launch_readout<T, D, SLA_PHI_SOFTMAX>(s, p, st);
    case SLA_PHI_RELU: return launch_readout<T, D, SLA_PHI_RELU>(s, p, st);
    default: return launch_readout<T, D, SLA_PHI_ELU>(s, p, st);
  }
}

template <typename T, int D>
static int launch_state_proj(const sla_shape* s, void* lin_state, const void* wbits, cudaStream_t st) {
  auto pk = state_proj_kernel<T, D>;
  int psmem = 2 * D * D * 2;
  SLA_CUDA_OK(cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, psmem));
  pk<<<s->B * s->H, D / 16 * 32, psmem, st>>>(static_cast<T*>(lin_state), static_cast<const T*>(wbits));
  SLA_LAUNCH_OK();
  return SLA_OK;
}

// Fills the H W^T part of every head's state record (needs H already there).
int run_state_proj(const sla_shape* s, void* lin_state, const void* wbits, cudaStream_t st) {
  if (s->dtype == SLA_BF16)
    return s->D == 64 ? launch_state_proj<__nv_bfloat16, 64>(s, lin_state, wbits, st)
                      : launch_state_proj<__nv_bfloat16, 128>(s, lin_state, wbits, st);
  return s->D == 64 ? launch_state_proj<__half, 64>(s, lin_state, wbits, st)
                    : launch_state_proj<__half, 128>(s, lin_state, wbits, st);
}

int run_linear_readout(const sla_shape* s, const FwdParams& p, cudaStream_t st) {
  if (s->dtype == SLA_BF16)
    return s->D == 64 ? readout_feat<__nv_bfloat16, 64>(s, p, st) : readout_feat<__nv_bfloat16, 128>(s, p, st);
  return s->D == 64 ? readout_feat<__half, 64>(s, p, st) : readout_feat<__half, 128>(s, p, st);
}

}  // namespace sla
