// H W^T per head (core.py:93,98-99 folded): the projected linear state that the tcgen05 forward kernels
// read in their epilogue, where the linear read-out  o = o_s + round(phi(q) (H W^T) / den + b)  is fused.
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
  pdl_wait();
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

template <typename T, int D>
static int launch_state_proj(const sla_shape* s, void* lin_state, const void* wbits, cudaStream_t st) {
  auto pk = state_proj_kernel<T, D>;
  int psmem = 2 * D * D * 2;
  SLA_CUDA_OK(cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, psmem));
  SLA_CUDA_OK(launch_pdl<false>(pk, dim3(s->B * s->H), dim3(D / 16 * 32), psmem, st, static_cast<T*>(lin_state),
                         static_cast<const T*>(wbits)));
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

}  // namespace sla
