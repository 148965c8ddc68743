// Backward of the linear branch in the "unselected" scope (the scope drawn in the reference's
// assets/overview_of_SLA.png; the reference's code, sparse_linear_attention/core.py:92-96, sums over all tokens
// and has no such branch, so nothing here has a counterpart to be checked against but the CPU restatement).
//
// Forward, per query row of query block i (linear_unselected.cu):
//   N = phi_q H_all - C_num,   den = 1e-5 + phi_q . z_all - C_den,   o_l = N / den,   y = o_l W^T + b
//   C_num = sum_{j in sel(i)} (phi_q phi(K_j)^T) V_j,   C_den = its row sums without V.
// Backward, with dY the gradient of the module output and u = dY W (= d o_l):
//   dN = u / den,   dden = -(u . o_l) / den = -(phi_q . t - u . C_num) / den^2   with t = u H_all^T = dY (W H_all^T)
//   all-token terms:  dphi_q += t / den + dden z_all,   dH_all = sum phi_q^T dN = G^T W,   dz_all = sum dden phi_q
//                     with G[n][i] = sum_rows dY[n] (phi_q / den)[i]   (the shape of the all-token scope's pass A)
//   selected terms:   dC_num = -dN, dC_den = -dden: the block-sparse product WITHOUT softmax is differentiated by the
//                     tcgen05 backward kernels in their plain mode on (phi_q, phi_k, v) with dO = -dN and
//                     delta = dden, which yields the remaining parts of dphi_q, dphi_k and dv
//   proj_l:           dW = sum dY^T o_l = G H_all - G2,  G2[n][d] = sum_rows dY[n] (C_num / den)[d];   db = sum dY.
// This file holds the row pass (everything above that is per query row or a sum over query rows) and the
// element-wise backward of the feature map that turns the accumulated dphi_q into dq.
#include "common.cuh"
#include "kernels.h"

namespace sla {

// One CTA = one chunk of rows of one head, D rows per tile, one warp per 16 rows (the structure of the mma.sync
// pass A in linear_bwd.cu). Per-chunk partial record: G (D*D) | dz (D) | db (D) | G2 (D*D), fp32.
template <typename T, int D>
__global__ void __launch_bounds__(D / 16 * 32) linear_bwd_q_unselected_kernel(UnselBwdParams p) {
  constexpr int NW = D / 16, NT = NW * 32, KS = D / 16;
  constexpr int TILE = D * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sM = smem;               // H W^T = M^T, stored [i][n]
  unsigned char* sW = sM + TILE;          // W, stored [n][k]
  unsigned char* sP = sW + TILE;          // phi(q) rows, later phi(q) / den
  unsigned char* sdY = sP + TILE;
  unsigned char* sC = sdY + TILE;         // C_num rows, later C_num / den
  unsigned char* sS = sC + TILE;          // staging of the two row outputs
  float* s_z = reinterpret_cast<float*>(sS + TILE);    // [D]
  float* s_rowc = s_z + D;                              // [D] dden * den per row of the tile

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ch = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* pqg = static_cast<const T*>(p.phiq) + head_off;
  const T* dyg = static_cast<const T*>(p.d_o) + head_off;
  const T* cng = static_cast<const T*>(p.cnum) + head_off;
  T* dng = static_cast<T*>(p.dn_neg) + head_off;
  T* dpg = static_cast<T*>(p.dphi) + head_off;
  const T* hs = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);
  const uint32_t sM_a = smem_u32(sM), sW_a = smem_u32(sW), sP_a = smem_u32(sP), sdY_a = smem_u32(sdY),
                 sC_a = smem_u32(sC);
  const int m0 = warp * 16;

  load_tile_async<D, D>(sM_a, hs + D * D + D, 0, D, tid, NT);
  load_tile_async<D, D>(sW_a, p.wbits, 0, D, tid, NT);
  cp_async_commit();
  for (int i = tid; i < D; i += NT) s_z[i] = Elem<T>::to_f(hs[D * D + i]);

  float gacc[D / 8][4], g2acc[D / 8][4];   // rows [16 warp, +16) of G[n][i] and of G2[n][d]
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    gacc[j][0] = gacc[j][1] = gacc[j][2] = gacc[j][3] = 0.f;
    g2acc[j][0] = g2acc[j][1] = g2acc[j][2] = g2acc[j][3] = 0.f;
  }
  float vec_acc = 0.f;   // thread tid < D: dz[tid]; tid >= D: db[tid - D]

  const int row_begin = ch * p.rows, row_end = min(L, row_begin + p.rows);
  for (int row0 = row_begin; row0 < row_end; row0 += D) {
    load_tile_async<D, D>(sP_a, pqg, row0, L, tid, NT);
    load_tile_async<D, D>(sdY_a, dyg, row0, L, tid, NT);
    load_tile_async<D, D>(sC_a, cng, row0, L, tid, NT);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    uint32_t pq[KS][4];
    load_a_frags<D, KS>(pq, sP_a, m0, 0, lane);
    // den = 1e-5 + phi_q . z_all - C_den, in fp32 as the forward's read-out computes it
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float2 ph = Elem<T>::unpack2(pq[kk][r]);
        const int col = 16 * kk + (r >> 1) * 8 + 2 * t;
        const float a = ph.x * s_z[col] + ph.y * s_z[col + 1];
        if (r & 1) d1 += a; else d0 += a;
      }
    }
    const int gr0 = row0 + m0 + g, gr1 = gr0 + 8;
    const float c0 = gr0 < L ? p.cden[static_cast<size_t>(bh) * L + gr0] : 0.f;
    const float c1 = gr1 < L ? p.cden[static_cast<size_t>(bh) * L + gr1] : 0.f;
    d0 = 1e-5f + (quad_sum(d0) - c0);
    d1 = 1e-5f + (quad_sum(d1) - c1);
    // every block selected: the forward defines o_l = 0, nothing but the bias gradient flows through this branch
    const float rd0 = p.all_selected ? 0.f : 1.f / d0, rd1 = p.all_selected ? 0.f : 1.f / d1;

    float acc[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    gemm_at_b_kn<T, D, D / 8, KS>(acc, sdY_a, m0, sW_a, lane);       // u[m][k] = sum_n dY[m][n] W[n][k]
    float uc0 = 0.f, uc1 = 0.f;                                       // u . C_num per row
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const float2 a = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sC + tile_off<D>(m0 + g, j) + t * 4));
      const float2 b = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(sC + tile_off<D>(m0 + g + 8, j) + t * 4));
      uc0 += acc[j][0] * a.x + acc[j][1] * a.y;
      uc1 += acc[j][2] * b.x + acc[j][3] * b.y;
      acc[j][0] *= -rd0; acc[j][1] *= -rd0;                           // -dN
      acc[j][2] *= -rd1; acc[j][3] *= -rd1;
    }
    uc0 = quad_sum(uc0);
    uc1 = quad_sum(uc1);
    store_acc_to_tile<T, D, D / 8>(sS, acc, m0, lane);
    flush16<T, D>(sS, m0, dng, row0 + m0, L, lane, false);

#pragma unroll
    for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    gemm_at_b_nk<T, D, D / 8, KS>(acc, sdY_a, m0, sM_a, lane);       // t[m][i] = sum_n dY[m][n] HW[i][n]
    float s0 = 0.f, s1 = 0.f;                                         // phi_q . t per row
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      const float2 p0 = Elem<T>::unpack2(pq[kk][0]), p1 = Elem<T>::unpack2(pq[kk][1]);
      const float2 p2 = Elem<T>::unpack2(pq[kk][2]), p3 = Elem<T>::unpack2(pq[kk][3]);
      s0 += acc[2 * kk][0] * p0.x + acc[2 * kk][1] * p0.y + acc[2 * kk + 1][0] * p2.x + acc[2 * kk + 1][1] * p2.y;
      s1 += acc[2 * kk][2] * p1.x + acc[2 * kk][3] * p1.y + acc[2 * kk + 1][2] * p3.x + acc[2 * kk + 1][3] * p3.y;
    }
    const float dden0 = -(quad_sum(s0) - uc0) * rd0 * rd0, dden1 = -(quad_sum(s1) - uc1) * rd1 * rd1;
    if (t == 0) {
      float2* st = p.stats + static_cast<size_t>(bh) * p.Lpad;
      if (gr0 < L) st[gr0] = make_float2(0.f, dden0);
      if (gr1 < L) st[gr1] = make_float2(0.f, dden1);
    }
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int col = 8 * j + 2 * t;
      acc[j][0] = acc[j][0] * rd0 + dden0 * s_z[col];
      acc[j][1] = acc[j][1] * rd0 + dden0 * s_z[col + 1];
      acc[j][2] = acc[j][2] * rd1 + dden1 * s_z[col];
      acc[j][3] = acc[j][3] * rd1 + dden1 * s_z[col + 1];
    }
    // the all-token part of dphi_q; the selected blocks' part is added by the plain dQ kernel before phi' is applied
    store_acc_to_tile<T, D, D / 8>(sS, acc, m0, lane);
    flush16<T, D>(sS, m0, dpg, row0 + m0, L, lane, false);

    // phi(q) / den and C_num / den as the B operands of the two D x D reductions, and the row constants for dz
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float2 ph = Elem<T>::unpack2(pq[kk][r]);
        const float rd = (r & 1) ? rd1 : rd0;
        pq[kk][r] = Elem<T>::pack2(ph.x * rd, ph.y * rd);
      }
    }
    store_a_frags_to_tile<D, KS>(sP, pq, m0, 0, lane);
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      uint32_t* a = reinterpret_cast<uint32_t*>(sC + tile_off<D>(m0 + g, j) + t * 4);
      uint32_t* b = reinterpret_cast<uint32_t*>(sC + tile_off<D>(m0 + g + 8, j) + t * 4);
      const float2 av = Elem<T>::unpack2(*a), bv = Elem<T>::unpack2(*b);
      *a = Elem<T>::pack2(av.x * rd0, av.y * rd0);
      *b = Elem<T>::pack2(bv.x * rd1, bv.y * rd1);
    }
    if (t == 0) {
      s_rowc[m0 + g] = dden0 * d0;
      s_rowc[m0 + g + 8] = dden1 * d1;
    }
    __syncthreads();
    gemm_atrans_b_kn<T, D, D / 8, KS>(gacc, sdY_a, m0, sP_a, lane);   // G[n][i]  += sum_m dY[m][n] (phi_q/den)[m][i]
    gemm_atrans_b_kn<T, D, D / 8, KS>(g2acc, sdY_a, m0, sC_a, lane);  // G2[n][d] += sum_m dY[m][n] (C_num/den)[m][d]
    if (tid < D) {
      float s = 0.f;
      const int chunk = tid >> 3, e = tid & 7;
      for (int m = 0; m < D; ++m) {
        const T* a = reinterpret_cast<const T*>(sP + tile_off<D>(m, chunk)) + e;
        s += s_rowc[m] * Elem<T>::to_f(*a);
      }
      vec_acc += s;
    } else {
      const int n = tid - D;
      float s = 0.f;
      const int chunk = n >> 3, e = n & 7;
      for (int m = 0; m < D; ++m) {
        const T* a = reinterpret_cast<const T*>(sdY + tile_off<D>(m, chunk)) + e;
        s += Elem<T>::to_f(*a);
      }
      vec_acc += s;
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  float* out = p.g_partial + (static_cast<size_t>(bh) * p.nch + ch) * (2 * D * D + 2 * D);
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int r0 = m0 + g, c = 8 * j + 2 * t;
    *reinterpret_cast<float2*>(out + r0 * D + c) = make_float2(gacc[j][0], gacc[j][1]);
    *reinterpret_cast<float2*>(out + (r0 + 8) * D + c) = make_float2(gacc[j][2], gacc[j][3]);
    *reinterpret_cast<float2*>(out + D * D + 2 * D + r0 * D + c) = make_float2(g2acc[j][0], g2acc[j][1]);
    *reinterpret_cast<float2*>(out + D * D + 2 * D + (r0 + 8) * D + c) = make_float2(g2acc[j][2], g2acc[j][3]);
  }
  out[D * D + tid] = vec_acc;  // [0,D): dz, [D,2D): db
}

template <typename T, int D>
static int unsel_rows_typed(const sla_shape* s, const UnselBwdParams& p, cudaStream_t st) {
  auto kern = linear_bwd_q_unselected_kernel<T, D>;
  const int smem = 6 * D * D * 2 + 2 * D * 4;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<dim3(p.nch, s->B * s->H), D / 16 * 32, smem, st>>>(p);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

int run_linear_bwd_unselected_rows(const sla_shape* s, const UnselBwdParams& p, cudaStream_t st) {
  if (s->dtype == SLA_BF16)
    return s->D == 64 ? unsel_rows_typed<__nv_bfloat16, 64>(s, p, st) : unsel_rows_typed<__nv_bfloat16, 128>(s, p, st);
  return s->D == 64 ? unsel_rows_typed<__half, 64>(s, p, st) : unsel_rows_typed<__half, 128>(s, p, st);
}

// dx = phi'(x) dphi row by row, in place over dphi, from phi(x) alone: softmax dx = phi (dphi - sum phi dphi),
// relu dx = dphi [phi > 0], elu + 1 dx = dphi (phi > 1 ? 1 : phi). One warp per row.
template <typename T, int D, int FEAT>
__global__ void __launch_bounds__(256) feature_map_bwd_kernel(const T* __restrict__ phi, T* __restrict__ d,
                                                              long long rows) {
  constexpr int EPL = D / 32;
  const long long r = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  float ph[EPL], dv[EPL];
  const T* ps = phi + r * D + lane * EPL;
  T* ds = d + r * D + lane * EPL;
#pragma unroll
  for (int e = 0; e < EPL; e += 2) {
    const float2 a = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(ps + e));
    const float2 b = Elem<T>::unpack2(*reinterpret_cast<const uint32_t*>(ds + e));
    ph[e] = a.x; ph[e + 1] = a.y; dv[e] = b.x; dv[e + 1] = b.y;
  }
  if (FEAT == SLA_PHI_SOFTMAX) {
    float sm = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) sm += ph[e] * dv[e];
    sm = warp_sum(sm);
#pragma unroll
    for (int e = 0; e < EPL; ++e) dv[e] = ph[e] * (dv[e] - sm);
  } else if (FEAT == SLA_PHI_RELU) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) dv[e] = ph[e] > 0.f ? dv[e] : 0.f;
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) dv[e] = ph[e] > 1.f ? dv[e] : dv[e] * ph[e];
  }
#pragma unroll
  for (int e = 0; e < EPL; e += 2) *reinterpret_cast<uint32_t*>(ds + e) = Elem<T>::pack2(dv[e], dv[e + 1]);
}

template <typename T, int D>
static int feature_map_bwd_typed(const sla_shape* s, const T* phi, T* d, cudaStream_t st) {
  const long long rows = static_cast<long long>(s->B) * s->H * s->L;
  const unsigned grid = static_cast<unsigned>((rows + 7) / 8);
  switch (s->feature_map) {
    case SLA_PHI_SOFTMAX: feature_map_bwd_kernel<T, D, SLA_PHI_SOFTMAX><<<grid, 256, 0, st>>>(phi, d, rows); break;
    case SLA_PHI_RELU: feature_map_bwd_kernel<T, D, SLA_PHI_RELU><<<grid, 256, 0, st>>>(phi, d, rows); break;
    default: feature_map_bwd_kernel<T, D, SLA_PHI_ELU><<<grid, 256, 0, st>>>(phi, d, rows); break;
  }
  SLA_LAUNCH_OK();
  return SLA_OK;
}

int run_feature_map_bwd(const sla_shape* s, const void* phi, void* d, cudaStream_t st) {
  if (s->dtype == SLA_BF16) {
    using T = __nv_bfloat16;
    return s->D == 64 ? feature_map_bwd_typed<T, 64>(s, (const T*)phi, (T*)d, st)
                      : feature_map_bwd_typed<T, 128>(s, (const T*)phi, (T*)d, st);
  }
  using T = __half;
  return s->D == 64 ? feature_map_bwd_typed<T, 64>(s, (const T*)phi, (T*)d, st)
                    : feature_map_bwd_typed<T, 128>(s, (const T*)phi, (T*)d, st);
}

}  // namespace sla
