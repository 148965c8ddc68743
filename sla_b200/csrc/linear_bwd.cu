// Backward of the linear branch and of proj_l (the reference leaves this to PyTorch autograd of
// sparse_linear_attention/core.py:90-100). With dY the gradient of the module output, o_l = phi_q H / den,
// den = 1e-5 + phi_q . z and proj = o_l W^T + b:
//   do_l = dY W,  t = do_l H^T = dY (W H^T) =: dY M            (M^T = H W^T is kept by the forward)
//   dphi_q = t / den + dden z,   dden = -(do_l . o_l) / den = -(phi_q . t) / den^2
//   dq_lin = phi'(q) dphi_q
//   G = sum_l dY_l^T (phi_q,l / den_l)                          (one D x D reduction per head)
//   dH = G^T W,  dW = sum_heads G H,  dz = sum_l dden_l phi_q,l,  db = sum_l dY_l
//   dphi_k = v dH^T + dz,  dk_lin = phi'(k) dphi_k,  dv_lin = phi_k dH
// Folding W into M and using phi_q . t for dden leaves two GEMMs per row tile in pass A (t and G)
// and two in pass B. Pass A writes dq_lin and per-chunk partials of G, dz, db; small per-head kernels
// turn them into dH, dz and the head's share of dW, db; pass B writes dk_lin, dv_lin.
#include "common.cuh"
#include "kernels.h"

namespace sla {

// ---------------------------------------------------------------------------------------------
// Pass A: D query rows per tile, one warp per 16 rows.
// ---------------------------------------------------------------------------------------------
template <typename T, int D, int FEAT>
__global__ void __launch_bounds__(D / 16 * 32) linear_bwd_q_kernel(LinBwdParams p) {
  constexpr int NW = D / 16, NT = NW * 32, KS = D / 16;
  constexpr int TILE = D * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sM = smem;         // H W^T = M^T, stored [i][n]
  // two {Q, dY} buffers: the next row tile is copied in while this one is worked on
  float* s_z = reinterpret_cast<float*>(smem + 5 * TILE);  // [D]
  float* s_rowc = s_z + D;                                 // [D] dden*den per row of the tile

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ch = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* qg = static_cast<const T*>(p.q) + head_off;
  const T* dyg = static_cast<const T*>(p.d_o) + head_off;
  T* dqg = static_cast<T*>(p.dq) + head_off;
  const T* hs = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);
  const T* mg = hs + D * D + D;
  const uint32_t sM_a = smem_u32(sM);
  const int m0 = warp * 16;

  load_tile_async<D, D>(sM_a, mg, 0, D, tid, NT);
  cp_async_commit();
  for (int i = tid; i < D; i += NT) s_z[i] = Elem<T>::to_f(hs[D * D + i]);

  float gacc[D / 8][4];  // rows [16*warp, +16) of G[n][i]
#pragma unroll
  for (int j = 0; j < D / 8; ++j) gacc[j][0] = gacc[j][1] = gacc[j][2] = gacc[j][3] = 0.f;
  float vec_acc = 0.f;   // thread tid < D: dz[tid]; tid >= D: db[tid - D]

  const int row_begin = ch * p.rows, row_end = min(L, row_begin + p.rows);
  auto prefetch = [&](int row0, int buf) {
    const uint32_t a = smem_u32(smem + (1 + 2 * buf) * TILE);
    load_tile_async<D, D>(a, qg, row0, L, tid, NT);
    load_tile_async<D, D>(a + TILE, dyg, row0, L, tid, NT);
    cp_async_commit();
  };
  if (row_begin < row_end) prefetch(row_begin, 0);
  int buf = 0;
  for (int row0 = row_begin; row0 < row_end; row0 += D, buf ^= 1) {
    unsigned char* sQ = smem + (1 + 2 * buf) * TILE;   // Q rows, then dq staging, then phi(q)/den
    unsigned char* sdY = sQ + TILE;
    const uint32_t sQ_a = smem_u32(sQ), sdY_a = smem_u32(sdY);
    if (row0 + D < row_end) {          // the other buffer was released by the barrier that ended the last tile
      prefetch(row0 + D, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    uint32_t pq[KS][4];
    {
      uint32_t qf[KS][4];
      load_a_frags<D, KS>(qf, sQ_a, m0, 0, lane);
      feature_map_frags<T, KS, FEAT>(pq, qf);
    }
    // den = 1e-5 + sum_d round(phi(q)*ksum) (core.py:95), each step rounded to T as in the forward
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
    d0 = round_to<T>(1e-5f + round_to<T>(quad_sum(d0)));
    d1 = round_to<T>(1e-5f + round_to<T>(quad_sum(d1)));
    const float rd0 = 1.f / d0, rd1 = 1.f / d1;

    float acc[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    gemm_at_b_nk<T, D, D / 8, KS>(acc, sdY_a, m0, sM_a, lane);  // t[m][i] = sum_n dY[m][n] HW[i][n]
    // s = phi_q . t per row
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      float2 p0 = Elem<T>::unpack2(pq[kk][0]), p1 = Elem<T>::unpack2(pq[kk][1]);
      float2 p2 = Elem<T>::unpack2(pq[kk][2]), p3 = Elem<T>::unpack2(pq[kk][3]);
      s0 += acc[2 * kk][0] * p0.x + acc[2 * kk][1] * p0.y + acc[2 * kk + 1][0] * p2.x + acc[2 * kk + 1][1] * p2.y;
      s1 += acc[2 * kk][2] * p1.x + acc[2 * kk][3] * p1.y + acc[2 * kk + 1][2] * p3.x + acc[2 * kk + 1][3] * p3.y;
    }
    const float dden0 = -quad_sum(s0) * rd0 * rd0, dden1 = -quad_sum(s1) * rd1 * rd1;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      int col = 8 * j + 2 * t;
      acc[j][0] = acc[j][0] * rd0 + dden0 * s_z[col];
      acc[j][1] = acc[j][1] * rd0 + dden0 * s_z[col + 1];
      acc[j][2] = acc[j][2] * rd1 + dden1 * s_z[col];
      acc[j][3] = acc[j][3] * rd1 + dden1 * s_z[col + 1];
    }
    feature_map_bwd_frags<T, KS, FEAT>(acc, pq);
    // dq_lin: stage in this warp's rows of the Q tile (its fragments are no longer needed) and flush
    store_acc_to_tile<T, D, D / 8>(sQ, acc, m0, lane);
    flush16<T, D>(sQ, m0, dqg, row0 + m0, L, lane, p.accumulate != 0);
    // phi(q)/den for the G reduction, and the row constants for dz
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float2 ph = Elem<T>::unpack2(pq[kk][r]);
        float rd = (r & 1) ? rd1 : rd0;
        pq[kk][r] = Elem<T>::pack2(ph.x * rd, ph.y * rd);
      }
    }
    store_a_frags_to_tile<D, KS>(sQ, pq, m0, 0, lane);
    if (t == 0) {
      s_rowc[m0 + g] = dden0 * d0;
      s_rowc[m0 + g + 8] = dden1 * d1;
    }
    __syncthreads();
    // G[n][i] += sum_m dY[m][n] * (phi_q/den)[m][i]
    gemm_atrans_b_kn<T, D, D / 8, KS>(gacc, sdY_a, m0, sQ_a, lane);
    if (tid < D) {
      float s = 0.f;
      int chunk = tid >> 3, e = tid & 7;
      for (int m = 0; m < D; ++m) {
        const T* a = reinterpret_cast<const T*>(sQ + tile_off<D>(m, chunk)) + e;
        s += s_rowc[m] * Elem<T>::to_f(*a);
      }
      vec_acc += s;
    } else {
      int n = tid - D;
      float s = 0.f;
      int chunk = n >> 3, e = n & 7;
      for (int m = 0; m < D; ++m) {
        const T* a = reinterpret_cast<const T*>(sdY + tile_off<D>(m, chunk)) + e;
        s += Elem<T>::to_f(*a);
      }
      vec_acc += s;
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  float* out = p.g_partial + (static_cast<size_t>(bh) * p.nch + ch) * (D * D + 2 * D);
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    int r0 = m0 + g, c = 8 * j + 2 * t;
    *reinterpret_cast<float2*>(out + r0 * D + c) = make_float2(gacc[j][0], gacc[j][1]);
    *reinterpret_cast<float2*>(out + (r0 + 8) * D + c) = make_float2(gacc[j][2], gacc[j][3]);
  }
  out[D * D + tid] = vec_acc;  // [0,D): dz, [D,2D): db
}

// ---------------------------------------------------------------------------------------------
// Per-head reductions. (1) sum the chunk partials; (2) G -> dH (T), and the head's dW; dz, db copied.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) linear_bwd_gsum_kernel(const float* __restrict__ part,
                                                              float* __restrict__ gsum, int nch, int n) {
  pdl_entry();
  const int bh = blockIdx.y;
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= n) return;
  const float* p = part + static_cast<size_t>(bh) * nch * n + i;
  float s = 0.f;
#pragma unroll 8
  for (int c = 0; c < nch; ++c) s += p[static_cast<size_t>(c) * n];   // loads batched, sum in order
  gsum[static_cast<size_t>(bh) * n + i] = s;
}

// One CTA per head, one warp per 16 output rows, both products on the tensor cores with G rounded to T:
//   dH[i][j] = sum_n G[n][i] W[n][j]      dW_head[n][k] = sum_i G[n][i] H[i][k]
template <typename T, int D>
__global__ void __launch_bounds__(D / 16 * 32) linear_bwd_reduce_kernel(LinBwdParams p) {
  constexpr int NT = D / 16 * 32, KS = D / 16, dd = D * D, n = dd + 2 * D;
  extern __shared__ __align__(128) unsigned char smem[];
  pdl_entry();
  unsigned char* sG = smem;              // [n][i] T
  unsigned char* sW = sG + dd * 2;       // [n][j] T
  unsigned char* sH = sW + dd * 2;       // [i][k] T
  const int bh = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int stride = p.g_stride ? p.g_stride : n;     // floats per head record: {G, dz, db} or {G, dz, db, G2}
  const float* G = p.g_sum + static_cast<size_t>(bh) * stride;
  const T* hs = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * dd + D);
  T* dh = static_cast<T*>(p.dh) + static_cast<size_t>(bh) * dd;
  float* dwp = p.dw_part + static_cast<size_t>(bh) * (dd + D);
  const uint32_t sG_a = smem_u32(sG), sW_a = smem_u32(sW), sH_a = smem_u32(sH);
  load_tile_async<D, D>(sW_a, p.wbits, 0, D, tid, NT);
  load_tile_async<D, D>(sH_a, hs, 0, D, tid, NT);
  cp_async_commit();
  for (int c = tid; c < dd / 8; c += NT) {   // 8 consecutive fp32 -> one 16-byte chunk of T
    const int r = c / (D / 8), ch = c % (D / 8);
    const float4 a = *reinterpret_cast<const float4*>(G + r * D + ch * 8);
    const float4 b = *reinterpret_cast<const float4*>(G + r * D + ch * 8 + 4);
    uint4 v;
    v.x = Elem<T>::pack2(a.x, a.y); v.y = Elem<T>::pack2(a.z, a.w);
    v.z = Elem<T>::pack2(b.x, b.y); v.w = Elem<T>::pack2(b.z, b.w);
    *reinterpret_cast<uint4*>(sG + tile_off<D>(r, ch)) = v;
  }
  for (int i = tid; i < 2 * D; i += NT) {
    if (i < D) p.dz[static_cast<size_t>(bh) * D + i] = G[dd + i];
    else dwp[dd + i - D] = G[dd + i];
  }
  cp_async_wait<0>();
  __syncthreads();
  const int m0 = warp * 16;
  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  gemm_atrans_b_kn<T, D, D / 8, KS>(acc, sG_a, m0, sW_a, lane);   // rows i of dH
  float acc2[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc2[j][0] = acc2[j][1] = acc2[j][2] = acc2[j][3] = 0.f;
  {
    uint32_t a[KS][4];
    load_a_frags<D, KS>(a, sG_a, m0, 0, lane);
    gemm_b_kn<T, D, D / 8, KS>(acc2, a, sH_a, 0, 0, lane);         // rows n of dW_head
  }
  if (p.has_g2) {   // "unselected" scope: dW_head = G H - G2
    const float* G2 = G + dd + 2 * D;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int r0 = m0 + g, c = 8 * j + 2 * t;
      const float2 a = *reinterpret_cast<const float2*>(G2 + r0 * D + c);
      const float2 b = *reinterpret_cast<const float2*>(G2 + (r0 + 8) * D + c);
      acc2[j][0] -= a.x; acc2[j][1] -= a.y; acc2[j][2] -= b.x; acc2[j][3] -= b.y;
    }
  }
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int r0 = m0 + g, c = 8 * j + 2 * t;
    *reinterpret_cast<float2*>(dwp + r0 * D + c) = make_float2(acc2[j][0], acc2[j][1]);
    *reinterpret_cast<float2*>(dwp + (r0 + 8) * D + c) = make_float2(acc2[j][2], acc2[j][3]);
  }
  __syncthreads();   // all warps are done reading W: reuse it as the staging tile for dH
  store_acc_to_tile<T, D, D / 8>(sW, acc, m0, lane);
  flush16<T, D>(sW, m0, dh, m0, D, lane, false);
}

__global__ void dw_final_kernel(const float* __restrict__ dw_part, float* __restrict__ dw,
                                float* __restrict__ dbias, int bh, int dd, int d) {
  pdl_entry();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= dd + d) return;
  float s = 0.f;
  for (int h = 0; h < bh; ++h) s += dw_part[static_cast<size_t>(h) * (dd + d) + i];
  if (i < dd) dw[i] = s; else dbias[i - dd] = s;
}

// ---------------------------------------------------------------------------------------------
// Pass B: dk_lin, dv_lin. A CTA keeps the head's dH in shared memory and streams its chunk of key rows
// through two {K, V} buffers of 64 rows (the next tile is copied in while this one is worked on).
// ---------------------------------------------------------------------------------------------
template <typename T, int D, int FEAT>
__global__ void __launch_bounds__(128) linear_bwd_kv_kernel(LinBwdParams p) {
  constexpr int NT = 128, KS = D / 16;
  constexpr int T64 = 64 * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sdH = smem;                  // [D][D]
  float* s_dz = reinterpret_cast<float*>(smem + D * D * 2 + 4 * T64);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = lane & 3;
  const int ch = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* kg = static_cast<const T*>(p.k) + head_off;
  const T* vg = static_cast<const T*>(p.v) + head_off;
  const T* dh = static_cast<const T*>(p.dh) + static_cast<size_t>(bh) * D * D;
  const uint32_t sdH_a = smem_u32(sdH);
  const int m0 = warp * 16;
  const int row_begin = ch * p.rows, row_end = min(L, row_begin + p.rows);
  auto prefetch = [&](int row0, int buf) {
    const uint32_t a = smem_u32(smem + D * D * 2 + 2 * buf * T64);
    load_tile_async<D, 64>(a, kg, row0, L, tid, NT);
    load_tile_async<D, 64>(a + T64, vg, row0, L, tid, NT);
    cp_async_commit();
  };
  load_tile_async<D, D>(sdH_a, dh, 0, D, tid, NT);
  if (row_begin < row_end) prefetch(row_begin, 0);
  else cp_async_commit();
  for (int i = tid; i < D; i += NT) s_dz[i] = p.dz[static_cast<size_t>(bh) * D + i];

  int buf = 0;
  for (int row0 = row_begin; row0 < row_end; row0 += 64, buf ^= 1) {
    unsigned char* sK = smem + D * D * 2 + 2 * buf * T64;
    unsigned char* sV = sK + T64;
    const uint32_t sK_a = smem_u32(sK), sV_a = smem_u32(sV);
    cp_async_wait<0>();
    __syncthreads();   // this tile has landed, and every warp is done with the other buffer
    if (row0 + 64 < row_end) prefetch(row0 + 64, buf ^ 1);

    uint32_t pk[KS][4];
    {
      uint32_t kf[KS][4];
      load_a_frags<D, KS>(kf, sK_a, m0, 0, lane);
      feature_map_frags<T, KS, FEAT>(pk, kf);
    }
    float acc[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      int col = 8 * j + 2 * t;
      acc[j][0] = s_dz[col]; acc[j][1] = s_dz[col + 1];
      acc[j][2] = s_dz[col]; acc[j][3] = s_dz[col + 1];
    }
    gemm_at_b_nk<T, D, D / 8, KS>(acc, sV_a, m0, sdH_a, lane);  // dphi_k = v dH^T + dz
    feature_map_bwd_frags<T, KS, FEAT>(acc, pk);
    // each warp stages and flushes its own 16 rows
    store_acc_to_tile<T, D, D / 8>(sK, acc, m0, lane);
    flush16<T, D>(sK, m0, static_cast<T*>(p.dk) + head_off, row0 + m0, L, lane, p.accumulate != 0);
#pragma unroll
    for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    gemm_b_kn<T, D, D / 8, KS>(acc, pk, sdH_a, 0, 0, lane);  // dv_lin = phi(k) dH
    store_acc_to_tile<T, D, D / 8>(sV, acc, m0, lane);
    flush16<T, D>(sV, m0, static_cast<T*>(p.dv) + head_off, row0 + m0, L, lane, p.accumulate != 0);
  }
  cp_async_wait<0>();
}

// Per-head reductions after a row pass: chunk partials -> head sums -> dH (16-bit), dz, the head's dW and db ->
// dW, db summed over the heads.
template <typename T, int D>
static int reductions_typed(const sla_shape* s, const LinBwdParams& p, cudaStream_t st) {
  const int bh = s->B * s->H, dd = D * D;
  const int n = p.g_stride ? p.g_stride : dd + 2 * D;
  SLA_CUDA_OK(launch_pdl(linear_bwd_gsum_kernel, dim3(ceil_div(n, 256), bh), dim3(256), 0, st,
                         static_cast<const float*>(p.g_partial), p.g_sum, p.nch, n));
  SLA_LAUNCH_OK();
  auto rk = linear_bwd_reduce_kernel<T, D>;
  SLA_CUDA_OK(cudaFuncSetAttribute(rk, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * dd * 2));
  SLA_CUDA_OK(launch_pdl(rk, dim3(bh), dim3(D / 16 * 32), 3 * dd * 2, st, p));
  SLA_LAUNCH_OK();
  SLA_CUDA_OK(launch_pdl(dw_final_kernel, dim3(ceil_div(dd + D, 256)), dim3(256), 0, st,
                         static_cast<const float*>(p.dw_part), p.dw, p.dbias, bh, dd, D));
  SLA_LAUNCH_OK();
  return SLA_OK;
}

int run_linear_bwd_reductions(const sla_shape* s, const LinBwdParams& p, cudaStream_t st) {
  if (s->dtype == SLA_BF16)
    return s->D == 64 ? reductions_typed<__nv_bfloat16, 64>(s, p, st) : reductions_typed<__nv_bfloat16, 128>(s, p, st);
  return s->D == 64 ? reductions_typed<__half, 64>(s, p, st) : reductions_typed<__half, 128>(s, p, st);
}

template <typename T, int D, int FEAT>
static int launch_lin_bwd(const sla_shape* s, const LinBwdParams& p, cudaStream_t st) {
  const int bh = s->B * s->H, dd = D * D;
  int rc_a = p.tc_pass_a ? run_linear_bwd_q_tc(s, p, st) : SLA_ERR_UNSUPPORTED;
  if (rc_a != SLA_OK && rc_a != SLA_ERR_UNSUPPORTED) return rc_a;
  if (rc_a != SLA_OK) {
    auto kern = linear_bwd_q_kernel<T, D, FEAT>;
    int smem = 5 * dd * 2 + 2 * D * 4;
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<dim3(p.nch, bh), D / 16 * 32, smem, st>>>(p);
    SLA_LAUNCH_OK();
  }
  {
    int rc = reductions_typed<T, D>(s, p, st);
    if (rc != SLA_OK) return rc;
  }
  if (!p.skip_kv) {
    auto kern = linear_bwd_kv_kernel<T, D, FEAT>;
    int smem = dd * 2 + 4 * 64 * D * 2 + D * 4;
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kern<<<dim3(p.nch, bh), 128, smem, st>>>(p);
    SLA_LAUNCH_OK();
  }
  return SLA_OK;
}

template <typename T, int D>
static int dispatch_lin_feat(const sla_shape* s, const LinBwdParams& p, cudaStream_t st) {
  switch (s->feature_map) {
    case SLA_PHI_SOFTMAX: return launch_lin_bwd<T, D, SLA_PHI_SOFTMAX>(s, p, st);
    case SLA_PHI_RELU: return launch_lin_bwd<T, D, SLA_PHI_RELU>(s, p, st);
    default: return launch_lin_bwd<T, D, SLA_PHI_ELU>(s, p, st);
  }
}

int run_linear_bwd(const sla_shape* s, const LinBwdParams& p, cudaStream_t st) {
  if (s->dtype == SLA_BF16) {
    if (s->D == 64) return dispatch_lin_feat<__nv_bfloat16, 64>(s, p, st);
    return dispatch_lin_feat<__nv_bfloat16, 128>(s, p, st);
  }
  if (s->D == 64) return dispatch_lin_feat<__half, 64>(s, p, st);
  return dispatch_lin_feat<__half, 128>(s, p, st);
}

}  // namespace sla
