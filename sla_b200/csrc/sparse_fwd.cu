// Block-sparse FlashAttention-style forward on warp-level MMA (mma.sync m16n8k16), with the linear
// branch read-out and proj_l fused into the epilogue. This is the legacy-tensor-path variant
// (SLA_FLAG_LEGACY_MMA); the tcgen05 variant lives in sparse_fwd_tc.cu.
//
// One CTA owns one query block (BM rows, one warp per 16 rows). It walks the block's LUT row,
// streaming the selected 64-row K and V tiles through a two-stage cp.async ring, and keeps the
// online-softmax state in registers, as sparse_linear_attention/kernel.py:21-82 does.
// Epilogue (core.py:90-100): phi(q) from the resident Q fragments, phi(q)H / (1e-5 + phi(q).z),
// proj_l in 16-bit with fp32 accumulation, o = o_s + proj, with the reference's rounding points.
#include "common.cuh"
#include "kernels.h"

namespace sla {

__device__ inline float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

template <typename T, int D, int BM, int FEAT, bool LIN>
__global__ void __launch_bounds__(BM / 16 * 32) sparse_fwd_mma_kernel(FwdParams p) {
  constexpr int NT = BM / 16 * 32;   // threads
  constexpr int KS = D / 16;         // k-steps over the head dimension
  constexpr int TILE_KV = 64 * D * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;                      // [BM][D]
  unsigned char* sK = sQ + BM * D * 2;           // [2][64][D]
  unsigned char* sV = sK + 2 * TILE_KV;          // [2][64][D]
  __shared__ float s_z[LIN ? D : 1];
  __shared__ float s_bias[LIN ? D : 1];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int ib = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  const size_t head_off = static_cast<size_t>(bh) * L * D;
  const T* qg = static_cast<const T*>(p.q) + head_off;
  const T* kg = static_cast<const T*>(p.k) + head_off;
  const T* vg = static_cast<const T*>(p.v) + head_off;
  const int32_t* lut = p.lut + (static_cast<size_t>(bh) * p.mb + ib) * p.topk;
  const int q_row0 = ib * BM;
  const int m0 = warp * 16;

  const uint32_t sQ_a = smem_u32(sQ), sK_a = smem_u32(sK), sV_a = smem_u32(sV);

  load_tile_async<D, BM>(sQ_a, qg, q_row0, L, tid, NT);
  int idx_n = lut[0];
  load_tile_async<D, 64>(sK_a, kg, idx_n * 64, L, tid, NT);
  load_tile_async<D, 64>(sV_a, vg, idx_n * 64, L, tid, NT);
  cp_async_commit();

  uint32_t qf[KS][4];
  float o_acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o_acc[j][0] = o_acc[j][1] = o_acc[j][2] = o_acc[j][3] = 0.f;
  float m_0 = -INFINITY, m_1 = -INFINITY, l_0 = 0.f, l_1 = 0.f;
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

    const int valid = L - idx_n * 64;  // keys of this block that exist (kernel.py:57)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float x = s[j][c] * sc;
        if (valid < 64 && (8 * j + 2 * t + (c & 1)) >= valid) x = -INFINITY;  // kernel.py:61-62
        s[j][c] = x;
      }
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = quad_max(mx0);
    mx1 = quad_max(mx1);
    const float mn0 = fmaxf(m_0, mx0), mn1 = fmaxf(m_1, mx1);
    const float al0 = fast_exp2(m_0 - mn0), al1 = fast_exp2(m_1 - mn1);
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      s[j][0] = fast_exp2(s[j][0] - mn0);
      s[j][1] = fast_exp2(s[j][1] - mn0);
      s[j][2] = fast_exp2(s[j][2] - mn1);
      s[j][3] = fast_exp2(s[j][3] - mn1);
      rs0 += s[j][0] + s[j][1];
      rs1 += s[j][2] + s[j][3];
    }
    l_0 = l_0 * al0 + rs0;  // per-thread partial of the row sum; alpha is uniform over the quad
    l_1 = l_1 * al1 + rs1;
    m_0 = mn0;
    m_1 = mn1;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      o_acc[j][0] *= al0;
      o_acc[j][1] *= al0;
      o_acc[j][2] *= al1;
      o_acc[j][3] *= al1;
    }
    uint32_t pf[4][4];
    acc_to_a_frags<T, 4>(pf, s);  // P rounded to T before P.V (kernel.py:71)
    gemm_b_kn<T, D, D / 8, 4>(o_acc, pf, sV_a + stage * TILE_KV, 0, 0, lane);
    __syncthreads();
    idx_n = next_n;
  }

  // ---- epilogue of the sparse branch ----
  l_0 = quad_sum(l_0);
  l_1 = quad_sum(l_1);
  const float inv0 = 1.f / l_0, inv1 = 1.f / l_1;
  const int r0 = q_row0 + m0 + g, r1 = r0 + 8;
  if (t == 0) {
    float* lse = p.lse + static_cast<size_t>(bh) * L;
    if (r0 < L) lse[r0] = m_0 + log2f(l_0);  // kernel.py:81
    if (r1 < L) lse[r1] = m_1 + log2f(l_1);
  }
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    o_acc[j][0] *= inv0;
    o_acc[j][1] *= inv0;
    o_acc[j][2] *= inv1;
    o_acc[j][3] *= inv1;
  }
  // The Q tile rows of this warp are only ever read by this warp: reuse them as a staging area
  // so that global stores are 16 bytes wide and row-contiguous.
  auto flush_rows = [&](void* gbase) {
    __syncwarp();
    constexpr int CH = D / 8;
    char* gp = reinterpret_cast<char*>(gbase);
    for (int i = lane; i < 16 * CH; i += 32) {
      int r = i / CH, c = i % CH;
      int gr = q_row0 + m0 + r;
      if (gr < L) {
        uint4 v4 = *reinterpret_cast<const uint4*>(sQ + tile_off<D>(m0 + r, c));
        *reinterpret_cast<uint4*>(gp + (static_cast<size_t>(gr) * D + c * 8) * 2) = v4;
      }
    }
    __syncwarp();
  };

  if constexpr (!LIN) {
    store_acc_to_tile<T, D, D / 8>(sQ, o_acc, m0, lane);
    flush_rows(static_cast<T*>(p.o) + head_off);
    return;
  } else {
    if (p.o_s != nullptr) {
      store_acc_to_tile<T, D, D / 8>(sQ, o_acc, m0, lane);
      flush_rows(static_cast<T*>(p.o_s) + head_off);
    }
    // o_s rounded to T, kept packed (core.py:100 adds two T tensors)
    uint32_t os_pk[D / 8][2];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      os_pk[j][0] = Elem<T>::pack2(o_acc[j][0], o_acc[j][1]);
      os_pk[j][1] = Elem<T>::pack2(o_acc[j][2], o_acc[j][3]);
    }
    // stage H (D x D, [i][j]) over the K ring and W ([n][k], 16-bit) over the V ring
    const T* hs = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);
    const T* wb = static_cast<const T*>(p.wbits);
    static_assert(2 * TILE_KV >= D * D * 2, "state tile must fit in the K/V ring");
    load_tile_async<D, D>(sK_a, hs, 0, D, tid, NT);
    load_tile_async<D, D>(sV_a, wb, 0, D, tid, NT);
    cp_async_commit();
    for (int i = tid; i < D; i += NT) {
      s_z[i] = Elem<T>::to_f(hs[D * D + i]);
      s_bias[i] = Elem<T>::to_f(wb[D * D + i]);
    }
    uint32_t pq[KS][4];
    feature_map_frags<T, KS, FEAT>(pq, qf);
    cp_async_wait<0>();
    __syncthreads();

    float num[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) num[j][0] = num[j][1] = num[j][2] = num[j][3] = 0.f;
    gemm_b_kn<T, D, D / 8, KS>(num, pq, sK_a, 0, 0, lane);  // phi(q) @ kvsum
    // den = 1e-5 + sum_d round(phi(q)*ksum) (core.py:95), each step rounded to T
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
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      num[j][0] = round_to<T>(num[j][0]) / d0;
      num[j][1] = round_to<T>(num[j][1]) / d0;
      num[j][2] = round_to<T>(num[j][2]) / d1;
      num[j][3] = round_to<T>(num[j][3]) / d1;
    }
    uint32_t ol[KS][4];
    acc_to_a_frags<T, KS>(ol, num);  // o_l in T
#pragma unroll
    for (int j = 0; j < D / 8; ++j) num[j][0] = num[j][1] = num[j][2] = num[j][3] = 0.f;
    gemm_b_nk<T, D, D / 8, KS>(num, ol, sV_a, 0, 0, lane);  // o_l @ W^T (core.py:99)
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      int col = 8 * j + 2 * t;
      float2 a = Elem<T>::unpack2(os_pk[j][0]), b = Elem<T>::unpack2(os_pk[j][1]);
      num[j][0] = a.x + round_to<T>(num[j][0] + s_bias[col]);
      num[j][1] = a.y + round_to<T>(num[j][1] + s_bias[col + 1]);
      num[j][2] = b.x + round_to<T>(num[j][2] + s_bias[col]);
      num[j][3] = b.y + round_to<T>(num[j][3] + s_bias[col + 1]);
    }
    store_acc_to_tile<T, D, D / 8>(sQ, num, m0, lane);
    flush_rows(static_cast<T*>(p.o) + head_off);
  }
}

// 16-bit copy of proj_l's weight and bias (what autocast feeds the GEMM, core.py:98-99):
// out[0 .. D*D) = W, out[D*D .. D*D + D) = bias (zeros when bias == nullptr).
template <typename T>
__global__ void convert_proj_kernel(const float* __restrict__ w, const float* __restrict__ bias,
                                    T* __restrict__ out, int dd, int d) {
  pdl_wait();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < dd) out[i] = Elem<T>::from_f(w[i]);
  else if (i < dd + d) out[i] = Elem<T>::from_f(bias ? bias[i - dd] : 0.f);
}

int convert_proj(const sla_shape* s, const float* w, const float* bias, void* out, cudaStream_t st) {
  int dd = s->D * s->D, n = dd + s->D;
  if (s->dtype == SLA_BF16)
    SLA_CUDA_OK(launch_pdl(convert_proj_kernel<__nv_bfloat16>, dim3(ceil_div(n, 256)), dim3(256), 0, st, w, bias,
                           static_cast<__nv_bfloat16*>(out), dd, s->D));
  else
    SLA_CUDA_OK(launch_pdl(convert_proj_kernel<__half>, dim3(ceil_div(n, 256)), dim3(256), 0, st, w, bias,
                           static_cast<__half*>(out), dd, s->D));
  SLA_LAUNCH_OK();
  return SLA_OK;
}

template <typename T, int D, int BM, int FEAT, bool LIN>
static int launch_fwd(const FwdParams& p, int bh, cudaStream_t st) {
  auto kern = sparse_fwd_mma_kernel<T, D, BM, FEAT, LIN>;
  int smem = BM * D * 2 + 4 * 64 * D * 2;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<dim3(p.mb, bh), BM / 16 * 32, smem, st>>>(p);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

template <typename T, int D, int BM>
static int dispatch_feat(const FwdParams& p, int bh, int feat, bool lin, cudaStream_t st) {
  if (!lin) return launch_fwd<T, D, BM, SLA_PHI_SOFTMAX, false>(p, bh, st);
  switch (feat) {
    case SLA_PHI_SOFTMAX: return launch_fwd<T, D, BM, SLA_PHI_SOFTMAX, true>(p, bh, st);
    case SLA_PHI_RELU: return launch_fwd<T, D, BM, SLA_PHI_RELU, true>(p, bh, st);
    default: return launch_fwd<T, D, BM, SLA_PHI_ELU, true>(p, bh, st);
  }
}

template <typename T>
static int dispatch_shape(const sla_shape* s, const FwdParams& p, bool lin, cudaStream_t st) {
  int bh = s->B * s->H;
  if (s->D == 64) {
    if (s->BLKQ == 64) return dispatch_feat<T, 64, 64>(p, bh, s->feature_map, lin, st);
    return dispatch_feat<T, 64, 128>(p, bh, s->feature_map, lin, st);
  }
  if (s->BLKQ == 64) return dispatch_feat<T, 128, 64>(p, bh, s->feature_map, lin, st);
  return dispatch_feat<T, 128, 128>(p, bh, s->feature_map, lin, st);
}

int run_sparse_fwd_mma(const sla_shape* s, const FwdParams& p, bool lin, cudaStream_t st) {
  if (s->dtype == SLA_BF16) return dispatch_shape<__nv_bfloat16>(s, p, lin, st);
  return dispatch_shape<__half>(s, p, lin, st);
}

}  // namespace sla
