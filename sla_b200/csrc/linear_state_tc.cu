// Linear-branch state (sparse_linear_attention/core.py:91,93-94) on tcgen05, head dim 128:
// per chunk of rows of one head, H_partial = phi(k)^T v (fp32, D x D) and z_partial = sum_rows phi(k).
// Same chunking, partial buffers and reduction kernel as the mma.sync kernel in linear_state.cu.
//
// Per tile of 32 rows the {K, V} pair is TMA-staged (16 KB, 128-byte swizzle), the row warps turn the K tile into
// phi(k) in place (rounded to the 16-bit type first, core.py:91; rows past the end of the sequence become zero) and
// one thread issues H += phi(K)^T V as two 128 x 128 x 16 MMAs, both operands MN-major (the contraction runs over
// the tile's rows, so a tile may have any multiple of 16 of them). 192 threads: warps 0-3 feature map and column
// sums (eight lanes per row, sixteen rows per pass: a lane owns the same sixteen columns in every row it sees, so z
// accumulates in registers), warp 4 TMA producer, warp 5 MMA issuer. A ring of four tile pairs per CTA (64 KB),
// three CTAs per SM. Tensor memory: H (128 columns).
// All waits are bounded (tc_common.cuh).
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace sla {
namespace tc {

enum : int { kSErrFull = 601, kSErrFree = 602, kSErrX = 603, kSErrG = 604 };
constexpr int kStateTileRows = 32;   // rows per tile
constexpr int kStateStages = 4;      // tile pairs in flight per CTA

struct LinStateParams {
  float* partial;          // [BH][NCH][D*D + D]
  int* err;
  int L, nch, rows;
};

__device__ __forceinline__ float ex2s(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// OR of a predicate over the 128 threads of the row warps (named barrier 1); the result is the same in all of them
__device__ __forceinline__ bool state_rows_any(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.or.pred p, 1, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(out)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return out != 0;
}

template <typename T, int FEAT>
__global__ void __launch_bounds__(192, (kStateStages * kStateTileRows * 512 + 1024 <= 72 * 1024) ? 3 : 2)
linear_state_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       LinStateParams p) {
  constexpr int D = 128;
  constexpr int TR = kStateTileRows, NS = kStateStages;
  static_assert(TR % 32 == 0, "the row warps take 32 rows per step");
  constexpr int SLAB = TR * 128, TILE = 2 * SLAB;        // 64 columns x TR rows of T; a tile is two slabs
  constexpr int STAGE = 2 * TILE;                        // {K, V}
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_H = idesc_f16(FMT, 128, D, 1, 1);   // phi(K)^T (MN-major) x V (MN-major)
  constexpr uint32_t TMEM_COLS = 128;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[3 * NS + 1];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ch = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  pdl_wait();
  const uint32_t raw_a = smem_u32(smem_raw);
  const uint32_t base_a = (raw_a + 1023u) & ~1023u;
  uint8_t* base_p = smem_raw + (base_a - raw_a);
  auto stage_k = [&](int st) { return base_a + st * STAGE; };      // the V tile follows at + TILE
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // per stage: tile pair landed | phi(k) written | the tile's MMAs done (the pair may be overwritten); tile t uses
  // stage t % NS and phase (t / NS) & 1 of its barriers. B_DONE: every MMA of the CTA has completed.
  constexpr int B_FULL = 0, B_X = NS, B_FREE = 2 * NS, B_DONE = 3 * NS;

  const int row_begin = ch * p.rows, row_end = min(L, row_begin + p.rows);
  const int n_tiles = row_end > row_begin ? (row_end - row_begin + TR - 1) / TR : 0;

  if (tid == 0) {
    s_abort = *reinterpret_cast<volatile int*>(p.err) != 0;
    for (int st = 0; st < NS; ++st) {
      mbar_init(BAR(B_FULL + st), 1);
      mbar_init(BAR(B_X + st), 4);
      mbar_init(BAR(B_FREE + st), 1);
    }
    mbar_init(BAR(B_DONE), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 4 && lane == 0) { prefetch_tmap(&tmK); prefetch_tmap(&tmV); }
  if (warp == 5) {
    tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  volatile int* abortp = &s_abort;
  float* out = p.partial + (static_cast<size_t>(bh) * p.nch + ch) * (D * D + D);

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      bool ok = !*abortp;
      int in_flight = -1;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int st = t % NS;
        if (t >= NS && !mbar_wait(BAR(B_FREE + st), (t / NS - 1) & 1, kSErrFree, p.err)) { ok = false; break; }
        if (*abortp) { ok = false; break; }
        const int row0 = row_begin + t * TR;
        const uint32_t sK = stage_k(st), sV = sK + TILE;
        mbar_expect_tx(BAR(B_FULL + st), STAGE);
        for (int c = 0; c < 2; ++c) {
          tma_load_3d(sK + c * SLAB, &tmK, BAR(B_FULL + st), c * 64, row0, bh);
          tma_load_3d(sV + c * SLAB, &tmV, BAR(B_FULL + st), c * 64, row0, bh);
        }
        in_flight = t;
      }
      if (!ok || *abortp) {
        *abortp = 1;
        // the copies still in flight must land before the CTA's shared memory goes away
        for (int t = max(0, in_flight - NS + 1); t <= in_flight; ++t)
          mbar_wait_drain(BAR(B_FULL + t % NS), (t / NS) & 1, p.err);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    bool ok = !*abortp;
    for (int t = 0; ok && t < n_tiles; ++t) {
      const int st = t % NS;
      ok = warp_all(mbar_wait(BAR(B_X + st), (t / NS) & 1, kSErrX, p.err));
      if (!ok) break;
      tc_fence_after();
      const uint32_t k_mn = desc_lo(stage_k(st), SLAB), v_mn = desc_lo(stage_k(st) + TILE, SLAB);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < TR / 16; ++kk) {       // k = tile rows, 16 per step = 2048 bytes of either operand
          const uint32_t ko = (kk * 2048) >> 4;
          mma_ss(tmem, k_mn + ko, v_mn + ko, IDESC_H, (t > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(BAR(B_FREE + st));
      }
      __syncwarp();
    }
    if (ok && n_tiles > 0) {
      if (elect_one()) tc_commit(BAR(B_DONE));
      __syncwarp();
    }
    if (!ok) *abortp = 1;
  } else {
    // ------------------------------ row warps ------------------------------
    const int e8 = tid & 7, prow = tid >> 3;                 // lane's 16-byte chunks e8 and e8 + 8 of rows prow + 16 i
    float zacc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) zacc[i] = 0.f;
    bool ok = !state_rows_any(*abortp != 0);
    for (int t = 0; ok && t < n_tiles; ++t) {
      const int row0 = row_begin + t * TR, st = t % NS;
      const uint32_t sK = stage_k(st);
      ok = !state_rows_any(!mbar_wait(BAR(B_FULL + st), (t / NS) & 1, kSErrFull, p.err));
      if (!ok) break;
      // two rows per lane and step (r and r + 16: same swizzle offset), loaded together, worked on as two
      // independent chains and stored together; maxima and sums as trees
      for (int r = prow; r < TR; r += 32) {
        const uint32_t a0 = sK + r * 128 + ((e8 ^ (r & 7)) << 4);     // chunk e8; chunk e8 + 8 sits SLAB further
        uint32_t w[2][8];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          ld_shared_v4(a0 + j * 2048, w[j][0], w[j][1], w[j][2], w[j][3]);
          ld_shared_v4(a0 + j * 2048 + SLAB, w[j][4], w[j][5], w[j][6], w[j][7]);
        }
        float x[2][16];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float2 f = Elem<T>::unpack2(w[j][i]);
            x[j][2 * i] = f.x; x[j][2 * i + 1] = f.y;
          }
        if (FEAT == SLA_PHI_SOFTMAX) {
          float mx[2], sm[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {      // the maximum on the packed pairs (exact: a maximum does not round)
            const uint32_t m01 = Elem<T>::max2(w[j][0], w[j][1]), m23 = Elem<T>::max2(w[j][2], w[j][3]);
            const uint32_t m45 = Elem<T>::max2(w[j][4], w[j][5]), m67 = Elem<T>::max2(w[j][6], w[j][7]);
            const float2 m = Elem<T>::unpack2(Elem<T>::max2(Elem<T>::max2(m01, m23), Elem<T>::max2(m45, m67)));
            mx[j] = fmaxf(m.x, m.y);
          }
#pragma unroll
          for (int o = 1; o < 8; o <<= 1) {
            const float o0 = __shfl_xor_sync(0xffffffffu, mx[0], o), o1 = __shfl_xor_sync(0xffffffffu, mx[1], o);
            mx[0] = fmaxf(mx[0], o0); mx[1] = fmaxf(mx[1], o1);
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float neg_mx = -mx[j] * kLog2e;
#pragma unroll
            for (int i = 0; i < 16; ++i) x[j][i] = ex2s(fmaf(x[j][i], kLog2e, neg_mx));
            sm[j] = (((x[j][0] + x[j][1]) + (x[j][2] + x[j][3])) + ((x[j][4] + x[j][5]) + (x[j][6] + x[j][7]))) +
                    (((x[j][8] + x[j][9]) + (x[j][10] + x[j][11])) + ((x[j][12] + x[j][13]) + (x[j][14] + x[j][15])));
          }
#pragma unroll
          for (int o = 1; o < 8; o <<= 1) {
            const float o0 = __shfl_xor_sync(0xffffffffu, sm[0], o), o1 = __shfl_xor_sync(0xffffffffu, sm[1], o);
            sm[0] += o0; sm[1] += o1;
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float inv = 1.f / sm[j];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[j][i] *= inv;
          }
        } else if (FEAT == SLA_PHI_RELU) {
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 16; ++i) x[j][i] = fmaxf(x[j][i], 0.f);
        } else {
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 16; ++i) x[j][i] = x[j][i] > 0.f ? x[j][i] + 1.f : __expf(x[j][i]);      // elu(x) + 1
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const bool live = row0 + r + 16 * j < L;   // rows past the end were zero-filled by the copy and contribute nothing
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            w[j][i] = live ? Elem<T>::pack2(x[j][2 * i], x[j][2 * i + 1]) : 0u;
            const float2 f = Elem<T>::unpack2(w[j][i]);     // phi(k) is rounded to T before it is used (core.py:91)
            zacc[2 * i] += f.x;
            zacc[2 * i + 1] += f.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          st_shared_v4(a0 + j * 2048, w[j][0], w[j][1], w[j][2], w[j][3]);
          st_shared_v4(a0 + j * 2048 + SLAB, w[j][4], w[j][5], w[j][6], w[j][7]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(BAR(B_X + st), lane);
    }
    if (ok && n_tiles > 0) ok = mbar_wait(BAR(B_DONE), 0, kSErrG, p.err);
    ok = !state_rows_any(!ok || *abortp != 0);
    if (!ok) *abortp = 1;
    if (ok) {
      tc_fence_after();
      // ---- H of this chunk: row i of H[i][j] is this thread's TMEM lane ----
      const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
      float* hrow = out + static_cast<size_t>(tid) * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t hv[32];
        if (n_tiles > 0) {
          tmem_ld_x32(tmem + lane_addr + c0, hv);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) hv[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(hrow + c0 + i) = make_float4(__uint_as_float(hv[i]), __uint_as_float(hv[i + 1]),
                                                                   __uint_as_float(hv[i + 2]), __uint_as_float(hv[i + 3]));
      }
      // ---- z of this chunk: the sixteen row groups' sums, folded in a fixed order (the first K tile is free: every
      // MMA has completed) ----
      float* red = reinterpret_cast<float*>(base_p);            // [16][D]
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        red[prow * D + e8 * 8 + i] = zacc[i];
        red[prow * D + 64 + e8 * 8 + i] = zacc[8 + i];
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      float s = 0.f;
#pragma unroll
      for (int g = 0; g < 16; ++g) s += red[g * D + tid];
      out[D * D + tid] = s;
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace tc

template <typename T>
static int launch_state_tc(const sla_shape* s, const void* k, const void* v, float* partial, int nch, int rows,
                           cudaStream_t st) {
  constexpr int D = 128;
  const int bh = s->B * s->H;
  CUtensorMap tk, tv;
  int rc;
  if ((rc = make_tmap_3d(&tk, k, s->dtype, D, s->L, bh, tc::kStateTileRows)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tv, v, s->dtype, D, s->L, bh, tc::kStateTileRows)) != SLA_OK) return rc;
  tc::LinStateParams p;
  p.partial = partial;
  p.err = tc_error_word();
  if (p.err == nullptr) return SLA_ERR_CUDA;
  p.L = s->L; p.nch = nch; p.rows = rows;
  const int smem = 1024 + tc::kStateStages * 2 * 2 * tc::kStateTileRows * 128;   // stages of {K, V}, two slabs each
  auto go = [&](auto kern) -> int {
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    SLA_CUDA_OK(launch_pdl<false>(kern, dim3(nch, bh), dim3(192), smem, st, tk, tv, p));
    SLA_LAUNCH_OK();
    return SLA_OK;
  };
  switch (s->feature_map) {
    case SLA_PHI_SOFTMAX: return go(tc::linear_state_tc_kernel<T, SLA_PHI_SOFTMAX>);
    case SLA_PHI_RELU: return go(tc::linear_state_tc_kernel<T, SLA_PHI_RELU>);
    default: return go(tc::linear_state_tc_kernel<T, SLA_PHI_ELU>);
  }
}

// The per-chunk partials of the linear state at head dim 128 and chunks that are whole tiles of 32 rows;
// SLA_ERR_UNSUPPORTED otherwise (the caller then runs the mma.sync kernel). The reduction over chunks is the caller's.
int run_linear_state_partials_tc(const sla_shape* s, const void* k, const void* v, float* partial, int nch, int rows,
                                 cudaStream_t st) {
  if (s->D != 128 || rows % tc::kStateTileRows != 0) return SLA_ERR_UNSUPPORTED;
  return s->dtype == SLA_BF16 ? launch_state_tc<__nv_bfloat16>(s, k, v, partial, nch, rows, st)
                              : launch_state_tc<__half>(s, k, v, partial, nch, rows, st);
}

}  // namespace sla
