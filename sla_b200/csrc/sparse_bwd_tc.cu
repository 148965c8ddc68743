// dK and dV of the block-sparse branch on tcgen05 / TMEM / TMA (mathematics:
// sparse_linear_attention/kernel.py:167-237) and the host entry of the tcgen05 backward. dQ is sparse_bwd_dq_tc.cu;
// it also leaves the row statistics this kernel reads (kernel.py:85-105).
//
// A CTA owns a 128-key tile (two adjacent KV blocks; K, V stationary in shared memory) and streams
// 64-row slices Q_i, dO_i of the query blocks that selected either block:
//   T1 = K Q_i^T,  T2 = V dO_i^T (transposed scores),  dV += P^T dO_i,  dK += dS^T Q_i.
// As in the forward, the tile walks the UNION of the two blocks' (ascending) column lists; two mask
// bits per entry say which half selected it and the other half contributes zeros, so all MMAs run at
// M = 128 while the mask stays 64 x 64.
//
// Roles (576 threads, one CTA per SM):
//   warps 0-15  four compute groups of 128 threads (thread = tile row = TMEM lane). Group g works on
//               entries j = g & 1 (mod 2) in TMEM buffer g & 1 and on the 32 score columns
//               [32 (g >> 1), +32): it reads T1, T2, forms P and dS (the backward has no cross-entry or
//               cross-column state) and writes them back as 16-bit A operands over its own columns.
//   warp 16     TMA producer (stationary tiles once, then a ring of streamed tiles + row stats)
//   warp 17     MMA issuer.
// TMEM: acc1 [0,D) (dK), acc2 [D,2D) (dV), then per buffer T1 (64 cols), T2 (64 cols).
// Row statistics (lse, delta) come from a padded (B*H, Lpad, 2) fp32 array written by the dQ kernel, which runs
// first (delta = rowsum(o_s * dO), kernel.py:102-105; padding rows hold lse = +inf).
// All waits are bounded; see tc_common.cuh.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace sla {
namespace tc {

struct TcBwdParams {
  const int32_t* list;       // col_index (B*H, mb*topk)
  const int32_t* offsets;    // col_offsets (B*H, nb+1)
  const float2* stats;       // (B*H, Lpad) {lse, delta}
  int* err;
  long long* trace;          // optional timeline of CTA (0,0): [role 0..3][entry < 64][4 events], SM clock cycles
  int L, Lpad, mb, nb, topk, max_entries;
  int accumulate;            // add the result to what dk / dv already hold (the linear branch's part)
  float scale, scale_log2;
  // the linear branch's dk, dv computed in the epilogue (feature < 0: not fused)
  int lin_feature;           // sla_feature or -1
  const float* dz;           // [BH][D] fp32 gradient of z = sum phi(k)
};

__device__ __forceinline__ float ex2b(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void trace_ev(long long* tr, int role, int j, int ev) {
  if (tr != nullptr && j < 64) tr[(role * 64 + j) * 4 + ev] = clock64();
}

enum : int { kBErrX = 201, kBErrYFull = 202, kBErrYEmpty = 203, kBErrTFull = 204, kBErrCFull = 205,
             kBErrAcc = 206, kBErrDrain = 207, kBErrDh = 208, kBErrPhi = 209, kBErrLin = 210 };

template <typename T, int D, int BM, bool PLAIN>
__global__ void __launch_bounds__(576, 1)
sparse_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                     const __grid_constant__ CUtensorMap tmY1, const __grid_constant__ CUtensorMap tmY2,
                     const __grid_constant__ CUtensorMap tmO1, const __grid_constant__ CUtensorMap tmO2,
                     const __grid_constant__ CUtensorMap tmDH, TcBwdParams p) {
  constexpr int SLABS = D / 64;
  constexpr int X_SLAB = 128 * 128, Y_SLAB = 64 * 128;
  constexpr int X_BYTES = SLABS * X_SLAB, Y_BYTES = SLABS * Y_SLAB;
  constexpr int NS = D == 128 ? 4 : 6;                       // ring stages
  constexpr int STAT_BYTES = 64 * 8;
  constexpr int SL = BM / 64;                                // 64-row slices per list entry (a query block)
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_T = idesc_f16(FMT, 128, 64, 0, 0);
  constexpr uint32_t IDESC_ACC = idesc_f16(FMT, 128, D, 0, 1);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int COL_ACC1 = 0, COL_ACC2 = D, COL_T = 2 * D;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * NS + 10];
  __shared__ float s_dz[D];                        // fused linear backward: gradient of z
  __shared__ float s_e[3][4][128];                 // row-wide maxima / sums handed between the four compute groups
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_n_entries;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  pdl_entry();

  const uint32_t raw_a = smem_u32(smem_raw);
  const uint32_t base_a = (raw_a + 1023u) & ~1023u;
  uint8_t* base_p = smem_raw + (base_a - raw_a);
  const uint32_t sX1 = base_a, sX2 = sX1 + X_BYTES;
  const uint32_t sY0 = sX2 + X_BYTES;                        // stage s: Y1 at sY0 + s*2*Y_BYTES, Y2 right after
  const uint32_t sStat0 = sY0 + NS * 2 * Y_BYTES;            // stage s: 64 x {lse, delta}
  const float2* stat_p = reinterpret_cast<const float2*>(base_p + 2 * X_BYTES + NS * 2 * Y_BYTES);
  int32_t* ulist = reinterpret_cast<int32_t*>(base_p + 2 * X_BYTES + NS * 2 * Y_BYTES + NS * STAT_BYTES);

  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // 0 x_full | 1..NS y_full | NS+1..2NS y_empty | then t_full[2], c_full[2], acc_done
  constexpr int B_X = 0, B_YF = 1, B_YE = 1 + NS, B_T = 1 + 2 * NS, B_C = 3 + 2 * NS, B_ACC = 5 + 2 * NS;
  // fused linear dk, dv: dH landed in stage 0 | phi(k) written over the K tile | the two GEMMs done
  constexpr int B_DH = 7 + 2 * NS, B_PHIK = 8 + 2 * NS, B_LIN = 9 + 2 * NS;
  const bool lin = p.lin_feature >= 0;

  if (warp == 16 && lane == 0) {
    // the producer lane sets the barriers up itself and requests the stationary tiles before it merges the lists
    s_abort = *reinterpret_cast<volatile int*>(p.err) != 0;
    mbar_init(BAR(B_X), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(BAR(B_YF + s), 1);
      mbar_init(BAR(B_YE + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(BAR(B_T + b), 1);
      mbar_init(BAR(B_C + b), 8);      // one arrival per warp of the buffer's two compute groups
    }
    mbar_init(BAR(B_ACC), 1);
    mbar_init(BAR(B_DH), 1);
    mbar_init(BAR(B_PHIK), 16);
    mbar_init(BAR(B_LIN), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
    if (!s_abort) {
      mbar_expect_tx(BAR(B_X), 2 * X_BYTES);
      for (int c = 0; c < SLABS; ++c) {
        tma_load_3d(sX1 + c * X_SLAB, &tmX1, BAR(B_X), c * 64, tile * 128, bh);
        tma_load_3d(sX2 + c * X_SLAB, &tmX2, BAR(B_X), c * 64, tile * 128, bh);
      }
    }
  }
  if (warp == 16) {
    if (lane == 0) {
      prefetch_tmap(&tmX1); prefetch_tmap(&tmX2); prefetch_tmap(&tmY1); prefetch_tmap(&tmY2);
      prefetch_tmap(&tmO1); prefetch_tmap(&tmO2);
    }
    // Entry list: index | bit 28 (first half of the tile selected it) | bit 29 (second half). The two
    // source lists are copied to shared memory with coalesced loads before the serial merge.
    const int32_t *ga, *gb;
    int na, nb2;
    {
      const int32_t* off = p.offsets + static_cast<size_t>(bh) * (p.nb + 1);
      const int32_t* ci = p.list + static_cast<size_t>(bh) * p.mb * p.topk;
      const int j0 = 2 * tile;
      const int o0 = off[j0], o1 = off[j0 + 1];
      ga = ci + o0; na = o1 - o0;
      if (j0 + 1 < p.nb) { gb = ci + o1; nb2 = off[j0 + 2] - o1; } else { gb = ga; nb2 = 0; }
    }
    int32_t* ra = ulist + p.max_entries;
    int32_t* rb = ra + na;
    for (int i = lane; i < na; i += 32) ra[i] = ga[i];
    for (int i = lane; i < nb2; i += 32) rb[i] = gb[i];
    __syncwarp();
    const int n = warp_union_lists(ra, na, rb, nb2, ulist, 1 << 28, 2 << 28, lane);
    if (lane == 0) s_n_entries = n;
  }
  if (warp == 17) {
    tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  if (lin && tid < D) s_dz[tid] = p.dz[static_cast<size_t>(bh) * D + tid];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const int n_ent = s_n_entries * SL;            // streamed 64-row tiles
  volatile int* abortp = &s_abort;
  long long* tr = (tile == 0 && bh == 0) ? p.trace : nullptr;

  // global row of the streamed tile j
  auto y_row0 = [&](int j) {
    const int e = ulist[j / SL] & 0x0fffffff;
    return e * BM + (j % SL) * 64;
  };

  if (warp == 16) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && !*abortp) {
      int issued = 0;
      for (int j = 0; j < n_ent; ++j) {
        const int s = j % NS, use = j / NS;
        if (use > 0 && !mbar_wait(BAR(B_YE + s), (use - 1) & 1, kBErrYEmpty, p.err)) { *abortp = 1; break; }
        if (*abortp) break;
        trace_ev(tr, 0, j, 0);
        const int row0 = y_row0(j);
        const uint32_t y1 = sY0 + s * 2 * Y_BYTES, y2 = y1 + Y_BYTES;
        mbar_expect_tx(BAR(B_YF + s), 2 * Y_BYTES + STAT_BYTES);
        for (int c = 0; c < SLABS; ++c) {
          tma_load_3d(y1 + c * Y_SLAB, &tmY1, BAR(B_YF + s), c * 64, row0, bh);
          tma_load_3d(y2 + c * Y_SLAB, &tmY2, BAR(B_YF + s), c * 64, row0, bh);
        }
        bulk_load_1d(sStat0 + s * STAT_BYTES, p.stats + static_cast<size_t>(bh) * p.Lpad + row0, STAT_BYTES,
                     BAR(B_YF + s));
        issued = j + 1;
      }
      if (lin && !*abortp) {
        // dH of this head (D x D) into stage 0 once its last streamed tiles have been consumed
        const int uses0 = (n_ent + NS - 1) / NS;
        bool free0 = uses0 == 0 || mbar_wait(BAR(B_YE), (uses0 - 1) & 1, kBErrYEmpty, p.err);
        if (!free0) *abortp = 1;
        else {
          mbar_expect_tx(BAR(B_DH), D * D * 2);
          for (int r = 0; r < D / 64; ++r)
            for (int c = 0; c < SLABS; ++c)
              tma_load_3d(sY0 + c * (D * 128) + r * (64 * 128), &tmDH, BAR(B_DH), c * 64, r * 64, bh);
          if (*abortp) mbar_wait_drain(BAR(B_DH), 0, p.err);
        }
      }
      if (*abortp) {
        mbar_wait_drain(BAR(B_X), 0, p.err);
        for (int j = max(0, issued - NS); j < issued; ++j) mbar_wait_drain(BAR(B_YF + j % NS), (j / NS) & 1, p.err);
      }
    }
  } else if (warp == 17) {
    // ------------------------------ MMA issuer ------------------------------
    // All 32 lanes run the control flow; one elected lane issues the tcgen05 instructions.
    if (!*abortp) {
      long long* trm = lane == 0 ? tr : nullptr;
      const uint32_t x1_lo = desc_lo(sX1, 16), x2_lo = desc_lo(sX2, 16);
      auto issue_t = [&](int j) {
        const int s = j % NS, b = j & 1;
        const uint32_t y1_lo = desc_lo(sY0 + s * 2 * Y_BYTES, 16), y2_lo = desc_lo(sY0 + s * 2 * Y_BYTES + Y_BYTES, 16);
        const uint32_t t1 = tmem + COL_T + b * 128, t2 = t1 + 64;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t yo = ((kk >> 2) * Y_SLAB + (kk & 3) * 32) >> 4;
            mma_ss(t1, x1_lo + (((kk >> 2) * X_SLAB + (kk & 3) * 32) >> 4), y1_lo + yo, IDESC_T, kk > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t yo = ((kk >> 2) * Y_SLAB + (kk & 3) * 32) >> 4;
            mma_ss(t2, x2_lo + (((kk >> 2) * X_SLAB + (kk & 3) * 32) >> 4), y2_lo + yo, IDESC_T, kk > 0 ? 1u : 0u);
          }
          tc_commit(BAR(B_T + b));
        }
        __syncwarp();
      };
      bool ok = warp_all(mbar_wait(BAR(B_X), 0, kBErrX, p.err));
      for (int j = 0; ok && j < 2 && j < n_ent; ++j) {
        ok = warp_all(mbar_wait(BAR(B_YF + j % NS), (j / NS) & 1, kBErrYFull, p.err));
        if (!ok) break;
        tc_fence_after();
        issue_t(j);
      }
      for (int j = 0; ok && j < n_ent; ++j) {
        const int s = j % NS, b = j & 1;
        trace_ev(trm, 1, j, 0);
        ok = warp_all(mbar_wait(BAR(B_C + b), (j >> 1) & 1, kBErrCFull, p.err));
        if (!ok) break;
        trace_ev(trm, 1, j, 1);
        tc_fence_after();
        // streamed tiles as MN-major B operands: 8-row groups 1024 B apart, 64-column slabs Y_SLAB apart
        const uint32_t y1_lo = desc_lo(sY0 + s * 2 * Y_BYTES, Y_SLAB), y2_lo = desc_lo(sY0 + s * 2 * Y_BYTES + Y_BYTES, Y_SLAB);
        const uint32_t a1 = tmem + COL_T + b * 128, a2 = a1 + 64;   // 16-bit operands written by the compute groups
        const uint32_t acc_on = j > 0 ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            // 16-bit operand columns: elements [0,32) packed at +0..15, elements [32,64) at +32..47
            const uint32_t ao = (kk >> 1) * 32 + (kk & 1) * 8;
            const uint32_t ko = (kk * 2048) >> 4;
            mma_ts(tmem + COL_ACC2, a1 + ao, y2_lo + ko, IDESC_ACC, kk > 0 ? 1u : acc_on);   // dV += P^T dO_i  (kernel.py:220)
            mma_ts(tmem + COL_ACC1, a2 + ao, y1_lo + ko, IDESC_ACC, kk > 0 ? 1u : acc_on);   // dK += dS^T Q_i (kernel.py:225)
          }
          tc_commit(BAR(B_YE + s));
        }
        __syncwarp();
        trace_ev(trm, 1, j, 2);
        if (j + 2 < n_ent) {
          ok = warp_all(mbar_wait(BAR(B_YF + (j + 2) % NS), ((j + 2) / NS) & 1, kBErrYFull, p.err));
          if (!ok) break;
          tc_fence_after();
          issue_t(j + 2);
        }
        trace_ev(trm, 1, j, 3);
      }
      if (ok) {
        if (elect_one()) tc_commit(BAR(B_ACC));
        __syncwarp();
      }
      if (ok && lin) {
        // linear branch (core.py:91-94 backwards): dV += phi(K) dH and dphi_k = V dH^T, with phi(K) written over
        // the K tile by the compute groups and dH ([i][j], one D x D tile) read once as MN-major and once as
        // K-major B operand
        ok = warp_all(mbar_wait(BAR(B_DH), 0, kBErrDh, p.err) && mbar_wait(BAR(B_PHIK), 0, kBErrPhi, p.err));
        if (ok) {
          tc_fence_after();
          constexpr uint32_t IDESC_DPHI = idesc_f16(FMT, 128, D, 0, 0);
          const uint32_t dh_mn = desc_lo(sY0, D * 128), dh_k = desc_lo(sY0, 16);
          const uint32_t acc_v = n_ent > 0 ? 1u : 0u;
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t xo = ((kk >> 2) * X_SLAB + (kk & 3) * 32) >> 4;          // K-major A: phi(K), V
              mma_ss(tmem + COL_ACC2, x1_lo + xo, dh_mn + ((kk * 2048) >> 4), IDESC_ACC, kk > 0 ? 1u : acc_v);
            }
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t xo = ((kk >> 2) * X_SLAB + (kk & 3) * 32) >> 4;
              const uint32_t ho = ((kk >> 2) * (D * 128) + (kk & 3) * 32) >> 4;        // K-major B: rows i, k = j
              mma_ss(tmem + COL_T, x2_lo + xo, dh_k + ho, IDESC_DPHI, kk > 0 ? 1u : 0u);
            }
            tc_commit(BAR(B_LIN));
          }
          __syncwarp();
        }
      }
      if (!ok) *abortp = 1;
    }
  } else {
    // ------------------------------ compute groups ------------------------------
    const int wg = warp >> 2;                               // 0..3
    const int buf = wg & 1, ch = wg >> 1;                   // TMEM buffer, column half
    const int row = tid & 127;                              // tile row == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int half = row >> 6;
    const float sc = p.scale_log2;
    const int grow = tile * 128 + row;                      // global key row
    const bool key_ok = grow < L;                           // keys past the end give P = 0 (kernel.py:216)
    bool ok = !*abortp;
    for (int j = buf; ok && j < n_ent; j += 2) {
      long long* trc = ((warp & 3) == 0 && lane == 0) ? tr : nullptr;
      trace_ev(trc, 2 + ch, j, 0);
      if (!mbar_wait(BAR(B_T + buf), (j >> 1) & 1, kBErrTFull, p.err)) { ok = false; break; }
      if (*abortp) { ok = false; break; }
      trace_ev(trc, 2 + ch, j, 1);
      if (!mbar_wait(BAR(B_YF + j % NS), (j / NS) & 1, kBErrYFull, p.err)) { ok = false; break; }  // row stats landed
      tc_fence_after();
      const int entry = ulist[j / SL];
      const bool active = (entry >> (28 + half)) & 1;
      const uint32_t t1 = tmem + lane_addr + COL_T + buf * 128 + ch * 32, t2 = t1 + 64;
      const float4* stc = reinterpret_cast<const float4*>(stat_p + (j % NS) * 64 + ch * 32);
      uint32_t pp[16], ds[16];
      if (active) {
        uint32_t sv[32], dv[32];
        tmem_ld_x32(t1, sv);
        tmem_ld_x32(t2, dv);
        tmem_wait_ld();
        trace_ev(trc, 2 + ch, j, 2);
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float4 st = stc[c >> 1];                                    // {lse, delta} of two query rows
          const float lse0 = st.x, del0 = st.y, lse1 = st.z, del1 = st.w;
          float p0, p1, w0, w1;                                             // P and the factor of (dP - delta) in dS
          if (PLAIN) {   // no softmax (BwdParams::plain): K and Q tiles are feature maps
            p0 = __uint_as_float(sv[c]); p1 = __uint_as_float(sv[c + 1]);   // zero rows (past the end) give S = 0
            w0 = w1 = 1.0f;
          } else {
            p0 = ex2b(__uint_as_float(sv[c]) * sc - lse0);
            p1 = ex2b(__uint_as_float(sv[c + 1]) * sc - lse1);
            if (!key_ok) p0 = p1 = 0.f;                                     // kernel.py:216
            w0 = p0; w1 = p1;
          }
          pp[c >> 1] = Elem<T>::pack2(p0, p1);
          ds[c >> 1] = Elem<T>::pack2(w0 * (__uint_as_float(dv[c]) - del0),
                                      w1 * (__uint_as_float(dv[c + 1]) - del1));   // kernel.py:161 / :224
        }
      } else {
#pragma unroll
        for (int c = 0; c < 16; ++c) pp[c] = ds[c] = 0u;
      }
      tmem_st_x16(t1, pp);
      tmem_st_x16(t2, ds);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(BAR(B_C + buf), lane);
      trace_ev(trc, 2 + ch, j, 3);
    }
    if (ok && n_ent > 0) ok = mbar_wait(BAR(B_ACC), 0, kBErrAcc, p.err);
    if (ok) ok = mbar_wait(BAR(B_X), 0, kBErrX, p.err);   // the stationary tiles (reused as staging) have landed
    if (!ok) *abortp = 1;
    asm volatile("bar.sync 1, 512;\n" ::: "memory");
    if (!*abortp) {
      tc_fence_after();
      if (lin) {
        // ---- fused backward of the linear branch for this key tile (core.py:91-94):
        //   dphi_k = V dH^T + dz,  dk_lin = phi'(k) dphi_k,  dv_lin = phi(k) dH
        // Each compute group owns D/4 columns of every row: it forms phi(k) for them (row-wide maxima and sums go
        // through s_e), writes phi(k) over the K tile as the A operand of the dV GEMM, and afterwards turns its
        // columns of dphi_k into dk_lin and adds the sparse branch's dK.
        constexpr int CW = D / 4;                             // columns per group
        const int c_lo = wg * CW;
        auto chunk_addr = [&](uint32_t tile_base, int c8) {
          return tile_base + (c8 >> 3) * X_SLAB + row * 128 + (((c8 & 7) ^ (row & 7)) << 4);
        };
        auto exchange = [&](int slot, float mine, bool take_max) {
          s_e[slot][wg][row] = mine;
          asm volatile("bar.sync 1, 512;\n" ::: "memory");
          float r = s_e[slot][0][row];
#pragma unroll
          for (int g2 = 1; g2 < 4; ++g2) r = take_max ? fmaxf(r, s_e[slot][g2][row]) : r + s_e[slot][g2][row];
          return r;
        };
        float x[CW];
#pragma unroll
        for (int c8 = 0; c8 < CW / 8; ++c8) {
          uint32_t w0, w1, w2, w3;
          ld_shared_v4(chunk_addr(sX1, c_lo / 8 + c8), w0, w1, w2, w3);
          const uint32_t w[4] = {w0, w1, w2, w3};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = Elem<T>::unpack2(w[i]);
            x[c8 * 8 + 2 * i] = f.x; x[c8 * 8 + 2 * i + 1] = f.y;
          }
        }
        if (PLAIN) {
          // the stationary tile already holds phi(k)
        } else if (p.lin_feature == SLA_PHI_SOFTMAX) {
          float mx = x[0];
#pragma unroll
          for (int c = 1; c < CW; ++c) mx = fmaxf(mx, x[c]);
          mx = exchange(0, mx, true);
          float sm = 0.f;
#pragma unroll
          for (int c = 0; c < CW; ++c) { x[c] = __expf(x[c] - mx); sm += x[c]; }
          const float inv_s = 1.f / exchange(1, sm, false);
#pragma unroll
          for (int c = 0; c < CW; ++c) x[c] *= inv_s;
        } else {
#pragma unroll
          for (int c = 0; c < CW; ++c) {
            if (p.lin_feature == SLA_PHI_RELU) x[c] = fmaxf(x[c], 0.f);
            else x[c] = x[c] > 0.f ? x[c] + 1.f : __expf(x[c]);      // elu(x) + 1
          }
        }
        const bool key_live = grow < L;                        // rows past the end: K was zero-filled, phi must be 0
        uint32_t phi[CW / 2];                                  // phi(k) rounded to T (core.py:91)
#pragma unroll
        for (int c = 0; c < CW; c += 2) phi[c >> 1] = key_live ? Elem<T>::pack2(x[c], x[c + 1]) : 0u;
#pragma unroll
        for (int c8 = 0; c8 < CW / 8; ++c8)
          st_shared_v4(chunk_addr(sX1, c_lo / 8 + c8), phi[4 * c8], phi[4 * c8 + 1], phi[4 * c8 + 2], phi[4 * c8 + 3]);
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive_warp(BAR(B_PHIK), lane);
        const bool lin_ok = mbar_wait(BAR(B_LIN), 0, kBErrLin, p.err);
        if (!lin_ok) *abortp = 1;
        float dk_out[CW];
        float ps = 0.f;                                        // sum_i phi_i dphi_i of this group's columns
        if (lin_ok) {
          tc_fence_after();
          uint32_t tv[CW], ak0[CW];
          if constexpr (CW == 32) tmem_ld_x32(tmem + lane_addr + COL_T + c_lo, tv); else tmem_ld_x16(tmem + lane_addr + COL_T + c_lo, tv);
          if (PLAIN && n_ent > 0) {    // dK of the un-normalised product is a gradient of phi(k): it goes through phi' too
            if constexpr (CW == 32) tmem_ld_x32(tmem + lane_addr + COL_ACC1 + c_lo, ak0); else tmem_ld_x16(tmem + lane_addr + COL_ACC1 + c_lo, ak0);
          } else {
#pragma unroll
            for (int c = 0; c < CW; ++c) ak0[c] = 0u;
          }
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < CW; c += 2) {
            const float2 ph = Elem<T>::unpack2(phi[c >> 1]);
            x[c] = ph.x; x[c + 1] = ph.y;
            dk_out[c] = __uint_as_float(tv[c]) + s_dz[c_lo + c] + __uint_as_float(ak0[c]);
            dk_out[c + 1] = __uint_as_float(tv[c + 1]) + s_dz[c_lo + c + 1] + __uint_as_float(ak0[c + 1]);
            ps += ph.x * dk_out[c] + ph.y * dk_out[c + 1];
          }
        }
        // every compute thread takes part in the exchange, whatever its wait returned (a named barrier is not bounded)
        if (p.lin_feature == SLA_PHI_SOFTMAX) ps = exchange(2, ps, false);
        if (lin_ok) {
          if (p.lin_feature == SLA_PHI_SOFTMAX) {
#pragma unroll
            for (int c = 0; c < CW; ++c) dk_out[c] = x[c] * (dk_out[c] - ps);
          } else if (p.lin_feature == SLA_PHI_RELU) {
#pragma unroll
            for (int c = 0; c < CW; ++c) dk_out[c] = x[c] > 0.f ? dk_out[c] : 0.f;
          } else {
#pragma unroll
            for (int c = 0; c < CW; ++c) dk_out[c] = x[c] > 1.f ? dk_out[c] : x[c] * dk_out[c];   // x > 0 iff phi > 1
          }
          // + the sparse branch's dK (times the softmax scale, kernel.py:236); dV already holds both parts
          uint32_t ak[CW], av[CW];
          if (n_ent > 0 && !PLAIN) {
            if constexpr (CW == 32) tmem_ld_x32(tmem + lane_addr + COL_ACC1 + c_lo, ak); else tmem_ld_x16(tmem + lane_addr + COL_ACC1 + c_lo, ak);
          } else {
#pragma unroll
            for (int c = 0; c < CW; ++c) ak[c] = 0u;
          }
          if constexpr (CW == 32) tmem_ld_x32(tmem + lane_addr + COL_ACC2 + c_lo, av); else tmem_ld_x16(tmem + lane_addr + COL_ACC2 + c_lo, av);
          tmem_wait_ld();
#pragma unroll
          for (int c8 = 0; c8 < CW / 8; ++c8) {
            uint32_t wk[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = c8 * 8 + 2 * i;
              wk[i] = Elem<T>::pack2(fmaf(__uint_as_float(ak[c]), p.scale, dk_out[c]),
                                     fmaf(__uint_as_float(ak[c + 1]), p.scale, dk_out[c + 1]));
              wv[i] = Elem<T>::pack2(__uint_as_float(av[c]), __uint_as_float(av[c + 1]));
            }
            st_shared_v4(chunk_addr(sX1, c_lo / 8 + c8), wk[0], wk[1], wk[2], wk[3]);
            st_shared_v4(chunk_addr(sX2, c_lo / 8 + c8), wv[0], wv[1], wv[2], wv[3]);
          }
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 512;\n" ::: "memory");
        if (tid == 0 && !*abortp) {
          for (int c = 0; c < SLABS; ++c) {
            tma_store_3d(&tmO1, sX1 + c * X_SLAB, c * 64, tile * 128, bh);
            tma_store_3d(&tmO2, sX2 + c * X_SLAB, c * 64, tile * 128, bh);
          }
          tma_store_commit();
          tma_store_wait_read();
        }
      } else {
      // accumulators -> T, staged over the (idle) stationary tiles in the swizzled slab layout, then
      // TMA stores; rows past the end of the sequence are clipped by the copy engine.
      // groups 0,1 convert the two column halves of acc1 (dK), groups 2,3 those of acc2 (dV)
      const bool second = wg >= 2;
      const int span = D / 2;
      const int c_lo = (wg & 1) * span, c_hi = c_lo + span;
      const uint32_t acc = tmem + lane_addr + (second ? COL_ACC2 : COL_ACC1);
      const uint32_t stage = second ? sX2 : sX1;
      const float mul = second ? 1.0f : p.scale;   // dK carries the softmax scale (kernel.py:236)
      for (int c0 = c_lo; c0 < c_hi; c0 += 16) {
        uint32_t ov[16];
        if (n_ent > 0) {
          tmem_ld_x16(acc + c0, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < 16; ++c) ov[c] = 0u;          // nothing selected this tile: gradient is zero
        }
        const uint32_t slab = stage + (c0 >> 6) * X_SLAB + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 2; ++q4) {
          uint32_t w0 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 0]) * mul, __uint_as_float(ov[q4 * 8 + 1]) * mul);
          uint32_t w1 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 2]) * mul, __uint_as_float(ov[q4 * 8 + 3]) * mul);
          uint32_t w2 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 4]) * mul, __uint_as_float(ov[q4 * 8 + 5]) * mul);
          uint32_t w3 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 6]) * mul, __uint_as_float(ov[q4 * 8 + 7]) * mul);
          const int chunk = ((c0 & 63) >> 3) + q4;
          const uint32_t addr = slab + ((chunk ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 512;\n" ::: "memory");
      if (tid == 0) {
        if (p.accumulate) {   // read-modify-write done by the copy engine in L2: no load stalls this CTA
          for (int c = 0; c < SLABS; ++c) tma_reduce_add_3d(&tmO1, sX1 + c * X_SLAB, c * 64, tile * 128, bh);
          for (int c = 0; c < SLABS; ++c) tma_reduce_add_3d(&tmO2, sX2 + c * X_SLAB, c * 64, tile * 128, bh);
        } else {
          for (int c = 0; c < SLABS; ++c) tma_store_3d(&tmO1, sX1 + c * X_SLAB, c * 64, tile * 128, bh);
          for (int c = 0; c < SLABS; ++c) tma_store_3d(&tmO2, sX2 + c * X_SLAB, c * 64, tile * 128, bh);
        }
        tma_store_commit();
        tma_store_wait_read();
      }
      }   // !lin
    }
  }
  // ------------------------------ teardown ------------------------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 17) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace tc

// Diagnostic timeline buffer (2 x 1024 int64), set through sla_debug_set_trace.
static long long* g_trace_buffer = nullptr;
void set_trace_buffer(long long* p) { g_trace_buffer = p; }
long long* trace_buffer() { return g_trace_buffer; }

static int bwd_tc_smem_bytes(int D, int max_entries) {
  const int NS = D == 128 ? 4 : 6;
  return 1024 + 2 * 128 * D * 2 + NS * 2 * 64 * D * 2 + NS * 512 + 2 * max_entries * 4 + 16;
}
constexpr int kBwdStaticSmem = 8 * 1024;   // statically allocated shared memory of the kernels (barriers, exchange slots)

template <typename T, int D, int BM, bool PLAIN>
static int launch_dkdv(const sla_shape* s, const BwdParams& bp, const float2* stats, int Lpad, cudaStream_t st) {
  const int bh = s->B * s->H;
  CUtensorMap x1, x2, y1, y2, o1, o2, dh;
  int rc;
  if ((rc = make_tmap_3d(&x1, bp.k, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&x2, bp.v, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&y1, bp.q, s->dtype, D, s->L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&y2, bp.d_o, s->dtype, D, s->L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&o1, bp.dk, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&o2, bp.dv, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  const bool lin = bp.lin_dh != nullptr;
  dh = o1;
  if (lin && (rc = make_tmap_rows(&dh, bp.lin_dh, s->dtype, D, D, bh, size_t(D) * D * 2, 64)) != SLA_OK) return rc;
  tc::TcBwdParams p;
  p.list = bp.col_index;
  p.offsets = bp.col_offsets;
  p.stats = stats;
  p.err = tc_error_word();
  if (p.err == nullptr) return SLA_ERR_CUDA;
  p.trace = g_trace_buffer ? g_trace_buffer + 1024 : nullptr;
  p.L = s->L; p.Lpad = Lpad; p.mb = bp.mb; p.nb = bp.nb; p.topk = bp.topk;
  p.scale = bp.scale; p.scale_log2 = bp.scale_log2; p.accumulate = bp.accumulate;
  p.lin_feature = lin ? s->feature_map : -1;
  p.dz = bp.lin_dz;
  p.max_entries = 2 * bp.mb;            // a KV block may have been selected by every query block
  const int smem = bwd_tc_smem_bytes(D, p.max_entries);
  if (smem + kBwdStaticSmem > 227 * 1024) return SLA_ERR_BAD_SHAPE;
  auto kern = tc::sparse_bwd_dkdv_kernel<T, D, BM, PLAIN>;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  SLA_CUDA_OK(launch_pdl(kern, dim3(ceil_div(bp.nb, 2), bh), dim3(576), smem, st, x1, x2, y1, y2, o1, o2, dh, p));
  SLA_LAUNCH_OK();
  return SLA_OK;
}

template <typename T, int D, int BM>
static int run_bwd_tc_typed(const sla_shape* s, const BwdParams& bp, float2* stats, int Lpad, cudaStream_t st) {
  const int bh = s->B * s->H;
  // nothing is launched unless both kernels fit: the caller falls back to another path on BAD_SHAPE
  if (!sparse_bwd_tc_fits(s)) return SLA_ERR_BAD_SHAPE;
  // The row statistics {lse, delta}: the dQ kernel takes delta of its own rows on the way and leaves both for the
  // dK/dV kernel; in plain mode the caller has filled them.
  int rc = run_sparse_bwd_dq_pair(s, bp, stats, Lpad, st);
  if (rc != SLA_OK) return rc;
  return bp.plain ? launch_dkdv<T, D, BM, true>(s, bp, stats, Lpad, st)
                  : launch_dkdv<T, D, BM, false>(s, bp, stats, Lpad, st);
}

// Whether the tcgen05 backward kernels fit this shape (so that a caller can decide what to fuse into them before
// it launches anything): the dK/dV kernel keeps a column-list union of up to 2 * M_BLOCKS entries in shared
// memory, the dQ kernel one of up to 2 * topk.
bool sparse_bwd_tc_fits(const sla_shape* s) {
  const int mb = ceil_div(s->L, s->BLKQ);
  return bwd_tc_smem_bytes(s->D, 2 * mb) + kBwdStaticSmem <= 227 * 1024 && sparse_bwd_dq_pair_fits(s);
}

// `stats` must hold B*H*Lpad float2 with Lpad = ceil(L/128)*128.
int run_sparse_bwd_tc(const sla_shape* s, const BwdParams& bp, void* stats, cudaStream_t st) {
  const int Lpad = ceil_div(s->L, 128) * 128;
  float2* sp = static_cast<float2*>(stats);
#define SLA_TCB(TT)                                                                                         \
  if (s->D == 64)                                                                                           \
    return s->BLKQ == 64 ? run_bwd_tc_typed<TT, 64, 64>(s, bp, sp, Lpad, st) : run_bwd_tc_typed<TT, 64, 128>(s, bp, sp, Lpad, st); \
  return s->BLKQ == 64 ? run_bwd_tc_typed<TT, 128, 64>(s, bp, sp, Lpad, st) : run_bwd_tc_typed<TT, 128, 128>(s, bp, sp, Lpad, st);
  if (s->dtype == SLA_BF16) { SLA_TCB(__nv_bfloat16) }
  SLA_TCB(__half)
#undef SLA_TCB
}

}  // namespace sla
