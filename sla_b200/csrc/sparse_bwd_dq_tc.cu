// dQ of the block-sparse branch (sparse_linear_attention/kernel.py:108-165) on tcgen05, processing the
// selected KV blocks of a 128-row query tile in PAIRS.
//
// An M=128, N=64 score MMA cannot be fed at the tensor peak (its operands come from shared or tensor memory
// at 46-60 clk per k-step against 32 at the peak); an N=128 one can. So two list entries (two 64-row KV
// blocks, any two: they need not be adjacent in the sequence) are loaded side by side as one 128-row tile and
//   T1 = Q [K_a; K_b]^T,   T2 = dO [V_a; V_b]^T            (128 x 128, 8 k-steps of N = 128 each)
//   dS = P * (T2 - delta),   dQ += dS [K_a; K_b]           (8 k-steps of N = D)
// 512 TMEM columns hold dQ (D), the 16-bit Q and dO operands (D) and ONE T1 and ONE T2 buffer of 128 columns.
// The single buffers still overlap everything: T1 is only read (P stays in registers), so T1 of the next pair
// is issued as soon as the compute threads have loaded this pair's T1; T2 of the next pair follows the
// accumulation GEMMs of this pair (which read dS from the T2 columns), the tensor pipe running in issue order.
// Steady state of the pipe: ACC(p), T2(p+1), T1(p+2) back to back while the compute threads turn T2(p+1) into dS.
//
// Roles (576 threads, one CTA per SM): warps 0-15 four compute groups of 128 threads (thread = tile row =
// TMEM lane); group g owns score columns [32 g, 32 g + 32), i.e. half of entry g / 2 of the pair. Warp 16 TMA
// producer, warp 17 MMA issuer. As in the other kernels a tile of two 64-row query blocks walks the union of
// their lists with two mask bits per entry; an odd list gets its last entry twice, the copy masked out.
// The kernel also takes the backward's row statistic delta = rowsum(o_s * dO) (kernel.py:102-105): the two groups that
// move the dO tile to tensor memory hold its rows in registers at that point and read the matching rows of o_s from
// global memory; {lse, delta} of the tile's rows go to the padded array the dK/dV kernel reads.
// All waits are bounded (tc_common.cuh).
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace sla {
namespace tc {

struct TcDqParams {
  const int32_t* lut;        // (B*H, mb, topk)
  const float2* stats;       // (B*H, Lpad) {lse, delta}: read in the no-softmax variant, WRITTEN otherwise (below)
  // softmax variant: the kernel takes delta = rowsum(o_s * dO) (kernel.py:102-105) of its own 128 rows while it
  // moves the dO tile to tensor memory, and leaves {lse, delta} (rows past L: {+inf, 0}) in `stats_out` for the
  // dK/dV kernel; no separate pass over o_s and dO
  const void* o_s;           // (B*H, L, D)
  const float* lse;          // (B*H, L)
  float2* stats_out;         // (B*H, Lpad)
  int* err;
  long long* trace;          // optional: 8 words per CTA {sm, start ns, end ns, then SM clocks since the start of the
                             // CTA: set-up done, operands in TMEM, first T1 there, accumulation done, stored}
  int L, Lpad, mb, topk;
  int accumulate;            // add to what dq already holds (the linear branch's part)
  float scale, scale_log2;
};

__device__ __forceinline__ float ex2q(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

enum : int { kQErrX = 401, kQErrYFull = 402, kQErrYEmpty = 403, kQErrT1 = 404, kQErrT2 = 405, kQErrT1C = 406,
             kQErrC = 407, kQErrAcc = 408, kQErrDrain = 409 };

template <typename T, int D, int BM, bool PLAIN>
__global__ void __launch_bounds__(576, 1)
sparse_bwd_dq_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                          const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                          const __grid_constant__ CUtensorMap tmdQ, TcDqParams p) {
  constexpr int SLABS = D / 64;
  constexpr int X_SLAB = 128 * 128;                         // one 64-column slab of a 128-row tile
  constexpr int X_BYTES = SLABS * X_SLAB;                   // Q, dO, and each pair tile [K_a; K_b], [V_a; V_b]
  constexpr int HALF = 64 * 128;                            // rows 64..127 of a slab start here
  constexpr int NK = 3, NV = 2;                             // ring slots of [K_a; K_b] and [V_a; V_b] tiles
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_T = idesc_f16(FMT, 128, 128, 0, 0);
  constexpr uint32_t IDESC_ACC = idesc_f16(FMT, 128, D, 0, 1);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int COL_ACC = 0, COL_XQ = D, COL_XDO = D + D / 2, COL_T1 = 2 * D, COL_T2 = 2 * D + 128;
  static_assert(COL_T2 + 128 <= 512, "tensor memory budget");

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * NK + 2 * NV + 8];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_n_entries;
  __shared__ int s_abort;
  __shared__ float s_delta[2][128];      // the two column halves' share of delta

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  pdl_entry();
  long long* trc = (p.trace != nullptr && tid == 0) ? p.trace + 8 * (static_cast<size_t>(bh) * gridDim.x + tile) : nullptr;
  const long long clk0 = clock64();
  if (trc) {
    unsigned sm;
    unsigned long long ns;
    asm volatile("mov.u32 %0, %%smid;\n" : "=r"(sm));
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(ns));
    trc[0] = sm; trc[1] = static_cast<long long>(ns);
  }

  const uint32_t raw_a = smem_u32(smem_raw);
  const uint32_t base_a = (raw_a + 1023u) & ~1023u;
  uint8_t* base_p = smem_raw + (base_a - raw_a);
  // Six tile slots of X_BYTES: Q (later the dQ staging) | dO, which becomes K slot 2 once it has been copied to
  // tensor memory | K slots 0, 1 | V slots 0, 1. A K tile lives from its T1 GEMM to its accumulation GEMM (three
  // slots), a V tile only until its T2 GEMM (two).
  const uint32_t sQ = base_a, sdO = sQ + X_BYTES;
  auto k_slot = [&](int i) { return i == 2 ? sdO : base_a + (2 + i) * X_BYTES; };
  auto v_slot = [&](int i) { return base_a + (4 + i) * X_BYTES; };
  int32_t* ulist = reinterpret_cast<int32_t*>(base_p + 6 * X_BYTES);

  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // x_full | k_full[NK] | k_empty[NK] | v_full[NV] | v_empty[NV] | t1_full | t2_full | t1_consumed |
  // c_full (dS written) | acc_done | x_in_tmem
  constexpr int B_X = 0, B_KF = 1, B_KE = 1 + NK, B_VF = 1 + 2 * NK, B_VE = 1 + 2 * NK + NV, B_T1 = 1 + 2 * NK + 2 * NV,
                B_T2 = B_T1 + 1, B_T1C = B_T1 + 2, B_C = B_T1 + 3, B_ACC = B_T1 + 4, B_XT = B_T1 + 5;

  // request the two tiles of list entries 2 pi, 2 pi + 1 (producer lane only)
  auto load_pair = [&](int pi) {
    const uint32_t yk = k_slot(pi % NK), yv = v_slot(pi % NV);
    mbar_expect_tx(BAR(B_KF + pi % NK), X_BYTES);
    mbar_expect_tx(BAR(B_VF + pi % NV), X_BYTES);
    for (int e = 0; e < 2; ++e) {
      const int row0 = (ulist[2 * pi + e] & 0x0fffffff) * 64;
      for (int c = 0; c < SLABS; ++c) {
        tma_load_3d(yk + c * X_SLAB + e * HALF, &tmK, BAR(B_KF + pi % NK), c * 64, row0, bh);
        tma_load_3d(yv + c * X_SLAB + e * HALF, &tmV, BAR(B_VF + pi % NV), c * 64, row0, bh);
      }
    }
  };
  // Set-up, ordered so that as little as possible sits in front of the first GEMM: the producer warp requests
  // its LUT rows from global memory first, its lane 0 sets the barriers up and requests the stationary tiles,
  // and an early CTA-wide barrier publishes barriers and the TMEM base. The compute groups then move Q and dO
  // into tensor memory while the producer warp merges the lists and requests the first pairs; everybody else
  // picks the list up behind the `list_ready` barrier.
  constexpr int B_LIST = B_XT + 1;
  const int rows = BM == 128 ? 1 : ((2 * tile + 1 < p.mb) ? 2 : 1);
  int32_t* raw = ulist + 2 * p.topk + 2;
  int lut_early[2] = {0, 0};
  if (warp == 16) {
    const int32_t* src = p.lut + (static_cast<size_t>(bh) * p.mb + (BM == 128 ? tile : 2 * tile)) * p.topk;
    if (rows * p.topk <= 64) {                 // the usual case: at most two elements per lane, loaded right away
      if (lane < rows * p.topk) lut_early[0] = src[lane];
      if (lane + 32 < rows * p.topk) lut_early[1] = src[lane + 32];
    }
    if (lane == 0) {
      s_abort = *reinterpret_cast<volatile int*>(p.err) != 0;
      mbar_init(BAR(B_X), 1);
      for (int s = 0; s < NK; ++s) { mbar_init(BAR(B_KF + s), 1); mbar_init(BAR(B_KE + s), 1); }
      for (int s = 0; s < NV; ++s) { mbar_init(BAR(B_VF + s), 1); mbar_init(BAR(B_VE + s), 1); }
      mbar_init(BAR(B_T1), 1);
      mbar_init(BAR(B_T2), 1);
      mbar_init(BAR(B_T1C), 16);     // one arrival per compute warp
      mbar_init(BAR(B_C), 16);
      mbar_init(BAR(B_ACC), 1);
      mbar_init(BAR(B_XT), 16);
      mbar_init(BAR(B_LIST), 1);
      fence_barrier_init();
      fence_proxy_async_smem();
      if (!s_abort) {
        mbar_expect_tx(BAR(B_X), 2 * X_BYTES);
        for (int c = 0; c < SLABS; ++c) {
          tma_load_3d(sQ + c * X_SLAB, &tmQ, BAR(B_X), c * 64, tile * 128, bh);
          tma_load_3d(sdO + c * X_SLAB, &tmdO, BAR(B_X), c * 64, tile * 128, bh);
        }
      }
    }
  }
  if (warp == 17) {
    tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  volatile int* abortp = &s_abort;
  if (warp == 16) {
    if (lane == 0) { prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdQ); }
    // Entry list: block index | bit 28 (first half of the tile selected it) | bit 29 (second half)
    if (rows * p.topk <= 64) {
      if (lane < rows * p.topk) raw[lane] = lut_early[0];
      if (lane + 32 < rows * p.topk) raw[lane + 32] = lut_early[1];
    } else {
      const int32_t* src = p.lut + (static_cast<size_t>(bh) * p.mb + (BM == 128 ? tile : 2 * tile)) * p.topk;
      for (int i = lane; i < rows * p.topk; i += 32) raw[i] = src[i];
    }
    __syncwarp();
    int n;
    if (BM == 128) {
      for (int i = lane; i < p.topk; i += 32) ulist[i] = raw[i] | (3 << 28);
      n = p.topk;
      __syncwarp();
    } else {
      n = warp_union_lists(raw, p.topk, raw + p.topk, rows == 2 ? p.topk : 0, ulist, 1 << 28, 2 << 28, lane);
    }
    if (lane == 0) {
      if (n & 1) { ulist[n] = ulist[n - 1] & 0x0fffffff; ++n; }   // pad to a pair: same (finite) tile, masked out
      s_n_entries = n;
      if (!*abortp && n > 0) load_pair(0);     // its slots are fresh
      mbar_arrive(BAR(B_LIST));                // releases ulist and s_n_entries to the other warps
    }
    __syncwarp();
  }
  // everybody but the producer warp needs the list only after its own set-up work; the wait is further down
  auto list_ready = [&]() { return mbar_wait(BAR(B_LIST), 0, kQErrX, p.err); };
  if (trc) trc[3] = clock64() - clk0;

  if (warp == 16) {
    // ------------------------------ TMA producer ------------------------------
    const int n_pairs = s_n_entries >> 1;
    if (lane == 0 && !*abortp) {
      int issued = min(1, n_pairs);
      for (int pi = 1; pi < n_pairs; ++pi) {
        const int ks = pi % NK, ku = pi / NK, vs = pi % NV, vu = pi / NV;
        if (ku > 0 && !mbar_wait(BAR(B_KE + ks), (ku - 1) & 1, kQErrYEmpty, p.err)) { *abortp = 1; break; }
        if (vu > 0 && !mbar_wait(BAR(B_VE + vs), (vu - 1) & 1, kQErrYEmpty, p.err)) { *abortp = 1; break; }
        if (pi == 2 && !mbar_wait(BAR(B_XT), 0, kQErrX, p.err)) { *abortp = 1; break; }   // K slot 2 is the dO tile
        if (*abortp) break;
        load_pair(pi);
        issued = pi + 1;
      }
      if (*abortp) {
        mbar_wait_drain(BAR(B_X), 0, p.err);
        for (int j = max(0, issued - NK); j < issued; ++j) mbar_wait_drain(BAR(B_KF + j % NK), (j / NK) & 1, p.err);
        for (int j = max(0, issued - NV); j < issued; ++j) mbar_wait_drain(BAR(B_VF + j % NV), (j / NV) & 1, p.err);
      }
    }
  } else if (warp == 17) {
    // ------------------------------ MMA issuer ------------------------------
    // All 32 lanes run the control flow; one elected lane issues the tcgen05 instructions.
    if (!*abortp) {
      auto issue_t = [&](int pi, bool second) {
        const uint32_t y_lo = desc_lo(second ? v_slot(pi % NV) : k_slot(pi % NK), 16);
        const uint32_t d = tmem + (second ? COL_T2 : COL_T1);
        const uint32_t a = tmem + (second ? COL_XDO : COL_XQ);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)   // k-step: 32 bytes further inside the swizzle atom, next slab every 4 steps
            mma_ts(d, a + kk * 8, y_lo + (((kk >> 2) * X_SLAB + (kk & 3) * 32) >> 4), IDESC_T, kk > 0 ? 1u : 0u);
          tc_commit(BAR(second ? B_T2 : B_T1));
          if (second) tc_commit(BAR(B_VE + pi % NV));        // the V tile is not needed again
        }
        __syncwarp();
      };
      bool ok = warp_all(list_ready() && mbar_wait(BAR(B_X), 0, kQErrX, p.err) && mbar_wait(BAR(B_XT), 0, kQErrX, p.err));
      const int n_pairs = s_n_entries >> 1;
      if (ok && n_pairs > 0) {
        ok = warp_all(mbar_wait(BAR(B_KF), 0, kQErrYFull, p.err) && mbar_wait(BAR(B_VF), 0, kQErrYFull, p.err));
        if (ok) {
          tc_fence_after();
          issue_t(0, false);
          issue_t(0, true);
        }
      }
      for (int pi = 0; ok && pi < n_pairs; ++pi) {
        if (pi + 1 < n_pairs) {
          // T1 of the next pair as soon as this pair's T1 has been read into registers
          ok = warp_all(mbar_wait(BAR(B_T1C), pi & 1, kQErrT1C, p.err) &&
                        mbar_wait(BAR(B_KF + (pi + 1) % NK), ((pi + 1) / NK) & 1, kQErrYFull, p.err));
          if (!ok) break;
          tc_fence_after();
          issue_t(pi + 1, false);
        }
        ok = warp_all(mbar_wait(BAR(B_C), pi & 1, kQErrC, p.err));
        if (!ok) break;
        tc_fence_after();
        // [K_a; K_b] as MN-major B operand: 8-row groups 1024 B apart, 64-column slabs X_SLAB apart
        const uint32_t k_lo = desc_lo(k_slot(pi % NK), X_SLAB);
        const uint32_t acc_on = pi > 0 ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            // dS as 16-bit A operand: group g packs its 32 columns into the first 16 of its own 32 fp32 columns
            const uint32_t ao = (kk >> 1) * 32 + (kk & 1) * 8;
            mma_ts(tmem + COL_ACC, tmem + COL_T2 + ao, k_lo + ((kk * 2048) >> 4), IDESC_ACC, kk > 0 ? 1u : acc_on);  // kernel.py:163
          }
          tc_commit(BAR(B_KE + pi % NK));
        }
        __syncwarp();
        if (pi + 1 < n_pairs) {
          // overwrites dS of this pair: issued after its accumulation GEMMs, the tensor pipe runs in issue order
          ok = warp_all(mbar_wait(BAR(B_VF + (pi + 1) % NV), ((pi + 1) / NV) & 1, kQErrYFull, p.err));
          if (!ok) break;
          tc_fence_after();
          issue_t(pi + 1, true);
        }
      }
      if (ok) {
        if (elect_one()) tc_commit(BAR(B_ACC));
        __syncwarp();
      }
      if (!ok) *abortp = 1;
    }
  } else {
    // ------------------------------ compute groups ------------------------------
    const int wg = warp >> 2;                               // 0..3: columns [32 wg, +32) of the pair
    const int ent = wg >> 1, ch = wg & 1;                   // entry of the pair, column half inside its block
    const int row = tid & 127;                              // tile row == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int half = row >> 6;
    const float sc = p.scale_log2;
    const int grow = tile * 128 + row;
    float my_lse = INFINITY, my_delta = 0.f;
    constexpr int NCH = D / 16;                             // 16-byte chunks per thread (D/2 elements)
    uint4 osr[PLAIN ? 1 : NCH];                             // this thread's half row of o_s (groups 2, 3)
    if constexpr (PLAIN) {
      float2 st = p.stats[static_cast<size_t>(bh) * p.Lpad + min(grow, p.Lpad - 1)];
      if (grow < L) { my_lse = st.x; my_delta = st.y; }
    } else {
      if (grow < L) my_lse = p.lse[static_cast<size_t>(bh) * L + grow];
      if (wg >= 2) {      // requested before the wait for the tiles, used behind it
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const T*>(p.o_s) +
                                                          (static_cast<size_t>(bh) * L + min(grow, L - 1)) * D +
                                                          (wg & 1) * (D / 2));
#pragma unroll
        for (int c = 0; c < NCH; ++c) osr[c] = grow < L ? src[c] : make_uint4(0u, 0u, 0u, 0u);
      }
    }
    bool ok = !*abortp;
    if (ok) {
      // stationary tiles -> TMEM as 16-bit A operands: groups 0,1 copy the two column halves of Q, groups 2,3 of dO
      ok = mbar_wait(BAR(B_X), 0, kQErrX, p.err);
      if (ok) {
        const uint32_t src = ((wg >> 1) ? sdO : sQ) + (((wg & 1) * (D / 2)) >> 6) * X_SLAB + row * 128;
        const int chunk0 = (((wg & 1) * (D / 2)) & 63) >> 3;
        uint32_t xr[NCH * 4];
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          ld_shared_v4(src + (((chunk0 + c) ^ (row & 7)) << 4), xr[4 * c], xr[4 * c + 1], xr[4 * c + 2], xr[4 * c + 3]);
        const uint32_t dst = tmem + lane_addr + ((wg >> 1) ? COL_XDO : COL_XQ) + (wg & 1) * (D / 4);
        if constexpr (NCH * 4 == 32) tmem_st_x32(dst, xr); else tmem_st_x16(dst, xr);
        if constexpr (!PLAIN) {
          if (wg >= 2) {   // dO half row (xr, in column order) times the o_s half row
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
              const uint32_t ow[4] = {osr[c].x, osr[c].y, osr[c].z, osr[c].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 a = Elem<T>::unpack2(xr[4 * c + e]), b = Elem<T>::unpack2(ow[e]);
                d0 = fmaf(a.x, b.x, d0);
                d1 = fmaf(a.y, b.y, d1);
              }
            }
            s_delta[wg & 1][row] = d0 + d1;
          }
        }
        tmem_wait_st();
        tc_fence_before();
      }
    }
    mbar_arrive_warp(BAR(B_XT), lane);
    if constexpr (!PLAIN) {
      asm volatile("bar.sync 2, 512;\n" ::: "memory");      // every compute thread, whatever its waits returned
      my_delta = grow < L ? s_delta[0][row] + s_delta[1][row] : 0.f;
      if (wg == 2) p.stats_out[static_cast<size_t>(bh) * p.Lpad + grow] = make_float2(my_lse, my_delta);
    }
    if (ok) ok = list_ready();
    const int n_pairs = s_n_entries >> 1;
    if (trc) trc[4] = clock64() - clk0;
    const uint32_t t1 = tmem + lane_addr + COL_T1 + wg * 32, t2 = tmem + lane_addr + COL_T2 + wg * 32;
    for (int pi = 0; ok && pi < n_pairs; ++pi) {
      if (!mbar_wait(BAR(B_T1), pi & 1, kQErrT1, p.err)) { ok = false; break; }
      if (*abortp) { ok = false; break; }
      if (trc && pi == 0) trc[5] = clock64() - clk0;
      tc_fence_after();
      const int entry = ulist[2 * pi + ent];
      const bool active = (entry >> (28 + half)) & 1;
      const int valid = L - (entry & 0x0fffffff) * 64;       // keys of this block that exist (kernel.py:157)
      uint32_t sv[32];
      tmem_ld_x32(t1, sv);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive_warp(BAR(B_T1C), lane);                               // T1 may be overwritten with the next pair's scores
      float pf[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        // PLAIN (BwdParams::plain): no softmax, dS = T2 - delta on the selected blocks whatever the scores are
        float pv = PLAIN ? 1.0f : ex2q(fmaf(__uint_as_float(sv[c]), sc, -my_lse));
        if (valid < 64 && ch * 32 + c >= valid) pv = 0.f;
        pf[c] = active ? pv : 0.f;
      }
      if (!mbar_wait(BAR(B_T2), pi & 1, kQErrT2, p.err)) { ok = false; break; }
      tc_fence_after();
      uint32_t dv[32], ds[16];
      tmem_ld_x32(t2, dv);
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < 32; c += 2)
        ds[c >> 1] = Elem<T>::pack2(pf[c] * (__uint_as_float(dv[c]) - my_delta),
                                    pf[c + 1] * (__uint_as_float(dv[c + 1]) - my_delta));   // kernel.py:161
      tmem_st_x16(t2, ds);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_warp(BAR(B_C), lane);
    }
    if (ok && n_pairs > 0) ok = mbar_wait(BAR(B_ACC), 0, kQErrAcc, p.err);
    if (trc) trc[6] = clock64() - clk0;
    if (ok) ok = mbar_wait(BAR(B_X), 0, kQErrX, p.err);   // the stationary tiles (reused as staging) have landed
    if (!ok) *abortp = 1;
    asm volatile("bar.sync 1, 512;\n" ::: "memory");
    if (!*abortp) {
      tc_fence_after();
      // dQ * scale -> T (kernel.py:164), staged over the idle Q tile in the swizzled slab layout, then TMA stores;
      // rows past the end of the sequence are clipped by the copy engine. Group g converts columns [g D/4, +D/4).
      for (int c0 = wg * (D / 4); c0 < (wg + 1) * (D / 4); c0 += 16) {
        uint32_t ov[16];
        if (n_pairs > 0) {
          tmem_ld_x16(tmem + lane_addr + COL_ACC + c0, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < 16; ++c) ov[c] = 0u;
        }
#pragma unroll
        for (int q4 = 0; q4 < 2; ++q4) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            w[e] = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 2 * e]) * p.scale, __uint_as_float(ov[q4 * 8 + 2 * e + 1]) * p.scale);
          const int chunk = ((c0 & 63) >> 3) + q4;
          st_shared_v4(sQ + (c0 >> 6) * X_SLAB + row * 128 + ((chunk ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 512;\n" ::: "memory");
      if (tid == 0) {
        for (int c = 0; c < SLABS; ++c) {
          if (p.accumulate) tma_reduce_add_3d(&tmdQ, sQ + c * X_SLAB, c * 64, tile * 128, bh);
          else tma_store_3d(&tmdQ, sQ + c * X_SLAB, c * 64, tile * 128, bh);
        }
        tma_store_commit();
        tma_store_wait_read();
        if (trc) {
          unsigned long long ns;
          asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(ns));
          trc[7] = clock64() - clk0; trc[2] = static_cast<long long>(ns);
        }
      }
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

static int dq_pair_smem_bytes(int D, int topk) { return 1024 + 6 * 128 * D * 2 + (4 * topk + 4) * 4 + 16; }
constexpr int kDqStaticSmem = 2048;   // statically allocated shared memory of the kernel (barriers, delta halves)

bool sparse_bwd_dq_pair_fits(const sla_shape* s) { return dq_pair_smem_bytes(s->D, s->topk) + kDqStaticSmem <= 227 * 1024; }

template <typename T, int D, int BM, bool PLAIN>
static int launch_dq_pair(const sla_shape* s, const BwdParams& bp, float2* stats, int Lpad, cudaStream_t st) {
  const int bh = s->B * s->H;
  const int smem = dq_pair_smem_bytes(D, bp.topk);
  if (!sparse_bwd_dq_pair_fits(s)) return SLA_ERR_BAD_SHAPE;
  CUtensorMap tq, tdo, tk, tv, tdq;
  int rc;
  if ((rc = make_tmap_3d(&tq, bp.q, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tdo, bp.d_o, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tk, bp.k, s->dtype, D, s->L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tv, bp.v, s->dtype, D, s->L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tdq, bp.dq, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  tc::TcDqParams p;
  p.lut = bp.lut; p.stats = stats;
  p.o_s = bp.o_s; p.lse = bp.lse; p.stats_out = stats;
  p.err = tc_error_word();
  if (p.err == nullptr) return SLA_ERR_CUDA;
  p.trace = trace_buffer() ? trace_buffer() + 2048 : nullptr;   // behind the two per-entry timelines of the other kernels
  p.L = s->L; p.Lpad = Lpad; p.mb = bp.mb; p.topk = bp.topk; p.accumulate = bp.accumulate;
  p.scale = bp.scale; p.scale_log2 = bp.scale_log2;
  auto kern = tc::sparse_bwd_dq_pair_kernel<T, D, BM, PLAIN>;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  SLA_CUDA_OK(launch_pdl(kern, dim3(ceil_div(s->L, 128), bh), dim3(576), smem, st, tq, tdo, tk, tv, tdq, p));
  SLA_LAUNCH_OK();
  return SLA_OK;
}

// dQ of the sparse branch; `stats` ({lse, delta} per row, padded to Lpad rows per head) is written by the kernel, or
// read by it in plain mode (filled by the caller). SLA_ERR_BAD_SHAPE (nothing
// launched) when the entry list does not fit the kernel's shared memory.
int run_sparse_bwd_dq_pair(const sla_shape* s, const BwdParams& bp, void* stats, int Lpad, cudaStream_t st) {
  float2* sp = static_cast<float2*>(stats);
#define SLA_DQ2(TT, DD, BB) \
  return bp.plain ? launch_dq_pair<TT, DD, BB, true>(s, bp, sp, Lpad, st) : launch_dq_pair<TT, DD, BB, false>(s, bp, sp, Lpad, st)
#define SLA_DQ(TT)                                  \
  if (s->D == 64) {                                 \
    if (s->BLKQ == 64) SLA_DQ2(TT, 64, 64);         \
    SLA_DQ2(TT, 64, 128);                           \
  }                                                 \
  if (s->BLKQ == 64) SLA_DQ2(TT, 128, 64);          \
  SLA_DQ2(TT, 128, 128);
  if (s->dtype == SLA_BF16) { SLA_DQ(__nv_bfloat16) }
  SLA_DQ(__half)
#undef SLA_DQ2
#undef SLA_DQ
}

}  // namespace sla
