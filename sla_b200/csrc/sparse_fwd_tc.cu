// Block-sparse attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
// Same mathematics as sparse_linear_attention/kernel.py:21-82 (online softmax over the KV blocks a
// LUT row selects, exp2 domain, LSE = m + log2 l).
//
// One CTA owns a 128-row query tile: one query block when BLKQ = 128, or two adjacent 64-row query
// blocks when BLKQ = 64. In the second case the CTA walks the UNION of the two (ascending) LUT rows
// and each entry carries two bits saying which half of the tile selected it; the other half gets
// P = 0 for that entry. This keeps every MMA at M = 128 (full tensor-core rate) while the mask
// granularity stays 64 x 64.
//
// Roles (192 threads):
//   warps 0-3  softmax: thread r owns tile row r == TMEM lane r. Reads S from TMEM, keeps m, l,
//              writes P (16-bit) back over S, rescales O in TMEM only when the running maximum grew
//              by more than 2^8 since the last rescale, normalises and stores O at the end.
//   warp 4     TMA producer: Q once, then K_j / V_j tiles into a 2-stage ring (128B-swizzled).
//   warp 5     MMA issuer: S_j = Q K_j^T (SS) into one of two S buffers, O += P_j V_j (TS).
// Tensor memory (256 columns): O [0, D), S0 [D, D+64), S1 [D+64, D+128); P_j aliases S_j.
// Two CTAs fit on an SM (about 103 KB of shared memory and 256 TMEM columns each), so one CTA's softmax
// overlaps the other's MMAs.
//
// Every wait on an mbarrier is bounded; on expiry the CTA records a code in a device error word,
// stops issuing work, and leaves through the common teardown (TMEM is freed).
#include <atomic>
#include <cstddef>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace sla {
namespace tc {

struct TcFwdParams {
  const int32_t* lut;
  float* lse;
  int* err;
  int L, mb, topk, n_tiles;
  float scale_log2;
  // fused linear branch (core.py:90,95-100); feature < 0: sparse branch only
  int feature;             // sla_feature, or -1
  int plain;               // no softmax: P = S (scale 1), O is left unnormalised and `lse` receives the row sums of P
  int store_os;            // also store the sparse branch output through tmOs
  const void* lin_state;   // [BH][2*D*D + D] T: H, z, H W^T
  const void* wbits;       // [D*D + D] T: W, bias
  void* gather[8];         // further destinations of the output tile (FwdParams::gather_dst)
  int n_gather;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

enum : int {
  kErrQ = 101, kErrKFull = 102, kErrVFull = 103, kErrEmpty = 104, kErrSFull = 105, kErrPFull = 106,
  kErrPvDone = 107, kErrDrain = 108, kErrHw = 109, kErrPhi = 110, kErrLin = 111
};

template <typename T, int D, int BM>
__global__ void __launch_bounds__(192, 2)
sparse_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                     const __grid_constant__ CUtensorMap tmOs, const __grid_constant__ CUtensorMap tmHW,
                     TcFwdParams p) {
  constexpr int SLABS = D / 64;                 // 64-column (128-byte) slabs per row
  constexpr int Q_SLAB = 128 * 128;             // bytes of one Q slab (128 rows x 128 B)
  constexpr int KV_SLAB = 64 * 128;             // bytes of one K/V slab (64 rows x 128 B)
  constexpr int Q_BYTES = SLABS * Q_SLAB;
  constexpr int KV_BYTES = SLABS * KV_SLAB;
  constexpr int FMT = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_S = idesc_f16(FMT, 128, 64, 0, 0);
  constexpr uint32_t IDESC_PV = idesc_f16(FMT, 128, D, 0, 1);
  constexpr uint32_t TMEM_COLS = 256;
  constexpr int COL_O = 0, COL_S = D;
  constexpr float kRescaleThreshold = 8.0f;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[18];
  __shared__ uint32_t s_zp[D / 2];   // z of the linear state, pairs of T
  __shared__ float s_bias[D];
  __shared__ float s_rden[128];      // 1 / den of the linear branch per tile row
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_n_entries;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  pdl_entry();

  // 1024-byte aligned tile area (required by the 128B swizzle pattern)
  const uint32_t raw_a = smem_u32(smem_raw);
  const uint32_t base_a = (raw_a + 1023u) & ~1023u;
  uint8_t* base_p = smem_raw + (base_a - raw_a);
  const uint32_t sQ = base_a;
  const uint32_t sK0 = sQ + Q_BYTES;            // stage s at sK0 + s * KV_BYTES
  const uint32_t sV0 = sK0 + 2 * KV_BYTES;
  int32_t* ulist = reinterpret_cast<int32_t*>(base_p + Q_BYTES + 4 * KV_BYTES);

  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // 0 q_full | 1,2 k_full | 3,4 v_full | 5,6 v_empty | 7,8 s_full | 9,10 p_full | 11,12 pv_done | 13,14 k_empty
  // 15 hw_full (H W^T landed in the K stages) | 16 phi_full (phi(q) written over Q) | 17 lin_done
  // pv_done alternates between two barriers (entry j -> barrier j & 1). A parity wait only tells
  // neighbouring phases apart, and a softmax thread that skipped the rescale for a while knows no more
  // than "P.V of entry j-2 is complete" when S_j arrives; with two barriers that is enough.
  constexpr int B_Q = 0, B_K = 1, B_V = 3, B_E = 5, B_S = 7, B_P = 9, B_PV = 11, B_KE = 13;
  constexpr int B_HW = 15, B_PHI = 16, B_LIN = 17;
  const bool fused = p.feature >= 0;

  if (tid == 0) {
    s_abort = *reinterpret_cast<volatile int*>(p.err) != 0;  // an earlier CTA failed: do no work
    mbar_init(BAR(B_Q), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(B_K + s), 1);
      mbar_init(BAR(B_V + s), 1);
      mbar_init(BAR(B_E + s), 1);
      mbar_init(BAR(B_KE + s), 1);
      mbar_init(BAR(B_S + s), 1);
      mbar_init(BAR(B_P + s), 128);
    }
    mbar_init(BAR(B_PV), 1);
    mbar_init(BAR(B_PV + 1), 1);
    mbar_init(BAR(B_HW), 1);
    mbar_init(BAR(B_PHI), 128);
    mbar_init(BAR(B_LIN), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 4) {
    if (lane == 0) {
      prefetch_tmap(&tmQ);
      prefetch_tmap(&tmK);
      prefetch_tmap(&tmV);
      prefetch_tmap(&tmO);
      if (fused) prefetch_tmap(&tmHW);
    }
    // Entry list: block index | bit 28 (upper half of the tile selects it) | bit 29 (lower half).
    // The LUT rows are first copied to shared memory with coalesced loads; a serial merge straight
    // from global memory would cost one DRAM/L2 round trip per element.
    int32_t* raw = ulist + 2 * p.topk;
    const int rows = BM == 128 ? 1 : ((2 * tile + 1 < p.mb) ? 2 : 1);
    const int32_t* src = p.lut + (static_cast<size_t>(bh) * p.mb + (BM == 128 ? tile : 2 * tile)) * p.topk;
    for (int i = lane; i < rows * p.topk; i += 32) raw[i] = src[i];
    __syncwarp();
    int n;
    if (BM == 128) {
      for (int i = lane; i < p.topk; i += 32) ulist[i] = raw[i] | (3 << 28);
      n = p.topk;
      __syncwarp();
    } else {
      n = warp_union_lists(raw, p.topk, raw + p.topk, rows == 2 ? p.topk : 0, ulist, 1 << 28, 2 << 28, lane);
    }
    if (lane == 0) s_n_entries = n;
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  if (fused && tid < D) {
    const T* rec = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);
    if (tid < D / 2) s_zp[tid] = reinterpret_cast<const uint32_t*>(rec + D * D)[tid];
    s_bias[tid] = Elem<T>::to_f(static_cast<const T*>(p.wbits)[D * D + tid]);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const int n_ent = s_n_entries;
  volatile int* abortp = &s_abort;

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && !*abortp) {
      mbar_expect_tx(BAR(B_Q), Q_BYTES);
      for (int c = 0; c < SLABS; ++c) tma_load_3d(sQ + c * Q_SLAB, &tmQ, BAR(B_Q), c * 64, tile * 128, bh);
      // K tiles run one entry ahead of V tiles: a K stage is free as soon as S_j has been computed,
      // a V stage only after P_j V_j.
      int issued_k = 0, issued_v = 0;
      // test hook: with the control block's drop_first_k_tile set, CTA (0,0) never requests its first K tile, so the
      // waits behind it run out and the CTA leaves through the abort path
      const bool drop_k0 = tile == 0 && bh == 0 && reinterpret_cast<volatile TcControl*>(p.err)->drop_first_k_tile != 0;
      for (int t = 0; t <= n_ent; ++t) {
        if (t < n_ent && !(drop_k0 && t == 0)) {
          const int s = t & 1;
          if (t >= 2 && !mbar_wait(BAR(B_KE + s), ((t >> 1) - 1) & 1, kErrEmpty, p.err)) { *abortp = 1; break; }
          if (*abortp) break;
          const int row0 = (ulist[t] & 0x0fffffff) * 64;
          mbar_expect_tx(BAR(B_K + s), KV_BYTES);
          for (int c = 0; c < SLABS; ++c) tma_load_3d(sK0 + s * KV_BYTES + c * KV_SLAB, &tmK, BAR(B_K + s), c * 64, row0, bh);
          issued_k = t + 1;
        }
        if (t >= 1) {
          const int j = t - 1, s = j & 1;
          if (j >= 2 && !mbar_wait(BAR(B_E + s), ((j >> 1) - 1) & 1, kErrEmpty, p.err)) { *abortp = 1; break; }
          if (*abortp) break;
          const int row0 = (ulist[j] & 0x0fffffff) * 64;
          mbar_expect_tx(BAR(B_V + s), KV_BYTES);
          for (int c = 0; c < SLABS; ++c) tma_load_3d(sV0 + s * KV_BYTES + c * KV_SLAB, &tmV, BAR(B_V + s), c * 64, row0, bh);
          issued_v = j + 1;
        }
      }
      if (fused && !*abortp) {
        // H W^T of this head (D x D) goes into the two K stages once the last S GEMMs have read them
        bool free_k = true;
        for (int j = max(0, n_ent - 2); free_k && j < n_ent; ++j)
          free_k = mbar_wait(BAR(B_KE + (j & 1)), (j >> 1) & 1, kErrEmpty, p.err);
        if (!free_k) *abortp = 1;
        else {
          mbar_expect_tx(BAR(B_HW), D * D * 2);
          for (int r = 0; r < D / 64; ++r)
            for (int c = 0; c < SLABS; ++c)
              tma_load_3d(sK0 + r * KV_BYTES + c * KV_SLAB, &tmHW, BAR(B_HW), c * 64, r * 64, bh);
          if (*abortp) mbar_wait_drain(BAR(B_HW), 0, p.err);
        }
      }
      if (*abortp) {
        // let the copies already in flight land before the CTA's shared memory goes away
        mbar_wait_drain(BAR(B_Q), 0, p.err);
        for (int j = max(0, issued_k - 2); j < issued_k; ++j)
          if (!(drop_k0 && j == 0)) mbar_wait_drain(BAR(B_K + (j & 1)), (j >> 1) & 1, p.err);
        for (int j = max(0, issued_v - 2); j < issued_v; ++j) mbar_wait_drain(BAR(B_V + (j & 1)), (j >> 1) & 1, p.err);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    // All 32 lanes run the control flow; one elected lane issues the tcgen05 instructions.
    if (!*abortp) {
      const uint32_t q_lo = desc_lo(sQ, 16);
      auto issue_s = [&](int j) {
        const uint32_t k_lo = desc_lo(sK0 + (j & 1) * KV_BYTES, 16);
        const uint32_t d = tmem + COL_S + (j & 1) * 64;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)   // k-step: 32 bytes further inside the swizzle atom, next slab every 4 steps
            mma_ss(d, q_lo + (((kk >> 2) * Q_SLAB + (kk & 3) * 32) >> 4), k_lo + (((kk >> 2) * KV_SLAB + (kk & 3) * 32) >> 4),
                   IDESC_S, kk > 0 ? 1u : 0u);
          tc_commit(BAR(B_S + (j & 1)));
          tc_commit(BAR(B_KE + (j & 1)));
        }
        __syncwarp();
      };
      bool ok = warp_all(mbar_wait(BAR(B_Q), 0, kErrQ, p.err) && mbar_wait(BAR(B_K), 0, kErrKFull, p.err));
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_ent; ++j) {
        if (j + 1 < n_ent) {
          ok = warp_all(mbar_wait(BAR(B_K + ((j + 1) & 1)), ((j + 1) >> 1) & 1, kErrKFull, p.err));
          if (!ok) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        ok = warp_all(mbar_wait(BAR(B_P + (j & 1)), (j >> 1) & 1, kErrPFull, p.err) &&
                      mbar_wait(BAR(B_V + (j & 1)), (j >> 1) & 1, kErrVFull, p.err));
        if (!ok) break;
        tc_fence_after();
        // B = V_j rows [16 kk, +16): MN-major, 8-row groups 1024 B apart, 64-column slabs KV_SLAB apart
        const uint32_t v_lo = desc_lo(sV0 + (j & 1) * KV_BYTES, KV_SLAB);
        const uint32_t pa = tmem + COL_S + (j & 1) * 64;   // P_j: 16-bit pairs packed over S_j
        const uint32_t acc_on = j > 0 ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ts(tmem + COL_O, pa + kk * 8, v_lo + ((kk * 2048) >> 4), IDESC_PV, kk > 0 ? 1u : acc_on);
          tc_commit(BAR(B_E + (j & 1)));
          tc_commit(BAR(B_PV + (j & 1)));
        }
        __syncwarp();
      }
      if (ok && fused) {
        // read-out of the linear branch: LIN[128 x D] = phi(Q) (H W^T) into the (now idle) S columns
        ok = warp_all(mbar_wait(BAR(B_HW), 0, kErrHw, p.err) && mbar_wait(BAR(B_PHI), 0, kErrPhi, p.err));
        if (ok) {
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t hw_lo = desc_lo(sK0 + (kk >> 2) * KV_BYTES, KV_SLAB) + (((kk & 3) * 2048) >> 4);
              mma_ss(tmem + COL_S, q_lo + (((kk >> 2) * Q_SLAB + (kk & 3) * 32) >> 4), hw_lo, IDESC_PV, kk > 0 ? 1u : 0u);
            }
            tc_commit(BAR(B_LIN));
          }
          __syncwarp();
        }
      }
      if (!ok) *abortp = 1;
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int row = tid;                                   // tile row == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const int half = BM == 128 ? 0 : (warp >> 1);
    const float sc = p.scale_log2;
    float m_true = -INFINITY, m_used = -INFINITY, l = 0.f;
    bool ok = !*abortp;
    for (int j = 0; ok && j < n_ent; ++j) {
      const int b = j & 1;
      if (!mbar_wait(BAR(B_S + b), (j >> 1) & 1, kErrSFull, p.err)) { ok = false; break; }
      if (*abortp) { ok = false; break; }
      tc_fence_after();
      const int entry = ulist[j];
      const bool active = BM == 128 || ((entry >> (28 + half)) & 1);
      const uint32_t s_addr = tmem + lane_addr + COL_S + b * 64;
      uint32_t pk[32];
      if (active) {
        uint32_t sv[64];
        tmem_ld_x64(s_addr, sv);
        tmem_wait_ld();
        if (p.plain) {
          // linear kernel over the selected blocks: keys past the end are zero rows, so S is 0 there
          float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            pk[c >> 1] = Elem<T>::pack2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
            const float2 pr = Elem<T>::unpack2(pk[c >> 1]);      // the sum uses what the P.V GEMM sees
            rs0 += pr.x; rs1 += pr.y;
          }
          l += rs0 + rs1;
          tmem_st_x32(s_addr, pk);
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(BAR(B_P + b));
          continue;
        }
        const int valid = L - (entry & 0x0fffffff) * 64;     // keys of this block that exist (kernel.py:57)
        // row maximum of the raw scores (the scale is positive, so it commutes with max); four
        // independent chains keep the dependent-issue latency off the critical path
        if (valid < 64) {                                       // kernel.py:61-62: keys past the end
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (c >= valid) sv[c] = 0xff800000u;                // -inf
        }
        float mx0 = __uint_as_float(sv[0]), mx1 = __uint_as_float(sv[1]);
        float mx2 = __uint_as_float(sv[2]), mx3 = __uint_as_float(sv[3]);
#pragma unroll
        for (int c = 4; c < 64; c += 4) {
          mx0 = fmaxf(mx0, __uint_as_float(sv[c]));
          mx1 = fmaxf(mx1, __uint_as_float(sv[c + 1]));
          mx2 = fmaxf(mx2, __uint_as_float(sv[c + 2]));
          mx3 = fmaxf(mx3, __uint_as_float(sv[c + 3]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sc;
        m_true = fmaxf(m_true, mx);
        const bool need = m_true > m_used + kRescaleThreshold;   // also true on the first active block
        if (j > 0 && __any_sync(0xffffffffu, need)) {
          // O holds sum_{j' < j} P V with the old reference maximum: wait for PV_{j-1}, then scale it
          if (!mbar_wait(BAR(B_PV + ((j - 1) & 1)), ((j - 1) >> 1) & 1, kErrPvDone, p.err)) { ok = false; break; }
          tc_fence_after();
          const float alpha = need ? ex2(m_used - m_true) : 1.0f;
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t ov[32];
            tmem_ld_x32(tmem + lane_addr + COL_O + c0, ov);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * alpha);
            tmem_st_x32(tmem + lane_addr + COL_O + c0, ov);
          }
        }
        if (need) {
          l *= ex2(m_used - m_true);
          m_used = m_true;
        }
        float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
        const float neg_m = -m_used;
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          float p0 = ex2(fmaf(__uint_as_float(sv[c]), sc, neg_m));          // exp2(s * scale * log2e - m)
          float p1 = ex2(fmaf(__uint_as_float(sv[c + 1]), sc, neg_m));
          float p2 = ex2(fmaf(__uint_as_float(sv[c + 2]), sc, neg_m));
          float p3 = ex2(fmaf(__uint_as_float(sv[c + 3]), sc, neg_m));
          rs0 += p0; rs1 += p1; rs2 += p2; rs3 += p3;
          pk[c >> 1] = Elem<T>::pack2(p0, p1);              // P rounded to T before P.V (kernel.py:71)
          pk[(c >> 1) + 1] = Elem<T>::pack2(p2, p3);
        }
        const float rs = (rs0 + rs1) + (rs2 + rs3);
        l += rs;
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = 0u;
      }
      tmem_st_x32(s_addr, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(BAR(B_P + b));
    }
    if (ok && n_ent > 0) ok = mbar_wait(BAR(B_PV + ((n_ent - 1) & 1)), ((n_ent - 1) >> 1) & 1, kErrPvDone, p.err);
    if (!ok) *abortp = 1;
    // all four softmax warps agree on whether the tile is good before touching the Q buffer
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    if (!*abortp) {
      tc_fence_after();
      const float inv = p.plain ? 1.0f : 1.0f / l;
      const int grow = tile * 128 + row;
      if (grow < L) p.lse[static_cast<size_t>(bh) * L + grow] = p.plain ? l : m_used + log2f(l);   // kernel.py:81
      // 16-byte chunk ch of this thread's row inside a 128-row tile at `tile_base` (128B-swizzled slabs)
      auto chunk_addr = [&](uint32_t tile_base, int ch) {
        return tile_base + (ch >> 3) * Q_SLAB + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
      };
      // The staged output tile once more to every gather destination, with plain stores (a destination may be
      // another GPU's memory: no TMA, no multicast). Sixteen-byte chunks of a row go to consecutive lanes, so a
      // warp writes whole rows; rows past the end of the sequence are skipped.
      auto gather_store = [&](uint32_t tile_base) {
        constexpr int CH = D / 8;
        for (int idx = tid; idx < 128 * CH; idx += 128) {
          const int r = idx / CH, ch = idx % CH;
          const int gr = tile * 128 + r;
          if (gr < L) {
            uint32_t w0, w1, w2, w3;
            ld_shared_v4(tile_base + (ch >> 3) * Q_SLAB + r * 128 + (((ch & 7) ^ (r & 7)) << 4), w0, w1, w2, w3);
            const size_t off = ((static_cast<size_t>(bh) * L + gr) * D + ch * 8) * sizeof(T);
            for (int g = 0; g < p.n_gather; ++g)
              *reinterpret_cast<uint4*>(static_cast<char*>(p.gather[g]) + off) = make_uint4(w0, w1, w2, w3);
          }
        }
      };
      // O / l -> T for columns [c0, c0 + 32), written to the staging tile
      auto stage_os = [&](uint32_t tile_base, int c0) {
        uint32_t ov[32];
        tmem_ld_x32(tmem + lane_addr + COL_O + c0, ov);
        tmem_wait_ld();
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t w0 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 0]) * inv, __uint_as_float(ov[q4 * 8 + 1]) * inv);
          uint32_t w1 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 2]) * inv, __uint_as_float(ov[q4 * 8 + 3]) * inv);
          uint32_t w2 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 4]) * inv, __uint_as_float(ov[q4 * 8 + 5]) * inv);
          uint32_t w3 = Elem<T>::pack2(__uint_as_float(ov[q4 * 8 + 6]) * inv, __uint_as_float(ov[q4 * 8 + 7]) * inv);
          st_shared_v4(chunk_addr(tile_base, (c0 >> 3) + q4), w0, w1, w2, w3);
        }
      };
      if (!fused) {
        // staged in the (idle) Q buffer, then one TMA store per slab; rows past the end of the
        // sequence are clipped by the copy engine
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) stage_os(sQ, c0);
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (tid == 0) {
          for (int c = 0; c < SLABS; ++c) tma_store_3d(&tmO, sQ + c * Q_SLAB, c * 64, tile * 128, bh);
          tma_store_commit();
        }
        if (p.n_gather > 0) gather_store(sQ);
        if (tid == 0) tma_store_wait_read();
      } else {
        // ---- phi(q) over the Q tile in place (core.py:90) and 1 / den per row (core.py:95) ----
        // Eight threads per row (thread = 16-byte chunk `pc` of every 64-column slab), sixteen rows per pass, eight
        // passes: the rows of a thread are independent, which hides the latency a one-thread-per-row loop exposes.
        {
          const int pc = tid & 7, rg = tid >> 3;
          uint32_t zz[SLABS][4];
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl)
#pragma unroll
            for (int i = 0; i < 4; ++i) zz[sl][i] = s_zp[(sl * 8 + pc) * 4 + i];
#pragma unroll 4
          for (int it = 0; it < 8; ++it) {
            const int r = rg + 16 * it;
            const uint32_t a0 = sQ + r * 128 + ((pc ^ (r & 7)) << 4);
            float f[SLABS][8];
#pragma unroll
            for (int sl = 0; sl < SLABS; ++sl) {
              uint32_t w0, w1, w2, w3;
              ld_shared_v4(a0 + sl * Q_SLAB, w0, w1, w2, w3);
              const float2 a = Elem<T>::unpack2(w0), b2 = Elem<T>::unpack2(w1), c = Elem<T>::unpack2(w2), d = Elem<T>::unpack2(w3);
              f[sl][0] = a.x; f[sl][1] = a.y; f[sl][2] = b2.x; f[sl][3] = b2.y;
              f[sl][4] = c.x; f[sl][5] = c.y; f[sl][6] = d.x; f[sl][7] = d.y;
            }
            if (p.feature == SLA_PHI_SOFTMAX) {
              float mx = -INFINITY;
#pragma unroll
              for (int sl = 0; sl < SLABS; ++sl)
#pragma unroll
                for (int i = 0; i < 8; ++i) mx = fmaxf(mx, f[sl][i]);
#pragma unroll
              for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
              const float neg_mx = -mx * kLog2e;
              float es = 0.f;
#pragma unroll
              for (int sl = 0; sl < SLABS; ++sl)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  f[sl][i] = ex2(fmaf(f[sl][i], kLog2e, neg_mx));
                  es += f[sl][i];
                }
#pragma unroll
              for (int o = 1; o < 8; o <<= 1) es += __shfl_xor_sync(0xffffffffu, es, o);
              const float inv_s = 1.f / es;
#pragma unroll
              for (int sl = 0; sl < SLABS; ++sl)
#pragma unroll
                for (int i = 0; i < 8; ++i) f[sl][i] *= inv_s;
            } else {
#pragma unroll
              for (int sl = 0; sl < SLABS; ++sl)
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float x = f[sl][i];
                  if (p.feature == SLA_PHI_RELU) f[sl][i] = fmaxf(x, 0.f);
                  else f[sl][i] = x > 0.f ? x + 1.f : __expf(x);      // elu(x) + 1
                }
            }
            float dsum = 0.f;        // sum_d round(phi_d * z_d), core.py:95
#pragma unroll
            for (int sl = 0; sl < SLABS; ++sl) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                w[i] = Elem<T>::pack2(f[sl][2 * i], f[sl][2 * i + 1]);
                const float2 pz = Elem<T>::unpack2(Elem<T>::mul2(w[i], zz[sl][i]));   // each product rounded to T
                dsum += pz.x + pz.y;
              }
              st_shared_v4(a0 + sl * Q_SLAB, w[0], w[1], w[2], w[3]);
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
            if (pc == 0) s_rden[r] = 1.f / round_to<T>(1e-5f + round_to<T>(dsum));
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(BAR(B_PHI));
        asm volatile("bar.sync 1, 128;\n" ::: "memory");     // s_rden of this thread's row was written by another thread
        const float rden = s_rden[row];
        // ---- while the read-out GEMM runs: the sparse branch's own output, staged in the idle V stages ----
        if (p.store_os) {
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) stage_os(sV0, c0);
        }
        const bool lin_ok = mbar_wait(BAR(B_LIN), 0, kErrLin, p.err);
        if (lin_ok) {
          tc_fence_after();
          // o = o_s + round(lin / den + bias) (core.py:96-100), staged over phi(q)
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t ov[32], lv[32];
            tmem_ld_x32(tmem + lane_addr + COL_O + c0, ov);
            tmem_ld_x32(tmem + lane_addr + COL_S + c0, lv);
            tmem_wait_ld();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int c = q4 * 8 + 2 * i;
                const uint32_t os2 = Elem<T>::pack2(__uint_as_float(ov[c]) * inv, __uint_as_float(ov[c + 1]) * inv);
                const uint32_t lin2 = Elem<T>::pack2(fmaf(__uint_as_float(lv[c]), rden, s_bias[c0 + c]),
                                                     fmaf(__uint_as_float(lv[c + 1]), rden, s_bias[c0 + c + 1]));
                w[i] = Elem<T>::add2(os2, lin2);
              }
              st_shared_v4(chunk_addr(sQ, (c0 >> 3) + q4), w[0], w[1], w[2], w[3]);
            }
          }
        } else {
          *abortp = 1;
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (tid == 0 && !*abortp) {
          if (p.store_os)
            for (int c = 0; c < SLABS; ++c) tma_store_3d(&tmOs, sV0 + c * Q_SLAB, c * 64, tile * 128, bh);
          for (int c = 0; c < SLABS; ++c) tma_store_3d(&tmO, sQ + c * Q_SLAB, c * 64, tile * 128, bh);
          tma_store_commit();
        }
        if (p.n_gather > 0 && !*abortp) gather_store(sQ);
        if (tid == 0) tma_store_wait_read();
      }
    }
  }
  // ------------------------------ teardown ------------------------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace tc

// The control block lives in this translation unit; other tcgen05 kernels receive its address.
__device__ tc::TcControl g_tc_control = {0, 0, tc::kDefaultWaitLimitNs};

int* tc_error_word() {
  static std::atomic<int*> ptrs[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  int* known = ptrs[dev].load(std::memory_order_acquire);
  if (known == nullptr) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_tc_control);
    if (e != cudaSuccess) {
      set_last_cuda_error(e);
      return nullptr;
    }
    known = static_cast<int*>(p);
    ptrs[dev].store(known, std::memory_order_release);
  }
  return known;
}

int set_tc_wait_limit(unsigned long long ns) {
  SLA_CUDA_OK(cudaMemcpyToSymbol(g_tc_control, &ns, sizeof(ns), offsetof(tc::TcControl, wait_limit_ns)));
  return SLA_OK;
}
int set_tc_drop_first_k_tile(int on) {
  SLA_CUDA_OK(cudaMemcpyToSymbol(g_tc_control, &on, sizeof(on), offsetof(tc::TcControl, drop_first_k_tile)));
  return SLA_OK;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
      if (e != cudaSuccess) set_last_cuda_error(e);
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int dtype, int D, int L, int BH, int box_rows) {
  return make_tmap_rows(out, base, dtype, D, L, BH, size_t(L) * D * 2, box_rows);
}

// (BH, L, D) 16-bit rows of D contiguous elements, consecutive heads `head_stride_bytes` apart
int make_tmap_rows(CUtensorMap* out, const void* base, int dtype, int D, int L, int BH, size_t head_stride_bytes,
                   int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return SLA_ERR_CUDA;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(L), static_cast<cuuint64_t>(BH)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(head_stride_bytes)};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dtype == SLA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue);
    return SLA_ERR_CUDA;
  }
  return SLA_OK;
}

int make_tmap_3d_u8(CUtensorMap* out, const void* base, int row_bytes, int L, int BH, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return SLA_ERR_CUDA;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(L), static_cast<cuuint64_t>(BH)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(L) * row_bytes};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(row_bytes), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue);
    return SLA_ERR_CUDA;
  }
  return SLA_OK;
}

constexpr int kFwdStaticSmem = 2 * 1024;   // statically allocated shared memory of the kernel (barriers, z, bias, 1/den)
static int fwd_tc_smem_bytes(int D, int topk) { return 1024 + 128 * D * 2 + 4 * 64 * D * 2 + 4 * topk * 4 + 16; }
bool sparse_fwd_tc_fits(const sla_shape* s) { return fwd_tc_smem_bytes(s->D, s->topk) + kFwdStaticSmem <= 227 * 1024; }

template <typename T, int D, int BM>
static int launch_tc(const sla_shape* s, const FwdParams& fp, cudaStream_t st) {
  const int bh = s->B * s->H;
  CUtensorMap tq, tk, tv, to, tos, thw;
  int rc;
  if ((rc = make_tmap_3d(&tq, fp.q, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tk, fp.k, s->dtype, D, s->L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tv, fp.v, s->dtype, D, s->L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&to, fp.o, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  tc::TcFwdParams p;
  const bool fused = fp.lin_state != nullptr;
  tos = to; thw = to;
  p.feature = fused ? s->feature_map : -1;
  p.store_os = fused && fp.o_s != nullptr && fp.o_s != fp.o;
  p.lin_state = fp.lin_state; p.wbits = fp.wbits;
  p.plain = fp.plain;
  p.n_gather = fp.n_gather;
  for (int g = 0; g < 8; ++g) p.gather[g] = g < fp.n_gather ? fp.gather_dst[g] : nullptr;
  if (p.store_os && (rc = make_tmap_3d(&tos, fp.o_s, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if (fused) {
    // H W^T sits behind H and z in each head's record: D rows of D elements, records 2*D*D + D apart
    const char* hw = static_cast<const char*>(fp.lin_state) + (size_t(D) * D + D) * 2;
    if ((rc = make_tmap_rows(&thw, hw, s->dtype, D, D, bh, size_t(2 * D * D + D) * 2, 64)) != SLA_OK) return rc;
  }
  p.err = tc_error_word();
  if (p.err == nullptr) return SLA_ERR_CUDA;
  p.lut = fp.lut; p.lse = fp.lse; p.L = s->L; p.mb = fp.mb; p.topk = fp.topk;
  p.n_tiles = ceil_div(s->L, 128);
  p.scale_log2 = fp.scale_log2;
  auto kern = tc::sparse_fwd_tc_kernel<T, D, BM>;
  // Up to 113 KB two CTAs share an SM; a longer entry list (top-k above about 1000 at D = 128) takes the SM alone.
  // SLA_ERR_BAD_SHAPE (nothing launched) when the list does not fit at all: the caller picks another path.
  const int smem = fwd_tc_smem_bytes(D, fp.topk);
  if (!sparse_fwd_tc_fits(s)) return SLA_ERR_BAD_SHAPE;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  SLA_CUDA_OK(launch_pdl<false>(kern, dim3(p.n_tiles, bh), dim3(192), smem, st, tq, tk, tv, to, tos, thw, p));
  SLA_LAUNCH_OK();
  return SLA_OK;
}

int run_sparse_fwd_tc(const sla_shape* s, const FwdParams& p, cudaStream_t st) {
#define SLA_TC(TT)                                                                     \
  if (s->D == 64) return s->BLKQ == 64 ? launch_tc<TT, 64, 64>(s, p, st) : launch_tc<TT, 64, 128>(s, p, st); \
  return s->BLKQ == 64 ? launch_tc<TT, 128, 64>(s, p, st) : launch_tc<TT, 128, 128>(s, p, st);
  if (s->dtype == SLA_BF16) { SLA_TC(__nv_bfloat16) }
  SLA_TC(__half)
#undef SLA_TC
}

int read_tc_error(int* out, bool clear) {
  int v = 0;
  SLA_CUDA_OK(cudaMemcpyFromSymbol(&v, g_tc_control, sizeof(int)));
  if (clear && v != 0) {
    int z = 0;
    SLA_CUDA_OK(cudaMemcpyToSymbol(g_tc_control, &z, sizeof(int)));
  }
  *out = v;
  return SLA_OK;
}

}  // namespace sla
