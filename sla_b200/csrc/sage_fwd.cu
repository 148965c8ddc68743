// SageSLA quantized forward (SageSLA/core.py:75-163): the sparse branch with INT8 Q.K^T and FP8 (e4m3)
// P.V on tcgen05, then the same linear branch and proj_l as the 16-bit path.
//
// The reference delegates the quantized arithmetic to the third-party package spas_sage_attn (not part of
// the reference tree); what its call sites fix is reproduced here: K is smoothed by its per-head mean
// before quantization (SageSLA/core.py:102,108), Q is quantized per 128-row block and K per 64-row block
// with one fp32 scale each (core.py:105-108), V is stored as e4m3 with one fp32 scale per (batch, head,
// channel) (core.py:127-129), scores use scale = D^-0.5 (core.py:110), no causal mask, no PV skipping
// (pvthreshold = 1e6, core.py:136). The recipe itself (symmetric abs-max scales, P scaled by 256 before
// the e4m3 rounding) is this library's own.
//
// Kernel structure = sparse_fwd_tc.cu with BLKQ = 128: S = Q8 K8^T by kind::i8 (s32 accumulators in
// TMEM), softmax in fp32 on S * sq * sk * scale * log2e, P written back to TMEM as e4m3 and multiplied
// with the e4m3 V tile (MN-major B operand) by kind::f8f6f4.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"
#include "workspace.h"

namespace sla {
namespace tc {

struct SageParams {
  const int32_t* lut;
  const float *qscale, *kscale, *vscale;   // [BH][MB], [BH][NB], [BH][D]
  float* lse;
  int* err;
  int L, mb, nb, topk;
  float scale_log2;
  // fused linear read-out + proj_l + sum in the epilogue (SageSLA/core.py:148-158); feature < 0: sparse branch only
  int feature;
  const void* lin_state;   // [BH][2*D*D + D] T: H, z, H W^T
  const void* wbits;       // [D*D + D] T: W, bias
  void* gather[8];         // further destinations of the output tile, written with plain stores (peers' memory allowed)
  int n_gather;
};

__device__ __forceinline__ float ex2s(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// four fp32 -> four e4m3 bytes, element 0 in the lowest byte
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

enum : int { kSErrQ = 301, kSErrK = 302, kSErrV = 303, kSErrEmpty = 304, kSErrS = 305, kSErrP = 306,
             kSErrPv = 307, kSErrDrain = 308, kSErrQ16 = 309, kSErrHw = 310, kSErrPhi = 311, kSErrLin = 312 };

// P is multiplied by 2^kPShift before rounding to e4m3 (largest finite value 448). The running maximum used
// in the exponent may lag the true one by up to kLazy (log2 units) before O is rescaled, so P <= 2^kLazy and
// P * 2^kPShift <= 256. Without the lag nearly every entry has some row of the warp whose maximum grew, and
// each such rescale has to wait for the previous P.V GEMM: the softmax and the tensor pipe then alternate
// instead of overlapping.
constexpr float kPShift = 5.0f;
constexpr float kLazy = 3.0f;

// Rows of the 8-bit tensors are one 128-byte swizzle atom whatever D is: with D = 64 the upper half of a row is
// padding that no GEMM reads (the S GEMM takes D / 32 K-steps inside the atom, the P.V GEMM has N = D).
template <typename T, int D>
__global__ void __launch_bounds__(192, 2)
sage_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                   const __grid_constant__ CUtensorMap tmQ16, const __grid_constant__ CUtensorMap tmHW, SageParams p) {
  constexpr int DP = 128;                                      // bytes per row of the 8-bit tensors
  constexpr int Q_BYTES = 128 * DP, KV_BYTES = 64 * DP;        // 8-bit tiles
  constexpr int O_SLAB = 128 * 128, NSLAB = D / 64;            // 16-bit output staging, slabs of 64 columns
  constexpr int NS = 4;                                        // ring stages (K and V each)
  constexpr uint32_t IDESC_S = idesc_i8(128, 64);
  constexpr uint32_t IDESC_PV = idesc_e4m3(128, D, 1);     // N = D: the first D bytes of each V8 row
  constexpr int FMT16 = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_LIN = idesc_f16(FMT16, 128, D, 0, 1);   // phi(Q) (K-major) x H W^T (MN-major), 16-bit
  constexpr int Q16_SLAB = 128 * 128, HW_STAGE = 64 * D * 2, HW_SLAB = 64 * 128;
  constexpr uint32_t TMEM_COLS = 256;
  constexpr int COL_O = 0, COL_S = DP;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[4 * NS + 11];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_vscale[D];
  __shared__ uint32_t s_zp[D / 2];   // z of the linear state, pairs of T
  __shared__ float s_bias[D];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  const uint32_t raw_a = smem_u32(smem_raw);
  const uint32_t base_a = (raw_a + 1023u) & ~1023u;
  uint8_t* base_p = smem_raw + (base_a - raw_a);
  const uint32_t sO = base_a;                        // 32 KB output staging (also holds Q8 in its first 16 KB)
  const uint32_t sQ = base_a;
  const uint32_t sK0 = sO + 2 * O_SLAB;
  const uint32_t sV0 = sK0 + NS * KV_BYTES;
  int32_t* ulist = reinterpret_cast<int32_t*>(base_p + 2 * O_SLAB + 2 * NS * KV_BYTES);
  float* sk_list = reinterpret_cast<float*>(ulist + p.topk);

  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // q_full | k_full[NS] | v_full[NS] | k_empty[NS] | v_empty[NS] | s_full[2] | p_full[2] | pv_done[2]
  // (entry j signals pv_done[j & 1]: a parity wait only tells neighbouring phases apart)
  constexpr int B_Q = 0, B_K = 1, B_V = 1 + NS, B_KE = 1 + 2 * NS, B_VE = 1 + 3 * NS, B_S = 1 + 4 * NS,
                B_P = 3 + 4 * NS, B_PV = 5 + 4 * NS;
  // fused read-out: 16-bit Q tile landed in the K ring | H W^T landed in the V ring | phi(q) written | GEMM done
  constexpr int B_Q16 = 7 + 4 * NS, B_HW = 8 + 4 * NS, B_PHI = 9 + 4 * NS, B_LIN = 10 + 4 * NS;
  const bool fused = p.feature >= 0;
  const uint32_t sQ16 = sK0, sHW = sV0;                // the rings are idle by then (4 x 8 KB each = 32 KB)

  if (tid == 0) {
    s_abort = *reinterpret_cast<volatile int*>(p.err) != 0;
    mbar_init(BAR(B_Q), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(BAR(B_K + s), 1); mbar_init(BAR(B_V + s), 1);
      mbar_init(BAR(B_KE + s), 1); mbar_init(BAR(B_VE + s), 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(BAR(B_S + b), 1); mbar_init(BAR(B_P + b), 128); }
    mbar_init(BAR(B_PV), 1);
    mbar_init(BAR(B_PV + 1), 1);
    mbar_init(BAR(B_Q16), 1);
    mbar_init(BAR(B_HW), 1);
    mbar_init(BAR(B_PHI), 128);
    mbar_init(BAR(B_LIN), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 4) {
    if (lane == 0) { prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmO); }
    const int32_t* row = p.lut + (static_cast<size_t>(bh) * p.mb + tile) * p.topk;
    for (int i = lane; i < p.topk; i += 32) {
      int idx = row[i];
      ulist[i] = idx;
      sk_list[i] = p.kscale[static_cast<size_t>(bh) * p.nb + idx];
    }
  }
  for (int i = tid; i < D; i += 192) s_vscale[i] = p.vscale[static_cast<size_t>(bh) * D + i];
  if (fused && tid < D) {
    const T* rec = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);
    if (tid < D / 2) s_zp[tid] = reinterpret_cast<const uint32_t*>(rec + D * D)[tid];
    s_bias[tid] = Elem<T>::to_f(static_cast<const T*>(p.wbits)[D * D + tid]);
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  const int n_ent = p.topk;
  volatile int* abortp = &s_abort;

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && !*abortp) {
      mbar_expect_tx(BAR(B_Q), Q_BYTES);
      tma_load_3d(sQ, &tmQ, BAR(B_Q), 0, tile * 128, bh);
      int issued_k = 0, issued_v = 0;
      for (int t = 0; t <= n_ent; ++t) {
        if (t < n_ent) {
          const int s = t % NS, use = t / NS;
          if (use > 0 && !mbar_wait(BAR(B_KE + s), (use - 1) & 1, kSErrEmpty, p.err)) { *abortp = 1; break; }
          if (*abortp) break;
          mbar_expect_tx(BAR(B_K + s), KV_BYTES);
          tma_load_3d(sK0 + s * KV_BYTES, &tmK, BAR(B_K + s), 0, ulist[t] * 64, bh);
          issued_k = t + 1;
        }
        if (t >= 1) {
          const int j = t - 1, s = j % NS, use = j / NS;
          if (use > 0 && !mbar_wait(BAR(B_VE + s), (use - 1) & 1, kSErrEmpty, p.err)) { *abortp = 1; break; }
          if (*abortp) break;
          mbar_expect_tx(BAR(B_V + s), KV_BYTES);
          tma_load_3d(sV0 + s * KV_BYTES, &tmV, BAR(B_V + s), 0, ulist[j] * 64, bh);
          issued_v = j + 1;
        }
      }
      if (fused && !*abortp) {
        // 16-bit Q tile into the K ring once the last S GEMMs have read it, H W^T into the V ring once the last
        // P.V GEMMs have (that load overlaps the feature map of the softmax warps)
        bool ring_free = true;
        for (int j = max(0, n_ent - NS); ring_free && j < n_ent; ++j)
          ring_free = mbar_wait(BAR(B_KE + j % NS), (j / NS) & 1, kSErrEmpty, p.err);
        if (ring_free) {
          mbar_expect_tx(BAR(B_Q16), NSLAB * Q16_SLAB);
          for (int c = 0; c < NSLAB; ++c) tma_load_3d(sQ16 + c * Q16_SLAB, &tmQ16, BAR(B_Q16), c * 64, tile * 128, bh);
          for (int j = max(0, n_ent - NS); ring_free && j < n_ent; ++j)
            ring_free = mbar_wait(BAR(B_VE + j % NS), (j / NS) & 1, kSErrEmpty, p.err);
          if (ring_free) {
            mbar_expect_tx(BAR(B_HW), D * D * 2);
            for (int r = 0; r < NSLAB; ++r)
              for (int c = 0; c < NSLAB; ++c)
                tma_load_3d(sHW + r * HW_STAGE + c * HW_SLAB, &tmHW, BAR(B_HW), c * 64, r * 64, bh);
            if (*abortp) mbar_wait_drain(BAR(B_HW), 0, p.err);
          }
          if (!ring_free || *abortp) mbar_wait_drain(BAR(B_Q16), 0, p.err);
        }
        if (!ring_free) *abortp = 1;
      }
      if (*abortp) {
        mbar_wait_drain(BAR(B_Q), 0, p.err);
        for (int j = max(0, issued_k - NS); j < issued_k; ++j) mbar_wait_drain(BAR(B_K + j % NS), (j / NS) & 1, p.err);
        for (int j = max(0, issued_v - NS); j < issued_v; ++j) mbar_wait_drain(BAR(B_V + j % NS), (j / NS) & 1, p.err);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    // All 32 lanes run the control flow; one elected lane issues the tcgen05 instructions.
    if (!*abortp) {
      const uint32_t q_lo = desc_lo(sQ, 16);
      auto issue_s = [&](int j) {
        const uint32_t k_lo = desc_lo(sK0 + (j % NS) * KV_BYTES, 16);
        const uint32_t d = tmem + COL_S + (j & 1) * 64;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 32; ++kk)   // K = 32 int8 = 32 bytes per step inside the 128-byte row
            mma_ss_i8(d, q_lo + ((kk * 32) >> 4), k_lo + ((kk * 32) >> 4), IDESC_S, kk > 0 ? 1u : 0u);
          tc_commit(BAR(B_S + (j & 1)));
          tc_commit(BAR(B_KE + j % NS));
        }
        __syncwarp();
      };
      bool ok = warp_all(mbar_wait(BAR(B_Q), 0, kSErrQ, p.err) && mbar_wait(BAR(B_K), 0, kSErrK, p.err));
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; ok && j < n_ent; ++j) {
        if (j + 1 < n_ent) {
          ok = warp_all(mbar_wait(BAR(B_K + (j + 1) % NS), ((j + 1) / NS) & 1, kSErrK, p.err));
          if (!ok) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        ok = warp_all(mbar_wait(BAR(B_P + (j & 1)), (j >> 1) & 1, kSErrP, p.err) &&
                      mbar_wait(BAR(B_V + j % NS), (j / NS) & 1, kSErrV, p.err));
        if (!ok) break;
        tc_fence_after();
        // B = V8_j rows [32 kk, +32): MN-major, one 128-byte atom per row, 8-row groups 1024 B apart
        const uint32_t v_lo = desc_lo(sV0 + (j % NS) * KV_BYTES, KV_BYTES);
        const uint32_t pa = tmem + COL_S + (j & 1) * 64;   // P_j: four e4m3 per column, 16 columns
        const uint32_t acc_on = j > 0 ? 1u : 0u;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
            mma_ts_f8(tmem + COL_O, pa + kk * 8, v_lo + ((kk * 4096) >> 4), IDESC_PV, kk > 0 ? 1u : acc_on);
          tc_commit(BAR(B_VE + j % NS));
          tc_commit(BAR(B_PV + (j & 1)));
        }
        __syncwarp();
      }
      if (ok && fused) {
        // LIN[128 x D] = phi(Q) (H W^T), 16-bit operands, into the idle S columns
        ok = warp_all(mbar_wait(BAR(B_HW), 0, kSErrHw, p.err) && mbar_wait(BAR(B_PHI), 0, kSErrPhi, p.err));
        if (ok) {
          tc_fence_after();
          const uint32_t a_lo = desc_lo(sQ16, 16);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t hw_lo = desc_lo(sHW + (kk >> 2) * HW_STAGE, HW_SLAB) + (((kk & 3) * 2048) >> 4);
              mma_ss(tmem + COL_S, a_lo + (((kk >> 2) * Q16_SLAB + (kk & 3) * 32) >> 4), hw_lo, IDESC_LIN, kk > 0 ? 1u : 0u);
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
    const int row = tid;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float sq = p.qscale[static_cast<size_t>(bh) * p.mb + tile] * p.scale_log2;
    float m_true = -INFINITY, m_used = -INFINITY, l = 0.f;
    bool ok = !*abortp;
    for (int j = 0; ok && j < n_ent; ++j) {
      const int b = j & 1;
      if (!mbar_wait(BAR(B_S + b), (j >> 1) & 1, kSErrS, p.err)) { ok = false; break; }
      if (*abortp) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem + lane_addr + COL_S + b * 64;
      uint32_t sv[64];
      tmem_ld_x64(s_addr, sv);
      tmem_wait_ld();
      const float sc = sq * sk_list[j];
      const int valid = L - ulist[j] * 64;
      if (valid < 64) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (c >= valid) sv[c] = 0x80000000u;          // most negative integer: exp2 gives 0
      }
      // row maximum on the integer scores (the dequantisation scale is positive); four chains
      int32_t im0 = static_cast<int32_t>(sv[0]), im1 = static_cast<int32_t>(sv[1]);
      int32_t im2 = static_cast<int32_t>(sv[2]), im3 = static_cast<int32_t>(sv[3]);
#pragma unroll
      for (int c = 4; c < 64; c += 4) {
        im0 = max(im0, static_cast<int32_t>(sv[c]));
        im1 = max(im1, static_cast<int32_t>(sv[c + 1]));
        im2 = max(im2, static_cast<int32_t>(sv[c + 2]));
        im3 = max(im3, static_cast<int32_t>(sv[c + 3]));
      }
      const float mx = static_cast<float>(max(max(im0, im1), max(im2, im3))) * sc;
      m_true = fmaxf(m_true, mx);
      const bool need = m_true > m_used + kLazy;   // also true on the first block (m_used = -inf)
      if (j > 0 && __any_sync(0xffffffffu, need)) {
        if (!mbar_wait(BAR(B_PV + ((j - 1) & 1)), ((j - 1) >> 1) & 1, kSErrPv, p.err)) { ok = false; break; }
        tc_fence_after();
        const float alpha = need ? ex2s(m_used - m_true) : 1.0f;
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
        l *= ex2s(m_used - m_true);
        m_used = m_true;
      }
      uint32_t pk[16];
      float rs0 = 0.f, rs1 = 0.f, rs2 = 0.f, rs3 = 0.f;
      const float off = kPShift - m_used;               // P * 2^kPShift straight out of the exponent
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        float p0 = ex2s(fmaf(static_cast<float>(static_cast<int32_t>(sv[c])), sc, off));
        float p1 = ex2s(fmaf(static_cast<float>(static_cast<int32_t>(sv[c + 1])), sc, off));
        float p2 = ex2s(fmaf(static_cast<float>(static_cast<int32_t>(sv[c + 2])), sc, off));
        float p3 = ex2s(fmaf(static_cast<float>(static_cast<int32_t>(sv[c + 3])), sc, off));
        rs0 += p0; rs1 += p1; rs2 += p2; rs3 += p3;
        pk[c >> 2] = pack_e4m3x4(p0, p1, p2, p3);
      }
      const float rs = (rs0 + rs1) + (rs2 + rs3);
      l += rs;
      tmem_st_x16(s_addr, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(BAR(B_P + b));
    }
    if (ok && n_ent > 0) ok = mbar_wait(BAR(B_PV + ((n_ent - 1) & 1)), ((n_ent - 1) >> 1) & 1, kSErrPv, p.err);
    if (!ok) *abortp = 1;
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    if (!*abortp) {
      tc_fence_after();
      const float inv = 1.0f / l;                       // l carries the 2^kPShift of P
      const int grow = tile * 128 + row;
      if (grow < L) p.lse[static_cast<size_t>(bh) * L + grow] = m_used + log2f(l) - kPShift;
      // 16-byte chunk ch of this thread's row inside a 128-row, 16-bit tile at `tile_base`
      auto chunk_addr = [&](uint32_t tile_base, int ch) {
        return tile_base + (ch >> 3) * O_SLAB + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
      };
      float rden = 0.f;
      bool lin_ok = true;
      if (fused) {
        // ---- phi(q) of this thread's row, written over the row of the 16-bit Q tile (core.py:90) ----
        lin_ok = mbar_wait(BAR(B_Q16), 0, kSErrQ16, p.err);
        if (lin_ok) {
          float dsum = 0.f;        // sum_d round(phi_d * z_d), core.py:95
          auto emit_phi = [&](int ch, const float (&f)[8]) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              w[i] = Elem<T>::pack2(f[2 * i], f[2 * i + 1]);
              const float2 pz = Elem<T>::unpack2(Elem<T>::mul2(w[i], s_zp[ch * 4 + i]));   // each product rounded to T
              dsum += pz.x + pz.y;
            }
            st_shared_v4(chunk_addr(sQ16, ch), w[0], w[1], w[2], w[3]);
          };
          auto load_x = [&](int ch, float (&f)[8]) {
            uint32_t w0, w1, w2, w3;
            ld_shared_v4(chunk_addr(sQ16, ch), w0, w1, w2, w3);
            float2 a = Elem<T>::unpack2(w0), b2 = Elem<T>::unpack2(w1), c = Elem<T>::unpack2(w2), d = Elem<T>::unpack2(w3);
            f[0] = a.x; f[1] = a.y; f[2] = b2.x; f[3] = b2.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
          };
          if (p.feature == SLA_PHI_SOFTMAX) {
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int ch = 0; ch < D / 8; ++ch) {
              float f[8];
              load_x(ch, f);
              mx0 = fmaxf(mx0, fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])));
              mx1 = fmaxf(mx1, fmaxf(fmaxf(f[4], f[5]), fmaxf(f[6], f[7])));
            }
            const float neg_mx = -fmaxf(mx0, mx1) * kLog2e;
            // exp(x - max) in fp32 is parked in the idle S columns of this thread's TMEM lane
            float e0 = 0.f, e1 = 0.f;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t ev[32];
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                float f[8];
                load_x((c0 >> 3) + q4, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float e = ex2s(fmaf(f[i], kLog2e, neg_mx));
                  if (i & 1) e1 += e; else e0 += e;
                  ev[q4 * 8 + i] = __float_as_uint(e);
                }
              }
              tmem_st_x32(tmem + lane_addr + COL_S + c0, ev);
            }
            tmem_wait_st();
            const float inv_s = 1.f / (e0 + e1);
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t ev[32];
              tmem_ld_x32(tmem + lane_addr + COL_S + c0, ev);
              tmem_wait_ld();
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(ev[q4 * 8 + i]) * inv_s;
                emit_phi((c0 >> 3) + q4, f);
              }
            }
          } else {
#pragma unroll
            for (int ch = 0; ch < D / 8; ++ch) {
              float f[8];
              load_x(ch, f);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (p.feature == SLA_PHI_RELU) f[i] = fmaxf(f[i], 0.f);
                else f[i] = f[i] > 0.f ? f[i] + 1.f : __expf(f[i]);      // elu(x) + 1
              }
              emit_phi(ch, f);
            }
          }
          rden = 1.f / round_to<T>(1e-5f + round_to<T>(dsum));
          fence_proxy_async_smem();
          tc_fence_before();
          mbar_arrive(BAR(B_PHI));
          lin_ok = mbar_wait(BAR(B_LIN), 0, kSErrLin, p.err);
          if (lin_ok) tc_fence_after();
        }
        if (!lin_ok) *abortp = 1;
      }
      if (lin_ok) {
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t ov[32], lv[32];
          tmem_ld_x32(tmem + lane_addr + COL_O + c0, ov);
          if (fused) tmem_ld_x32(tmem + lane_addr + COL_S + c0, lv);
          tmem_wait_ld();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int ci = q4 * 8 + 2 * e, c = c0 + ci;
              w[e] = Elem<T>::pack2(__uint_as_float(ov[ci]) * inv * s_vscale[c],
                                    __uint_as_float(ov[ci + 1]) * inv * s_vscale[c + 1]);
              if (fused) {   // o = o_s + round(lin / den + bias) (core.py:96-100)
                const uint32_t lin2 = Elem<T>::pack2(fmaf(__uint_as_float(lv[ci]), rden, s_bias[c]),
                                                     fmaf(__uint_as_float(lv[ci + 1]), rden, s_bias[c + 1]));
                w[e] = Elem<T>::add2(w[e], lin2);
              }
            }
            st_shared_v4(chunk_addr(sO, (c0 >> 3) + q4), w[0], w[1], w[2], w[3]);
          }
        }
      }
      fence_proxy_async_smem();
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      if (tid == 0 && !*abortp) {
        for (int c = 0; c < NSLAB; ++c) tma_store_3d(&tmO, sO + c * O_SLAB, c * 64, tile * 128, bh);
        tma_store_commit();
      }
      if (p.n_gather > 0 && !*abortp) {
        // the staged tile once more to every gather destination (sla_fwd_gather's scheme: consecutive lanes write
        // consecutive 16-byte chunks of a row; no TMA and no multicast touch memory that may be another GPU's)
        constexpr int CH = D / 8;
        for (int idx = tid; idx < 128 * CH; idx += 128) {
          const int r = idx / CH, ch = idx % CH;
          const int gr = tile * 128 + r;
          if (gr < L) {
            uint32_t w0, w1, w2, w3;
            ld_shared_v4(sO + (ch >> 3) * O_SLAB + r * 128 + (((ch & 7) ^ (r & 7)) << 4), w0, w1, w2, w3);
            const size_t off = ((static_cast<size_t>(bh) * L + gr) * D + ch * 8) * sizeof(T);
            for (int g = 0; g < p.n_gather; ++g)
              *reinterpret_cast<uint4*>(static_cast<char*>(p.gather[g]) + off) = make_uint4(w0, w1, w2, w3);
          }
        }
      }
      if (tid == 0) tma_store_wait_read();
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

// ---------------------------------------------------------------------------------------------
// Quantization pre-passes (HBM-bound)
// ---------------------------------------------------------------------------------------------
// One CTA per block of `blk` rows: symmetric abs-max INT8, scale = amax / 127 (zero blocks get scale 1e-8/127).
// z = 0: Q in blocks of 128 rows; z = 1: K - mean in blocks of 64 rows.
// The 8-bit rows are written 128 bytes apart whatever D is (the pad of a D = 64 row is never read).
template <typename T, int D>
__global__ void __launch_bounds__(256, 3) sage_quant_qk_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                               const float* __restrict__ kmean, int8_t* __restrict__ q8,
                                                               int8_t* __restrict__ k8, float* __restrict__ qscale,
                                                               float* __restrict__ kscale, int L, int mb, int nb) {
  constexpr int TPR = D / 8, RPP = 256 / TPR;   // threads per row (8 elements each), rows per pass
  __shared__ float red[8];
  const bool is_k = blockIdx.z == 1;
  const int blk = is_k ? 64 : 128, nblk = is_k ? nb : mb;
  if (static_cast<int>(blockIdx.x) >= nblk) return;
  const int bh = blockIdx.y, ib = blockIdx.x, tid = threadIdx.x;
  const T* src = (is_k ? k : q) + static_cast<size_t>(bh) * L * D;
  int8_t* dst = (is_k ? k8 : q8) + static_cast<size_t>(bh) * L * 128;
  const int c = (tid % TPR) * 8;
  float mean[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) mean[e] = is_k ? kmean[static_cast<size_t>(bh) * D + c + e] : 0.f;
  // The rows stay packed in registers (4 words per row) between the abs-max pass and the rounding pass, which
  // keeps three CTAs per SM resident; all loads of a thread are issued up front.
  uint4 raw[8];                                 // up to 8 rows per thread (128 rows / 16 row groups)
  const int rows_per_thread = blk / RPP;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = ib * blk + tid / TPR + RPP * i;
    raw[i] = (i < rows_per_thread && r < L) ? *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * D + c)
                                            : make_uint4(0u, 0u, 0u, 0u);
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = ib * blk + tid / TPR + RPP * i;
    if (i < rows_per_thread && r < L) {
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw[i]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = Elem<T>::unpack2(u[e]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x - mean[2 * e]), fabsf(f.y - mean[2 * e + 1])));
      }
    }
  }
  amax = warp_max(amax);
  if ((tid & 31) == 0) red[tid >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);
  const float scale = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / scale;
  if (tid == 0) (is_k ? kscale : qscale)[static_cast<size_t>(bh) * nblk + ib] = scale;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = ib * blk + tid / TPR + RPP * i;
    if (i < rows_per_thread && r < L) {
      const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw[i]);
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float2 f0 = Elem<T>::unpack2(u[2 * h]), f1 = Elem<T>::unpack2(u[2 * h + 1]);
        int b0 = __float2int_rn((f0.x - mean[4 * h]) * inv), b1 = __float2int_rn((f0.y - mean[4 * h + 1]) * inv);
        int b2 = __float2int_rn((f1.x - mean[4 * h + 2]) * inv), b3 = __float2int_rn((f1.y - mean[4 * h + 3]) * inv);
        w[h] = (b0 & 0xff) | ((b1 & 0xff) << 8) | ((b2 & 0xff) << 16) | (static_cast<uint32_t>(b3 & 0xff) << 24);
      }
      *reinterpret_cast<uint2*>(dst + static_cast<size_t>(r) * 128 + c) = make_uint2(w[0], w[1]);
    }
  }
}

// per-channel abs-max of V over chunks of 512 rows: partial[bh][chunk][D]
template <typename T, int D>
__global__ void __launch_bounds__(256) sage_v_amax_kernel(const T* __restrict__ v, float* __restrict__ partial,
                                                          int L, int nch) {
  constexpr int TPR = D / 8, RPP = 256 / TPR;
  __shared__ float red[RPP][D];
  const int bh = blockIdx.y, ch = blockIdx.x, tid = threadIdx.x;
  const int rg = tid / TPR, c = (tid % TPR) * 8;
  const T* base = v + static_cast<size_t>(bh) * L * D;
  float am[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) am[e] = 0.f;
  const int row1 = min(L, (ch + 1) * 512);
  for (int r = ch * 512 + rg; r < row1; r += RPP) {
    uint4 raw = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(r) * D + c);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = Elem<T>::unpack2(u[e]);
      am[2 * e] = fmaxf(am[2 * e], fabsf(f.x));
      am[2 * e + 1] = fmaxf(am[2 * e + 1], fabsf(f.y));
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[rg][c + e] = am[e];
  __syncthreads();
  if (tid < D) {
    float m = 0.f;
#pragma unroll
    for (int g = 0; g < RPP; ++g) m = fmaxf(m, red[g][tid]);
    partial[(static_cast<size_t>(bh) * nch + ch) * D + tid] = m;
  }
}
__global__ void sage_v_scale_kernel(const float* __restrict__ partial, float* __restrict__ vscale, int nch) {
  const int bh = blockIdx.x, d = threadIdx.x, D = blockDim.x;
  float m = 0.f;
  for (int c = 0; c < nch; ++c) m = fmaxf(m, partial[(static_cast<size_t>(bh) * nch + c) * D + d]);
  vscale[static_cast<size_t>(bh) * D + d] = fmaxf(m, 1e-8f) / 448.f;
}
template <typename T, int D>
__global__ void __launch_bounds__(256) sage_quant_v_kernel(const T* __restrict__ v, const float* __restrict__ vscale,
                                                           uint8_t* __restrict__ v8, int L) {
  constexpr int TPR = D / 8, RPP = 256 / TPR;
  const int bh = blockIdx.y, tid = threadIdx.x;
  const int c = (tid % TPR) * 8;
  float inv[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) inv[e] = 1.f / vscale[static_cast<size_t>(bh) * D + c + e];
  const T* base = v + static_cast<size_t>(bh) * L * D;
  uint8_t* out = v8 + static_cast<size_t>(bh) * L * 128;
  for (int r = blockIdx.x * 64 + tid / TPR; r < min(L, (static_cast<int>(blockIdx.x) + 1) * 64); r += RPP) {
    uint4 raw = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(r) * D + c);
    const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw);
    float f[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 t = Elem<T>::unpack2(u[e]);
      f[2 * e] = t.x * inv[2 * e];
      f[2 * e + 1] = t.y * inv[2 * e + 1];
    }
    uint2 w = make_uint2(tc::pack_e4m3x4(f[0], f[1], f[2], f[3]), tc::pack_e4m3x4(f[4], f[5], f[6], f[7]));
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(r) * 128 + c) = w;
  }
}

// The quantization pre-passes: need q, k, v only.
template <typename T, int D>
static int run_sage_quant_typed(const sla_shape* s, const void* q, const void* k, const void* v, unsigned char* ws,
                                cudaStream_t st) {
  const int bh = s->B * s->H, L = s->L;
  const int mb = ceil_div(L, 128), nb = ceil_div(L, 64);
  WsSage w = ws_sage(s);
  float* kmean = reinterpret_cast<float*>(ws + w.kmean);
  float* part = reinterpret_cast<float*>(ws + w.colsum);
  int8_t* q8 = reinterpret_cast<int8_t*>(ws + w.q8);
  int8_t* k8 = reinterpret_cast<int8_t*>(ws + w.k8);
  uint8_t* v8 = ws + w.v8;
  float* qs = reinterpret_cast<float*>(ws + w.qscale);
  float* ks = reinterpret_cast<float*>(ws + w.kscale);
  float* vs = reinterpret_cast<float*>(ws + w.vscale);
  int rc = run_k_mean(s, k, part, kmean, st);
  if (rc != SLA_OK) return rc;
  sage_quant_qk_kernel<T, D><<<dim3(nb, bh, 2), 256, 0, st>>>(static_cast<const T*>(q), static_cast<const T*>(k), kmean,
                                                          q8, k8, qs, ks, L, mb, nb);
  SLA_LAUNCH_OK();
  sage_v_amax_kernel<T, D><<<dim3(w.nch, bh), 256, 0, st>>>(static_cast<const T*>(v), part, L, w.nch);
  SLA_LAUNCH_OK();
  sage_v_scale_kernel<<<bh, D, 0, st>>>(part, vs, w.nch);
  SLA_LAUNCH_OK();
  sage_quant_v_kernel<T, D><<<dim3(nb, bh), 256, 0, st>>>(static_cast<const T*>(v), vs, v8, L);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

// The attention kernel on the quantized copies.
template <typename T, int D>
static int run_sage_main_typed(const sla_shape* s, const void* q, const int32_t* lut, void* o_s, float* lse,
                               unsigned char* ws, const void* lin_state, const void* wbits, cudaStream_t st,
                               void* const* gather_dst, int n_gather) {
  const int bh = s->B * s->H, L = s->L;
  const int mb = ceil_div(L, 128), nb = ceil_div(L, 64);
  WsSage w = ws_sage(s);
  int8_t* q8 = reinterpret_cast<int8_t*>(ws + w.q8);
  int8_t* k8 = reinterpret_cast<int8_t*>(ws + w.k8);
  uint8_t* v8 = ws + w.v8;
  float* qs = reinterpret_cast<float*>(ws + w.qscale);
  float* ks = reinterpret_cast<float*>(ws + w.kscale);
  float* vs = reinterpret_cast<float*>(ws + w.vscale);
  int rc;
  CUtensorMap tq, tk, tv, to, tq16, thw;
  if ((rc = make_tmap_3d_u8(&tq, q8, 128, L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d_u8(&tk, k8, 128, L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d_u8(&tv, v8, 128, L, bh, 64)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&to, o_s, s->dtype, D, L, bh, 128)) != SLA_OK) return rc;
  const bool fused = lin_state != nullptr;
  tq16 = to; thw = to;
  if (fused) {
    if ((rc = make_tmap_3d(&tq16, q, s->dtype, D, L, bh, 128)) != SLA_OK) return rc;
    const char* hw = static_cast<const char*>(lin_state) + (size_t(D) * D + D) * 2;   // H W^T behind H and z
    if ((rc = make_tmap_rows(&thw, hw, s->dtype, D, D, bh, size_t(2 * D * D + D) * 2, 64)) != SLA_OK) return rc;
  }
  tc::SageParams p;
  p.feature = fused ? s->feature_map : -1;
  p.lin_state = lin_state; p.wbits = wbits;
  p.lut = lut; p.qscale = qs; p.kscale = ks; p.vscale = vs; p.lse = lse;
  p.err = tc_error_word();
  if (p.err == nullptr) return SLA_ERR_CUDA;
  p.L = L; p.mb = mb; p.nb = nb; p.topk = s->topk;
  p.scale_log2 = softmax_scale(s) * kLog2e;
  p.n_gather = n_gather;
  for (int g = 0; g < 8; ++g) p.gather[g] = g < n_gather ? gather_dst[g] : nullptr;
  auto kern = tc::sage_fwd_tc_kernel<T, D>;
  const int smem = 1024 + 2 * 128 * 128 + 2 * 4 * 64 * 128 + s->topk * 8 + 16;
  // up to 113 KB two CTAs share an SM, a longer list takes the SM alone; beyond 227 KB there is no quantized path
  if (smem + 2048 > 227 * 1024) return SLA_ERR_UNSUPPORTED;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<dim3(mb, bh), 192, smem, st>>>(tq, tk, tv, to, tq16, thw, p);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

}  // namespace sla

namespace sla {

static int sage_quant(const sla_shape* s, const void* q, const void* k, const void* v, unsigned char* ws, cudaStream_t st) {
  if (s->D == 64)
    return s->dtype == SLA_BF16 ? run_sage_quant_typed<__nv_bfloat16, 64>(s, q, k, v, ws, st)
                                : run_sage_quant_typed<__half, 64>(s, q, k, v, ws, st);
  return s->dtype == SLA_BF16 ? run_sage_quant_typed<__nv_bfloat16, 128>(s, q, k, v, ws, st)
                              : run_sage_quant_typed<__half, 128>(s, q, k, v, ws, st);
}
static int sage_main(const sla_shape* s, const void* q, const int32_t* lut, void* o, float* lse, unsigned char* ws,
                     const void* state, const void* wbits, cudaStream_t st, void* const* gather_dst = nullptr,
                     int n_gather = 0) {
  if (s->D == 64)
    return s->dtype == SLA_BF16 ? run_sage_main_typed<__nv_bfloat16, 64>(s, q, lut, o, lse, ws, state, wbits, st, gather_dst, n_gather)
                                : run_sage_main_typed<__half, 64>(s, q, lut, o, lse, ws, state, wbits, st, gather_dst, n_gather);
  return s->dtype == SLA_BF16 ? run_sage_main_typed<__nv_bfloat16, 128>(s, q, lut, o, lse, ws, state, wbits, st, gather_dst, n_gather)
                              : run_sage_main_typed<__half, 128>(s, q, lut, o, lse, ws, state, wbits, st, gather_dst, n_gather);
}
static int sage_check(const sla_shape* s) {
  int rc = validate_shape(s);
  if (rc != SLA_OK) return rc;
  if (s->BLKQ != 128 || s->BLKK != 64) return SLA_ERR_BAD_SHAPE;   // SageSLA/README.md:16-17
  if (s->D != 64 && s->D != 128) return SLA_ERR_UNSUPPORTED;       // SageSLA/core.py:112
  return check_device_arch();
}
// linear-branch state (SageSLA/core.py:148-158 uses the same branch as the 16-bit module); the read-out, proj_l
// and the final sum run in the epilogue of the quantized kernel
static int sage_state(const sla_shape* s, const void* k, const void* v, const float* w, const float* bias,
                      void* lin_state, unsigned char* base, cudaStream_t st) {
  WsSage wsz = ws_sage(s);
  WsLinearState wl = ws_linear_state(s);
  void* wbits = base + wsz.wbits;
  int rc;
  if ((rc = convert_proj(s, w, bias, wbits, st)) != SLA_OK) return rc;
  if ((rc = run_linear_state(s, k, v, lin_state, reinterpret_cast<float*>(base + wsz.lin + wl.partial), wl.nch, wl.rows, st)) != SLA_OK) return rc;
  return run_state_proj(s, lin_state, wbits, st);
}

}  // namespace sla

extern "C" int sage_sla_prepare(const sla_shape* s, const void* q, const void* k, const void* v, const float* w,
                                const float* bias, void* lin_state, void* ws, size_t ws_bytes, sla_stream_t stream) {
  using namespace sla;
  if (!q || !k || !v || !ws) return SLA_ERR_NULL;
  int rc = sage_check(s);
  if (rc != SLA_OK) return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(ws)) return SLA_ERR_BAD_ALIGN;
  if (ws_bytes < ws_sage(s).total) return SLA_ERR_WS_TOO_SMALL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* base = static_cast<unsigned char*>(ws);
  if (!(s->flags & SLA_FLAG_SPARSE_ONLY)) {
    if (!w || !lin_state) return SLA_ERR_NULL;
    if (!aligned16(lin_state)) return SLA_ERR_BAD_ALIGN;
    if ((rc = sage_state(s, k, v, w, bias, lin_state, base, st)) != SLA_OK) return rc;
  }
  return sage_quant(s, q, k, v, base, st);
}

static int sage_fwd_impl(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
                         const float* w, const float* bias, void* o, void* lin_state, void* ws, size_t ws_bytes,
                         void* const* gather_dst, int n_gather, sla_stream_t stream) {
  using namespace sla;
  if (!q || !k || !v || !lut || !o || !ws) return SLA_ERR_NULL;
  int rc = sage_check(s);
  if (rc != SLA_OK) return rc;
  if (n_gather < 0 || n_gather > 8 || (n_gather > 0 && gather_dst == nullptr)) return SLA_ERR_UNSUPPORTED;
  for (int g = 0; g < n_gather; ++g) {
    if (gather_dst[g] == nullptr) return SLA_ERR_NULL;
    if (!aligned16(gather_dst[g])) return SLA_ERR_BAD_ALIGN;
  }
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(ws)) return SLA_ERR_BAD_ALIGN;
  WsSage wsz = ws_sage(s);
  if (ws_bytes < wsz.total) return SLA_ERR_WS_TOO_SMALL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* base = static_cast<unsigned char*>(ws);
  float* lse = reinterpret_cast<float*>(base + wsz.lse);
  const bool ready = (s->flags & SLA_FLAG_STATE_READY) != 0;   // sage_sla_prepare has filled lin_state and ws
  const void* state = nullptr;
  if (!(s->flags & SLA_FLAG_SPARSE_ONLY)) {
    if (!w || !lin_state) return SLA_ERR_NULL;
    if (!aligned16(lin_state)) return SLA_ERR_BAD_ALIGN;
    if (!ready && (rc = sage_state(s, k, v, w, bias, lin_state, base, st)) != SLA_OK) return rc;
    state = lin_state;
  }
  if (!ready && (rc = sage_quant(s, q, k, v, base, st)) != SLA_OK) return rc;
  return sage_main(s, q, lut, o, lse, base, state, base + wsz.wbits, st, gather_dst, n_gather);
}

extern "C" int sage_sla_fwd(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
                            const float* w, const float* bias, void* o, void* lin_state, void* ws, size_t ws_bytes,
                            sla_stream_t stream) {
  return sage_fwd_impl(s, q, k, v, lut, w, bias, o, lin_state, ws, ws_bytes, nullptr, 0, stream);
}

extern "C" int sage_sla_fwd_gather(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
                                   const float* w, const float* bias, void* o, void* lin_state, void* ws,
                                   size_t ws_bytes, void* const* gather_dst, int n_gather, sla_stream_t stream) {
  return sage_fwd_impl(s, q, k, v, lut, w, bias, o, lin_state, ws, ws_bytes, gather_dst, n_gather, stream);
}
