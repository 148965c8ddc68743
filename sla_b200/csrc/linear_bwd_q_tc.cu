// Pass A of the linear-branch backward (see linear_bwd.cu for the algebra) on tcgen05, head dim 128.
//
// Per tile of 128 query rows:  t = dY (H W^T)^T  and  G += dY^T (phi_q / den)  are two 128 x 128 x 128 GEMMs;
// everything else is row-wise: phi(q), den, dden = -(phi_q . t) / den^2, dphi_q = t / den + dden z,
// dq_lin = phi'(q) dphi_q, plus two column sums over the rows of the tile (dz += sum_m dden_m phi_q,m and
// db += sum_m dY_m).
//
// One CTA = one chunk of rows of one head (the chunking of the mma.sync pass A: same partial buffers, same
// per-head reduction kernels afterwards). 192 threads: warps 0-3 own one tile row each (thread = row = TMEM lane),
// warp 4 is the TMA producer and sums the columns of dY for db, warp 5 issues the MMAs and sums the columns
// of phi_q / den for dz. Shared memory holds H W^T (32 KB) and ONE {Q, dY} tile pair (64 KB): two CTAs share
// an SM, and one computes while the other waits for its loads. Tensor memory: G (128 columns, accumulated
// over the CTA's tiles) and t (128 columns, which first park exp(q - max) of the softmax feature map).
//   Q tile:  q  ->  phi_q / den (MN-major B operand of the G GEMM, then read for dz)
//   dY tile: K-major A operand of the t GEMM, MN-major A operand of the G GEMM  ->  dq staging for the TMA store
// All waits are bounded (tc_common.cuh).
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"

namespace sla {
namespace tc {

enum : int { kLErrHw = 501, kLErrFull = 502, kLErrFree = 503, kLErrX = 504, kLErrT = 505, kLErrG = 506,
             kLErrC = 507, kLErrDb = 508 };

struct LinQParams {
  const void* lin_state;   // [BH][2*D*D + D] T: H, z, H W^T
  float* g_partial;        // [BH][NCH][D*D + 2*D]
  int* err;
  int L, nch, rows, feature, accumulate;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// OR of a predicate over the 128 threads of the row warps (named barrier 1); the result is the same in all of them
__device__ __forceinline__ bool rows_any(bool pred) {
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

template <typename T>
__global__ void __launch_bounds__(192, 2)
linear_bwd_q_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDY,
                       const __grid_constant__ CUtensorMap tmDQ, const __grid_constant__ CUtensorMap tmHW,
                       LinQParams p) {
  constexpr int D = 128;
  constexpr int SLAB = 128 * 128, TILE = 2 * SLAB;       // 64 columns x 128 rows of T; a tile is two slabs
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr uint32_t IDESC_T = idesc_f16(FMT, 128, D, 0, 0);   // dY (K-major) x H W^T (K-major: rows i, k = n)
  constexpr uint32_t IDESC_G = idesc_f16(FMT, 128, D, 1, 1);   // dY^T (MN-major) x phi_q/den (MN-major)
  constexpr uint32_t TMEM_COLS = 256;
  constexpr int COL_G = 0, COL_T = D;

  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[8];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ __align__(16) float s_z[D];
  __shared__ __align__(16) uint32_t s_zp[D / 2];     // z as pairs of T
  __shared__ float s_rowc[128];        // dden * den of the tile's rows

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ch = blockIdx.x, bh = blockIdx.y;
  const int L = p.L;
  pdl_entry();
  const uint32_t raw_a = smem_u32(smem_raw);
  const uint32_t base_a = (raw_a + 1023u) & ~1023u;
  const uint32_t sHW = base_a, sQ = base_a + TILE, sDY = base_a + 2 * TILE;
  const uint32_t bar0 = smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  // H W^T landed | tile pair landed | tile pair free again (dq store has read the dY tile, dz sums have read the
  // Q tile) | phi_q/den written | t done | G done | row constants written | column sums of dY taken.
  // Apart from B_HW every barrier completes one phase per tile.
  constexpr int B_HW = 0, B_FULL = 1, B_FREE = 2, B_X = 3, B_T = 4, B_G = 5, B_C = 6, B_DB = 7;

  const int row_begin = ch * p.rows, row_end = min(L, row_begin + p.rows);
  const int n_tiles = row_end > row_begin ? (row_end - row_begin + 127) / 128 : 0;
  const T* rec = static_cast<const T*>(p.lin_state) + static_cast<size_t>(bh) * (2 * D * D + D);

  if (tid == 0) {
    s_abort = *reinterpret_cast<volatile int*>(p.err) != 0;
    mbar_init(BAR(B_HW), 1);
    mbar_init(BAR(B_FULL), 1);
    mbar_init(BAR(B_FREE), 2);
    mbar_init(BAR(B_X), 4);
    mbar_init(BAR(B_T), 1);
    mbar_init(BAR(B_G), 1);
    mbar_init(BAR(B_C), 4);
    mbar_init(BAR(B_DB), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (tid < D) s_z[tid] = Elem<T>::to_f(rec[D * D + tid]);
  if (tid < D / 2) s_zp[tid] = reinterpret_cast<const uint32_t*>(rec + D * D)[tid];
  if (warp == 4 && lane == 0) { prefetch_tmap(&tmQ); prefetch_tmap(&tmDY); prefetch_tmap(&tmDQ); prefetch_tmap(&tmHW); }
  if (warp == 5) {
    tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;
  volatile int* abortp = &s_abort;
  float* out = p.g_partial + (static_cast<size_t>(bh) * p.nch + ch) * (D * D + 2 * D);

  // byte offset of the 8 bytes holding columns [4 lane, 4 lane + 4) of row m inside a 128-row swizzled tile
  auto col4_off = [&](int m) {
    const int slab = lane >> 4, c = (lane & 15) * 4;           // column inside the 64-column slab
    return static_cast<uint32_t>(slab * SLAB + m * 128 + ((((c >> 3) ^ (m & 7))) << 4) + (c & 7) * 2);
  };

  if (warp == 4) {
    // ------------------------------ TMA producer, and db = column sums of dY ------------------------------
    float db[4] = {0.f, 0.f, 0.f, 0.f};
    bool ok = !*abortp;
    const bool hw_issued = ok;
    if (ok && lane == 0) {
      mbar_expect_tx(BAR(B_HW), TILE);
      for (int r = 0; r < 2; ++r)
        for (int c = 0; c < 2; ++c) tma_load_3d(sHW + c * SLAB + r * (64 * 128), &tmHW, BAR(B_HW), c * 64, r * 64, bh);
    }
    for (int t = 0; ok && t < n_tiles; ++t) {
      const int row0 = row_begin + t * 128;
      int issued = 0;
      if (lane == 0 && (t == 0 || mbar_wait(BAR(B_FREE), (t - 1) & 1, kLErrFree, p.err))) {
        mbar_expect_tx(BAR(B_FULL), 2 * TILE);
        for (int c = 0; c < 2; ++c) {
          tma_load_3d(sQ + c * SLAB, &tmQ, BAR(B_FULL), c * 64, row0, bh);
          tma_load_3d(sDY + c * SLAB, &tmDY, BAR(B_FULL), c * 64, row0, bh);
        }
        issued = 1;
      }
      issued = __shfl_sync(0xffffffffu, issued, 0);
      if (!issued) { ok = false; break; }          // nothing of this tile is in flight
      ok = warp_all(mbar_wait(BAR(B_FULL), t & 1, kLErrFull, p.err));   // also the drain of these loads
      if (!ok) break;
#pragma unroll 8
      for (int m = 0; m < 128; ++m) {
        uint32_t w0, w1;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(w0), "=r"(w1) : "r"(sDY + col4_off(m)));
        const float2 a = Elem<T>::unpack2(w0), b = Elem<T>::unpack2(w1);
        db[0] += a.x; db[1] += a.y; db[2] += b.x; db[3] += b.y;
      }
      mbar_arrive_warp(BAR(B_DB), lane);   // dY may now be overwritten by the staged dq
    }
    if (!ok) *abortp = 1;
    if (hw_issued && lane == 0) mbar_wait(BAR(B_HW), 0, kLErrHw, p.err);   // H W^T has landed before the CTA leaves
#pragma unroll
    for (int e = 0; e < 4; ++e) out[D * D + D + 4 * lane + e] = db[e];
  } else if (warp == 5) {
    // ------------------------------ MMA issuer, and dz = column sums of c_m phi_q,m / den_m ------------------------------
    float dz[4] = {0.f, 0.f, 0.f, 0.f};
    bool ok = !*abortp && warp_all(mbar_wait(BAR(B_HW), 0, kLErrHw, p.err));
    const uint32_t dy_k = desc_lo(sDY, 16), hw_k = desc_lo(sHW, 16);
    const uint32_t dy_mn = desc_lo(sDY, SLAB), x_mn = desc_lo(sQ, SLAB);
    for (int t = 0; ok && t < n_tiles; ++t) {
      ok = warp_all(mbar_wait(BAR(B_FULL), t & 1, kLErrFull, p.err) && mbar_wait(BAR(B_X), t & 1, kLErrX, p.err));
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t ko = ((kk >> 2) * SLAB + (kk & 3) * 32) >> 4;
          mma_ss(tmem + COL_T, dy_k + ko, hw_k + ko, IDESC_T, kk > 0 ? 1u : 0u);
        }
        tc_commit(BAR(B_T));
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk) {      // k = tile rows, 16 per step = 2048 bytes of either operand
          const uint32_t ko = (kk * 2048) >> 4;
          mma_ss(tmem + COL_G, dy_mn + ko, x_mn + ko, IDESC_G, (t > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(BAR(B_G));
      }
      __syncwarp();
      ok = warp_all(mbar_wait(BAR(B_C), t & 1, kLErrC, p.err));
      if (!ok) break;
#pragma unroll 8
      for (int m = 0; m < 128; ++m) {
        uint32_t w0, w1;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(w0), "=r"(w1) : "r"(sQ + col4_off(m)));
        const float2 a = Elem<T>::unpack2(w0), b = Elem<T>::unpack2(w1);
        const float c = s_rowc[m];
        dz[0] = fmaf(c, a.x, dz[0]); dz[1] = fmaf(c, a.y, dz[1]);
        dz[2] = fmaf(c, b.x, dz[2]); dz[3] = fmaf(c, b.y, dz[3]);
      }
      mbar_arrive_warp(BAR(B_FREE), lane);
    }
    if (!ok) *abortp = 1;
#pragma unroll
    for (int e = 0; e < 4; ++e) out[D * D + 4 * lane + e] = dz[e];
  } else {
    // ------------------------------ row warps ------------------------------
    const int row = tid;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    // 16-byte chunk ch (8 columns) of this thread's row inside a swizzled 128-row tile
    auto chunk_addr = [&](uint32_t tile_base, int ch) {
      return tile_base + (ch >> 3) * SLAB + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
    };
    auto load_x = [&](int ch, float (&f)[8]) {
      uint32_t w0, w1, w2, w3;
      ld_shared_v4(chunk_addr(sQ, ch), w0, w1, w2, w3);
      const float2 a = Elem<T>::unpack2(w0), b = Elem<T>::unpack2(w1), c = Elem<T>::unpack2(w2), d = Elem<T>::unpack2(w3);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    };
    const bool softmax = p.feature == SLA_PHI_SOFTMAX;
    bool ok = warp_all(!*abortp);
    for (int t = 0; t < n_tiles; ++t) {
      const int row0 = row_begin + t * 128;
      uint32_t ph[D / 2];        // phi(q) of the row as pairs of T; later dq_lin
      float rd = 0.f, den = 0.f, sum_pz = 0.f;
      ok = ok && warp_all(mbar_wait(BAR(B_FULL), t & 1, kLErrFull, p.err));
      if (ok) {
        // ---- phi(q) (core.py:90), den = 1e-5 + sum_d round(phi_d z_d) (core.py:95) ----
        float dsum = 0.f;
        auto take_phi = [&](int ch, const float (&f)[8]) {
          const uint4 zq = *reinterpret_cast<const uint4*>(&s_zp[ch * 4]);
          const uint32_t zz[4] = {zq.x, zq.y, zq.z, zq.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t w = Elem<T>::pack2(f[2 * i], f[2 * i + 1]);
            ph[ch * 4 + i] = w;
            const float2 pz = Elem<T>::unpack2(Elem<T>::mul2(w, zz[i]));   // each product rounded to T
            dsum += pz.x + pz.y;
            const float2 pf = Elem<T>::unpack2(w), zf = Elem<T>::unpack2(zz[i]);
            sum_pz = fmaf(pf.x, zf.x, fmaf(pf.y, zf.y, sum_pz));
          }
        };
        if (softmax) {
          uint32_t m0, m1, m2, m3;                 // row maximum on the packed pairs (exact: no rounding in a max)
          ld_shared_v4(chunk_addr(sQ, 0), m0, m1, m2, m3);
#pragma unroll
          for (int ch = 1; ch < D / 8; ++ch) {
            uint32_t w0, w1, w2, w3;
            ld_shared_v4(chunk_addr(sQ, ch), w0, w1, w2, w3);
            m0 = Elem<T>::max2(m0, w0); m1 = Elem<T>::max2(m1, w1);
            m2 = Elem<T>::max2(m2, w2); m3 = Elem<T>::max2(m3, w3);
          }
          const float2 mxp = Elem<T>::unpack2(Elem<T>::max2(Elem<T>::max2(m0, m1), Elem<T>::max2(m2, m3)));
          const float neg_mx = -fmaxf(mxp.x, mxp.y) * kLog2e;
          // exp(x - max) in fp32 is parked in the t columns of this thread's TMEM lane (idle until phi is written)
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
                const float e = ex2f(fmaf(f[i], kLog2e, neg_mx));
                if (i & 1) e1 += e; else e0 += e;
                ev[q4 * 8 + i] = __float_as_uint(e);
              }
            }
            tmem_st_x32(tmem + lane_addr + COL_T + c0, ev);
          }
          tmem_wait_st();
          const float inv_s = 1.f / (e0 + e1);
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t ev[32];
            tmem_ld_x32(tmem + lane_addr + COL_T + c0, ev);
            tmem_wait_ld();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(ev[q4 * 8 + i]) * inv_s;
              take_phi((c0 >> 3) + q4, f);
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
            take_phi(ch, f);
          }
        }
        den = round_to<T>(1e-5f + round_to<T>(dsum));
        rd = 1.f / den;
        // phi_q / den over the row of the Q tile: B operand of the G GEMM
#pragma unroll
        for (int ch = 0; ch < D / 8; ++ch) {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 pf = Elem<T>::unpack2(ph[ch * 4 + i]);
            w[i] = Elem<T>::pack2(pf.x * rd, pf.y * rd);
          }
          st_shared_v4(chunk_addr(sQ, ch), w[0], w[1], w[2], w[3]);
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive_warp(BAR(B_X), lane);
      }
      ok = ok && warp_all(mbar_wait(BAR(B_T), t & 1, kLErrT, p.err));
      if (ok) {
        tc_fence_after();
        // ---- s = phi_q . t, dden = -s / den^2 ----
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t tv[32];
          tmem_ld_x32(tmem + lane_addr + COL_T + c0, tv);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 pf = Elem<T>::unpack2(ph[(c0 >> 1) + i]);
            s0 = fmaf(pf.x, __uint_as_float(tv[2 * i]), s0);
            s1 = fmaf(pf.y, __uint_as_float(tv[2 * i + 1]), s1);
          }
        }
        const float sdot = s0 + s1;
        const float dden = -sdot * rd * rd;
        s_rowc[row] = dden * den;
        mbar_arrive_warp(BAR(B_C), lane);
        const float c2 = softmax ? fmaf(rd, sdot, dden * sum_pz) : 0.f;   // sum_d phi_d dphi_d
        // ---- dphi_q = t / den + dden z, dq_lin = phi'(q) dphi_q ----
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t tv[32];
          tmem_ld_x32(tmem + lane_addr + COL_T + c0, tv);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 pf = Elem<T>::unpack2(ph[(c0 >> 1) + i]);
            const float2 zf = *reinterpret_cast<const float2*>(&s_z[c0 + 2 * i]);
            // dphi (minus the softmax's sum_d phi_d dphi_d, c2 = 0 for the other feature maps)
            float g0 = fmaf(__uint_as_float(tv[2 * i]), rd, fmaf(dden, zf.x, -c2));
            float g1 = fmaf(__uint_as_float(tv[2 * i + 1]), rd, fmaf(dden, zf.y, -c2));
            if (softmax) {
              g0 *= pf.x;
              g1 *= pf.y;
            } else if (p.feature == SLA_PHI_RELU) {
              g0 = pf.x > 0.f ? g0 : 0.f;
              g1 = pf.y > 0.f ? g1 : 0.f;
            } else {                                   // elu(x) + 1: derivative 1 for x > 0 (phi > 1), phi otherwise
              g0 = pf.x > 1.f ? g0 : g0 * pf.x;
              g1 = pf.y > 1.f ? g1 : g1 * pf.y;
            }
            ph[(c0 >> 1) + i] = Elem<T>::pack2(g0, g1);
          }
        }
        tc_fence_before();
      }
      // dq is staged over the dY tile once the G GEMM and the db sums have read it
      ok = ok && warp_all(mbar_wait(BAR(B_G), t & 1, kLErrG, p.err) && mbar_wait(BAR(B_DB), t & 1, kLErrDb, p.err));
      if (ok) {
#pragma unroll
        for (int ch = 0; ch < D / 8; ++ch)
          st_shared_v4(chunk_addr(sDY, ch), ph[ch * 4], ph[ch * 4 + 1], ph[ch * 4 + 2], ph[ch * 4 + 3]);
        fence_proxy_async_smem();
      }
      const bool failed = rows_any(!ok || *abortp != 0);
      if (failed) { ok = false; break; }
      if (tid == 0) {
        for (int c = 0; c < 2; ++c) {
          if (p.accumulate) tma_reduce_add_3d(&tmDQ, sDY + c * SLAB, c * 64, row0, bh);
          else tma_store_3d(&tmDQ, sDY + c * SLAB, c * 64, row0, bh);
        }
        tma_store_commit();
        tma_store_wait_read();
        mbar_arrive(BAR(B_FREE));
      }
    }
    if (!ok) *abortp = 1;
    // ---- G of this chunk: row n of G[n][i] is this thread's TMEM lane ----
    if (ok) {
      tc_fence_after();
      float* grow = out + static_cast<size_t>(row) * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t gv[32];
        if (n_tiles > 0) {
          tmem_ld_x32(tmem + lane_addr + COL_G + c0, gv);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) gv[i] = 0u;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(grow + c0 + i) = make_float4(__uint_as_float(gv[i]), __uint_as_float(gv[i + 1]),
                                                                   __uint_as_float(gv[i + 2]), __uint_as_float(gv[i + 3]));
      }
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
static int launch_lin_q_tc(const sla_shape* s, const LinBwdParams& lp, cudaStream_t st) {
  constexpr int D = 128;
  const int bh = s->B * s->H;
  CUtensorMap tq, tdy, tdq, thw;
  int rc;
  if ((rc = make_tmap_3d(&tq, lp.q, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tdy, lp.d_o, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  if ((rc = make_tmap_3d(&tdq, lp.dq, s->dtype, D, s->L, bh, 128)) != SLA_OK) return rc;
  const char* hw = static_cast<const char*>(lp.lin_state) + (size_t(D) * D + D) * 2;   // H W^T behind H and z
  if ((rc = make_tmap_rows(&thw, hw, s->dtype, D, D, bh, size_t(2 * D * D + D) * 2, 64)) != SLA_OK) return rc;
  tc::LinQParams p;
  p.lin_state = lp.lin_state;
  p.g_partial = lp.g_partial;
  p.err = tc_error_word();
  if (p.err == nullptr) return SLA_ERR_CUDA;
  p.L = s->L; p.nch = lp.nch; p.rows = lp.rows; p.feature = s->feature_map; p.accumulate = lp.accumulate;
  auto kern = tc::linear_bwd_q_tc_kernel<T>;
  const int smem = 1024 + 3 * 2 * 128 * 128;
  SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  SLA_CUDA_OK(launch_pdl(kern, dim3(lp.nch, bh), dim3(192), smem, st, tq, tdy, tdq, thw, p));
  SLA_LAUNCH_OK();
  return SLA_OK;
}

// Head dim 128 and chunks that are whole tiles of 128 rows; SLA_ERR_UNSUPPORTED otherwise (the caller then runs the
// mma.sync pass A).
int run_linear_bwd_q_tc(const sla_shape* s, const LinBwdParams& lp, cudaStream_t st) {
  if (s->D != 128 || lp.rows % 128 != 0) return SLA_ERR_UNSUPPORTED;
  return s->dtype == SLA_BF16 ? launch_lin_q_tc<__nv_bfloat16>(s, lp, st) : launch_lin_q_tc<__half>(s, lp, st);
}

}  // namespace sla
