// Block-mask prediction: K column mean -> pooled Q / pooled (K - mean) -> pooled scores -> per-row
// top-k -> block LUT (+ optional 0/1 map and per-KV-block column lists).
// Follows sparse_linear_attention/utils.py:21-67 including its rounding points: the column mean, the
// smoothed K, the pooled means and the pooled scores are each rounded to the input dtype.
// All kernels here are HBM/L2-bound streaming, integer and compare work; the one contraction (pooled Q x pooled K,
// 3 MB of operands) runs on mma.sync for 16-bit inputs.
#include <type_traits>

#include "common.cuh"
#include "workspace.h"

namespace sla {

template <typename TIn>
struct VecLoad {
  static constexpr int N = 16 / sizeof(TIn);
  __device__ static inline void load(float (&out)[N], const TIn* p) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const TIn* e = reinterpret_cast<const TIn*>(&raw);
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = Elem<TIn>::to_f(e[i]);
  }
};

// ---- 1. column sums of K over chunks of rows: partial[bh][chunk][D] (fp32) ----
template <typename TIn, int D>
__global__ void __launch_bounds__(256) colsum_kernel(const TIn* __restrict__ k, float* __restrict__ partial,
                                                     int L, int nch) {
  constexpr int N = VecLoad<TIn>::N;
  constexpr int TPR = D / N;       // threads per row
  constexpr int RP = 256 / TPR;    // rows per pass
  __shared__ float red[RP][D];
  pdl_wait();
  int bh = blockIdx.y, ch = blockIdx.x;
  int tid = threadIdx.x, rg = tid / TPR, c = (tid % TPR) * N;
  int row0 = ch * kColsumRows, row1 = min(L, row0 + kColsumRows);
  const TIn* base = k + static_cast<size_t>(bh) * L * D;
  float acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.f;
#pragma unroll 8
  for (int r = row0 + rg; r < row1; r += RP) {   // unrolled so that several loads are in flight per thread
    float v[N];
    VecLoad<TIn>::load(v, base + static_cast<size_t>(r) * D + c);
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] += v[i];
  }
#pragma unroll
  for (int i = 0; i < N; ++i) red[rg][c + i] = acc[i];
  __syncthreads();
  if (tid < D) {
    float s = 0.f;
#pragma unroll 4
    for (int g = 0; g < RP; ++g) s += red[g][tid];
    partial[(static_cast<size_t>(bh) * nch + ch) * D + tid] = s;
  }
}

// ---- 2. mean[bh][d] = round_T(sum / L) (torch.mean keeps the input dtype, utils.py:56) ----
template <typename TIn>
__global__ void kmean_finalize_kernel(const float* __restrict__ partial, float* __restrict__ kmean, int L,
                                      int nch, int D) {
  pdl_wait();
  int bh = blockIdx.x, d = threadIdx.x;
  if (d >= D) return;
  float s = 0.f;
  for (int c = 0; c < nch; ++c) s += partial[(static_cast<size_t>(bh) * nch + c) * D + d];
  kmean[static_cast<size_t>(bh) * D + d] = round_to<TIn>(s / static_cast<float>(L));
}

// ---- 3. mean pooling of Q and of K - mean, utils.py:21-40 ----
// One warp pools one block: a row is D / N lanes of 16 bytes, so a warp-wide load covers 32 * N / D rows and every
// lane keeps N running sums; the row groups are folded with shuffles at the end. Eight blocks per CTA.
constexpr int kPoolWarps = 8;

template <typename TIn, int D, bool IS_K>
__device__ inline void pool_blocks(const TIn* __restrict__ x, const float* __restrict__ kmean,
                                   TIn* __restrict__ pooled, int L, int blk, int nblk) {
  constexpr int N = VecLoad<TIn>::N;
  constexpr int TPR = D / N;        // lanes per row
  constexpr int RPW = 32 / TPR;     // rows per warp-wide load
  static_assert(TPR <= 32 && 32 % TPR == 0, "a row is a whole fraction of a warp");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ib = blockIdx.x * kPoolWarps + warp, bh = blockIdx.y;
  if (ib >= nblk) return;
  const int rg = lane / TPR, c = (lane % TPR) * N;
  const int row0 = ib * blk, row1 = min(L, row0 + blk);
  const TIn* base = x + static_cast<size_t>(bh) * L * D + c;
  float mean[N];
#pragma unroll
  for (int i = 0; i < N; ++i) mean[i] = IS_K ? kmean[static_cast<size_t>(bh) * D + c + i] : 0.f;
  float acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.f;
#pragma unroll 8
  for (int r = row0 + rg; r < row1; r += RPW) {
    float v[N];
    VecLoad<TIn>::load(v, base + static_cast<size_t>(r) * D);
    if constexpr (IS_K && sizeof(TIn) == 2) {
      // K - mean rounded to the 16-bit type two at a time: the packed conversion does not go through the SFU pipe
#pragma unroll
      for (int i = 0; i < N; i += 2) {
        const float2 r = Elem<TIn>::unpack2(Elem<TIn>::pack2(v[i] - mean[i], v[i + 1] - mean[i + 1]));
        acc[i] += r.x;
        acc[i + 1] += r.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += IS_K ? round_to<TIn>(v[i] - mean[i]) : v[i];
    }
  }
#pragma unroll
  for (int o = 16; o >= TPR; o >>= 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
  if (rg == 0) {
    const float nx = static_cast<float>(row1 - row0);
    alignas(16) TIn o[N];
#pragma unroll
    for (int i = 0; i < N; ++i) o[i] = Elem<TIn>::from_f(acc[i] / nx);
    *reinterpret_cast<uint4*>(pooled + (static_cast<size_t>(bh) * nblk + ib) * D + c) = *reinterpret_cast<uint4*>(o);
  }
}

// z = 0: Q, z = 1: K - mean
template <typename TIn, int D>
__global__ void __launch_bounds__(kPoolWarps * 32) pool_kernel(const TIn* __restrict__ q, const TIn* __restrict__ k,
                                                               const float* __restrict__ kmean,
                                                               TIn* __restrict__ pooled_q, TIn* __restrict__ pooled_k,
                                                               int L, int blkq, int blkk, int mb, int nb) {
  pdl_wait();
  if (blockIdx.z == 0) pool_blocks<TIn, D, false>(q, nullptr, pooled_q, L, blkq, mb);
  else pool_blocks<TIn, D, true>(k, kmean, pooled_k, L, blkk, nb);
}

// ---- 4. pooled scores + per-row top-k ----
__device__ inline uint32_t order_key(float x) {
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One warp selects the top-k of one row of order-preserving keys (shared memory, nb of them) by a bitwise search
// for the k-th largest key and writes the selected indices in ascending order; ties at the k-th score go to the
// lower index.
template <typename TIn>
__device__ inline void select_topk_row(const uint32_t* kr, int nb, int topk, int lane, int32_t* out,
                                       int8_t* map_row, int32_t* cols) {
  // Key of the topk-th largest element, one bit at a time from the top: the largest value v with
  // count(key >= v) >= topk. Counting is a compare and an add per key and one warp reduction per bit; no
  // histogram, so rows whose scores share their high bits (all of them) cost the same as any other.
  // The first 32 * kKeyRegs keys of the row sit in registers (all of them up to 512 KV blocks), the rest is re-read
  // from shared memory; a missing key is 0, below every candidate (a candidate has at least one bit set).
  constexpr int kKeyRegs = 16;
  uint32_t kreg[kKeyRegs];
#pragma unroll
  for (int i = 0; i < kKeyRegs; ++i) kreg[i] = lane + 32 * i < nb ? kr[lane + 32 * i] : 0u;
  // Scores were rounded to TIn, so the kLowZero low bits of a score's fp32 pattern are clear. order_key() keeps
  // them clear for a non-negative score and turns them all into ones for a negative one (it complements the
  // pattern). Keys that agree above bit kLowZero have the same sign, hence the same low bits: the search only
  // has to decide the high bits, and the low bits follow from the sign of what it found.
  constexpr int kLowZero = std::is_same<TIn, __nv_bfloat16>::value ? 16 : (std::is_same<TIn, __half>::value ? 13 : 0);
  uint32_t prefix = 0;
  for (int bit = 31; bit >= kLowZero; --bit) {
    const uint32_t cand = prefix | (1u << bit);
    int c0 = 0, c1 = 0;
#pragma unroll
    for (int i = 0; i < kKeyRegs; i += 2) {
      c0 += kreg[i] >= cand ? 1 : 0;
      c1 += kreg[i + 1] >= cand ? 1 : 0;
    }
    for (int j = lane + 32 * kKeyRegs; j < nb; j += 32) c0 += kr[j] >= cand ? 1 : 0;
    if (__reduce_add_sync(0xffffffffu, c0 + c1) >= topk) prefix = cand;
  }
  if (kLowZero > 0 && !(prefix & 0x80000000u)) prefix |= (1u << kLowZero) - 1u;   // k-th score is negative
  int above = 0;
#pragma unroll
  for (int i = 0; i < kKeyRegs; ++i) above += kreg[i] > prefix ? 1 : 0;
  for (int j = lane + 32 * kKeyRegs; j < nb; j += 32) above += kr[j] > prefix ? 1 : 0;
  const int need = topk - __reduce_add_sync(0xffffffffu, above);
  const uint32_t thr = prefix;  // key of the k-th largest; `need` of the elements equal to it are taken
  int n_out = 0, eq_seen = 0;
  const uint32_t lt_mask = (1u << lane) - 1u;
  int n_eq = 0;
#pragma unroll
  for (int i = 0; i < kKeyRegs; ++i) n_eq += kreg[i] == thr ? 1 : 0;
  for (int j = lane + 32 * kKeyRegs; j < nb; j += 32) n_eq += kr[j] == thr ? 1 : 0;
  if (__reduce_add_sync(0xffffffffu, n_eq) == need) {
    // no surplus ties at the threshold (nearly every row): exactly topk keys are >= thr, one ballot per 32 keys
#pragma unroll 4
    for (int base = 0; base < nb; base += 32) {
      const int j = base + lane;
      const bool sel = j < nb && kr[j] >= thr;
      const uint32_t bs = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        out[n_out + __popc(bs & lt_mask)] = j;
        if (cols) atomicAdd(&cols[j + 1], 1);
      }
      if (map_row && j < nb) map_row[j] = sel ? 1 : 0;
      n_out += __popc(bs);
    }
    return;
  }
  for (int base = 0; base < nb; base += 32) {
    int j = base + lane;
    uint32_t key = j < nb ? kr[j] : 0u;
    bool gt = j < nb && key > thr;
    bool eq = j < nb && key == thr;
    uint32_t be = __ballot_sync(0xffffffffu, eq);
    int eq_rank = eq_seen + __popc(be & lt_mask);
    bool sel = gt || (eq && eq_rank < need);
    uint32_t bs = __ballot_sync(0xffffffffu, sel);
    // a row never emits more than topk entries, whatever the scores are (NaNs included): the LUT row, the 0/1
    // map and the column counts are sized for exactly topk
    sel = sel && n_out + __popc(bs & lt_mask) < topk;
    bs = __ballot_sync(0xffffffffu, sel);
    if (sel) {
      out[n_out + __popc(bs & lt_mask)] = j;
      if (cols) atomicAdd(&cols[j + 1], 1);
    }
    if (map_row && j < nb) map_row[j] = sel ? 1 : 0;
    n_out += __popc(bs);
    eq_seen += __popc(be);
  }
}

constexpr int kTopkRows = 8;  // query-block rows per CTA == warps per CTA
constexpr int kScoreStages = 5;   // depth of each thread's private prefetch ring of pooled-K chunks

// One CTA scores kTopkRows query-block rows against every KV block of the head, then each warp
// selects the top-k of one row by a bitwise search for the k-th largest order-preserving key and writes the
// selected indices in ascending order; ties at the k-th score go to the lower index.
template <typename TIn, int D>
__global__ void __launch_bounds__(kTopkRows * 32) score_topk_kernel(
    const TIn* __restrict__ pooled_q, const TIn* __restrict__ pooled_k, int32_t* __restrict__ lut,
    int8_t* __restrict__ sparse_map, int32_t* __restrict__ col_offsets, int mb, int nb, int topk) {
  constexpr int N = VecLoad<TIn>::N;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float2* spq = reinterpret_cast<float2*>(smem_raw);                      // [R][D], every value twice: (q, q)
  uint32_t* keys = reinterpret_cast<uint32_t*>(spq + kTopkRows * D);       // [R][nb]
  const int bh = blockIdx.y, row_base = blockIdx.x * kTopkRows;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();

  for (int i = tid; i < kTopkRows * D; i += blockDim.x) {
    int r = i / D, d = i % D;
    int row = row_base + r;
    const float qv = row < mb ? Elem<TIn>::to_f(pooled_q[(static_cast<size_t>(bh) * mb + row) * D + d]) : 0.f;
    spq[i] = make_float2(qv, qv);
  }
  __syncthreads();

  const TIn* pk = pooled_k + static_cast<size_t>(bh) * nb * D;
  unsigned char* ring = reinterpret_cast<unsigned char*>(keys + kTopkRows * nb);   // [stages][2][threads] x 16 B
  auto slot_off = [&](int st, int h) { return ((st * 2 + h) * (kTopkRows * 32) + tid) * 16; };
  auto slot = [&](int st, int h) { return smem_u32(ring) + slot_off(st, h); };
  // two KV blocks per thread and pass, their two sums kept as the halves of one packed fp32 FMA (fma.rn.f32x2:
  // two independent round-to-nearest FMAs, so each score is still one sequential fp32 sum over d)
  for (int j = tid; j < nb; j += 2 * blockDim.x) {
    const int j1 = j + blockDim.x;
    const bool has1 = j1 < nb;
    const TIn* k0 = pk + static_cast<size_t>(j) * D;
    const TIn* k1 = pk + static_cast<size_t>(has1 ? j1 : j) * D;
    float2 acc[kTopkRows];       // .x: block j, .y: block j1
#pragma unroll
    for (int r = 0; r < kTopkRows; ++r) acc[r] = make_float2(0.f, 0.f);
    // The two pooled-K rows of this thread come through a private ring of 16-byte slots filled by cp.async
    // kScoreStages - 1 steps ahead: a thread's own loads are 256 bytes apart from its neighbours', so what bounds
    // this loop is the latency of those loads, not their number.
#pragma unroll
    for (int st = 0; st < kScoreStages - 1; ++st) {
      cp_async16(slot(st, 0), k0 + st * N, true);
      cp_async16(slot(st, 1), k1 + st * N, true);
      cp_async_commit();
    }
#pragma unroll
    for (int ci = 0; ci < D / N; ++ci) {
      const int c = ci * N, pf = ci + kScoreStages - 1;
      if (pf < D / N) {
        cp_async16(slot(pf % kScoreStages, 0), k0 + pf * N, true);
        cp_async16(slot(pf % kScoreStages, 1), k1 + pf * N, true);
      }
      cp_async_commit();
      cp_async_wait<kScoreStages - 1>();
      float kv0[N], kv1[N];
      VecLoad<TIn>::load(kv0, reinterpret_cast<const TIn*>(ring + slot_off(ci % kScoreStages, 0)));
      VecLoad<TIn>::load(kv1, reinterpret_cast<const TIn*>(ring + slot_off(ci % kScoreStages, 1)));
#pragma unroll
      for (int r = 0; r < kTopkRows; ++r) {
#pragma unroll
        for (int e = 0; e < N; e += 2) {
          const float4 qq = *reinterpret_cast<const float4*>(spq + r * D + c + e);   // (q_e, q_e, q_e+1, q_e+1)
          acc[r] = __ffma2_rn(make_float2(qq.x, qq.y), make_float2(kv0[e], kv1[e]), acc[r]);
          acc[r] = __ffma2_rn(make_float2(qq.z, qq.w), make_float2(kv0[e + 1], kv1[e + 1]), acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kTopkRows; ++r) {
      keys[r * nb + j] = order_key(round_to<TIn>(acc[r].x));  // utils.py:59
      if (has1) keys[r * nb + j1] = order_key(round_to<TIn>(acc[r].y));
    }
  }
  __syncthreads();

  const int row = row_base + warp;
  if (row >= mb) return;
  select_topk_row<TIn>(keys + warp * nb, nb, topk, lane, lut + (static_cast<size_t>(bh) * mb + row) * topk,
                       sparse_map ? sparse_map + (static_cast<size_t>(bh) * mb + row) * nb : nullptr,
                       col_offsets ? col_offsets + static_cast<size_t>(bh) * (nb + 1) : nullptr);
}

// ---- 4b. the same for 16-bit inputs, scores on the tensor cores ----
// One CTA scores kMmaRows query-block rows against every KV block of the head with mma.m16n8k16 (fp32 accumulate;
// the products of two 16-bit values are exact in fp32, so only the order of the fp32 additions differs from the
// scalar kernel above, as it does from any other GEMM), rounds each score to the input type (utils.py:59) and
// selects per row as above. Operands go from global memory straight into fragments: the contraction index is
// permuted so that a thread's share of 32 consecutive dimensions is the 16 contiguous bytes [8t, 8t + 8), the same
// permutation on both operands, which leaves every dot product unchanged.
constexpr int kMmaRows = 16;
__host__ __device__ inline int score_key_stride(int nb) { return (nb + 31) / 32 * 32 + 8; }
constexpr int kMmaWarps = 16;   // one row per warp in the selection phase

template <typename TIn, int D>
__global__ void __launch_bounds__(kMmaWarps * 32, 2) score_topk_mma_kernel(
    const TIn* __restrict__ pooled_q, const TIn* __restrict__ pooled_k, int32_t* __restrict__ lut,
    int8_t* __restrict__ sparse_map, int32_t* __restrict__ col_offsets, int mb, int nb, int topk) {
  static_assert(D % 32 == 0, "head dimension in steps of 32");
  constexpr int KP = D / 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint32_t* keys = reinterpret_cast<uint32_t*>(smem_raw);   // [kMmaRows][stride]
  const int stride = score_key_stride(nb);
  const int bh = blockIdx.y, row_base = blockIdx.x * kMmaRows;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  pdl_wait();

  // rows past the last query block repeat it; their scores are never selected from
  const TIn* q0 = pooled_q + (static_cast<size_t>(bh) * mb + min(row_base + g, mb - 1)) * D + t * 8;
  const TIn* q1 = pooled_q + (static_cast<size_t>(bh) * mb + min(row_base + g + 8, mb - 1)) * D + t * 8;
  uint4 a0[KP], a1[KP];
#pragma unroll
  for (int kp = 0; kp < KP; ++kp) {
    a0[kp] = __ldg(reinterpret_cast<const uint4*>(q0 + kp * 32));
    a1[kp] = __ldg(reinterpret_cast<const uint4*>(q1 + kp * 32));
  }
  const TIn* pkh = pooled_k + static_cast<size_t>(bh) * nb * D;
  const int ntiles = (nb + 7) / 8;
#pragma unroll 2
  for (int nt = warp; nt < ntiles; nt += kMmaWarps) {
    const TIn* kr = pkh + static_cast<size_t>(min(nt * 8 + g, nb - 1)) * D + t * 8;
    uint4 b[KP];
#pragma unroll
    for (int kp = 0; kp < KP; ++kp) b[kp] = __ldg(reinterpret_cast<const uint4*>(kr + kp * 32));
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kp = 0; kp < KP; ++kp) {
      const uint32_t lo[4] = {a0[kp].x, a1[kp].x, a0[kp].y, a1[kp].y};
      const uint32_t hi[4] = {a0[kp].z, a1[kp].z, a0[kp].w, a1[kp].w};
      mma16816<TIn>(acc, lo, b[kp].x, b[kp].y);
      mma16816<TIn>(acc, hi, b[kp].z, b[kp].w);
    }
    // a row of keys is `stride` words, a multiple of 32 plus 8: the 8-byte stores of a half-warp (g = 0..3,
    // t = 0..3) then fall on 32 different banks; the words past nb are padding that nothing reads
    const int c = nt * 8 + 2 * t;
    *reinterpret_cast<uint2*>(keys + g * stride + c) =
        make_uint2(order_key(round_to<TIn>(acc[0])), order_key(round_to<TIn>(acc[1])));
    *reinterpret_cast<uint2*>(keys + (g + 8) * stride + c) =
        make_uint2(order_key(round_to<TIn>(acc[2])), order_key(round_to<TIn>(acc[3])));
  }
  __syncthreads();

  for (int r = warp; r < kMmaRows; r += kMmaWarps) {
    const int row = row_base + r;
    if (row >= mb) break;
    select_topk_row<TIn>(keys + r * stride, nb, topk, lane, lut + (static_cast<size_t>(bh) * mb + row) * topk,
                         sparse_map ? sparse_map + (static_cast<size_t>(bh) * mb + row) * nb : nullptr,
                         col_offsets ? col_offsets + static_cast<size_t>(bh) * (nb + 1) : nullptr);
  }
}

// ---- 5. column lists: in-place inclusive scan of the per-column counts ----
__global__ void __launch_bounds__(1024) col_scan_kernel(int32_t* __restrict__ col_offsets, int nb) {
  __shared__ int32_t warp_tot[32];
  pdl_wait();
  int32_t* c = col_offsets + static_cast<size_t>(blockIdx.x) * (nb + 1);
  int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int per = (nb + 1 + 1023) / 1024;
  int lo = tid * per, hi = min(nb + 1, lo + per);
  int32_t s = 0;
  for (int i = lo; i < hi; ++i) s += c[i];
  int32_t incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int32_t w = warp_tot[lane], wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_tot[lane] = wi - w;
  }
  __syncthreads();
  int32_t run = warp_tot[warp] + incl - s;
  for (int i = lo; i < hi; ++i) {
    run += c[i];
    c[i] = run;
  }
}

// ---- 6. column lists: for KV block j the ascending list of query blocks whose row selects j ----
// One CTA fills the lists of 32 neighbouring KV blocks: a thread reads the 32 map bytes of one query-block row (one
// 32-byte sector), each warp transposes its 32 x 32 bits with ballots so that lane c holds column c's rows, and
// the position of a warp's first entry in a column is the column's running offset plus the counts of the warps
// below it. Rows go in ascending order: passes, then warps, then bits.
__global__ void __launch_bounds__(1024) col_fill_kernel(const int8_t* __restrict__ sparse_map,
                                                        const int32_t* __restrict__ col_offsets,
                                                        int32_t* __restrict__ col_index, int mb, int nb,
                                                        int topk) {
  __shared__ int32_t cnt[32][33];   // [warp][column]
  __shared__ int32_t col_pos[32];   // next free position of each column
  pdl_wait();
  const int bh = blockIdx.y, j0 = blockIdx.x * 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int8_t* m = sparse_map + static_cast<size_t>(bh) * mb * nb;
  int32_t* out = col_index + static_cast<size_t>(bh) * mb * topk;
  if (warp == 0) col_pos[lane] = j0 + lane < nb ? col_offsets[static_cast<size_t>(bh) * (nb + 1) + j0 + lane] : 0;
  const bool vec = nb % 16 == 0 && j0 + 32 <= nb &&
                   (reinterpret_cast<uintptr_t>(sparse_map) & 15) == 0;   // every row's 32 bytes 16-byte aligned
  auto nonzero4 = [](uint32_t w) {   // bit b set when byte b of w is not zero
    uint32_t y = __vcmpne4(w, 0u) & 0x08040201u;
    return (y | (y >> 8) | (y >> 16) | (y >> 24)) & 0xfu;
  };
  for (int i0 = 0; i0 < mb; i0 += 1024) {
    const int i = i0 + tid;
    uint32_t mask = 0;
    if (i < mb) {
      const int8_t* row = m + static_cast<size_t>(i) * nb + j0;
      if (vec) {
        const uint4 x = *reinterpret_cast<const uint4*>(row), y = *reinterpret_cast<const uint4*>(row + 16);
        mask = nonzero4(x.x) | nonzero4(x.y) << 4 | nonzero4(x.z) << 8 | nonzero4(x.w) << 12 |
               nonzero4(y.x) << 16 | nonzero4(y.y) << 20 | nonzero4(y.z) << 24 | nonzero4(y.w) << 28;
      } else {
        for (int c = 0; c < 32 && j0 + c < nb; ++c) mask |= row[c] != 0 ? 1u << c : 0u;
      }
    }
    uint32_t colbits = 0;   // lane c: which of this warp's 32 rows select column j0 + c
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const uint32_t b = __ballot_sync(0xffffffffu, (mask >> c) & 1u);
      if (lane == c) colbits = b;
    }
    cnt[warp][lane] = __popc(colbits);
    __syncthreads();
    int pos = col_pos[lane];
    for (int w = 0; w < warp; ++w) pos += cnt[w][lane];
    while (colbits) {
      out[pos++] = i0 + warp * 32 + __ffs(colbits) - 1;
      colbits &= colbits - 1;
    }
    __syncthreads();
    if (warp == 0) {
      int tot = 0;
#pragma unroll 8
      for (int w = 0; w < 32; ++w) tot += cnt[w][lane];
      col_pos[lane] += tot;
    }
    __syncthreads();
  }
}

// ---- 6b. per-column counts straight from a 0/1 map (for maps not produced by sla_block_map) ----
__global__ void __launch_bounds__(1024) col_count_kernel(const int8_t* __restrict__ sparse_map,
                                                         int32_t* __restrict__ col_offsets, int mb, int nb) {
  int bh = blockIdx.y;
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int j = blockIdx.x * 32 + warp;
  if (j >= nb) return;
  const int8_t* m = sparse_map + static_cast<size_t>(bh) * mb * nb;
  int cnt = 0;
  for (int i0 = 0; i0 < mb; i0 += 32) {
    int i = i0 + lane;
    bool f = i < mb && m[static_cast<size_t>(i) * nb + j] != 0;
    cnt += __popc(__ballot_sync(0xffffffffu, f));
  }
  if (lane == 0) col_offsets[static_cast<size_t>(bh) * (nb + 1) + j + 1] = cnt;
}

template <typename TIn, int D>
static int score_and_select(const sla_shape* s, const TIn* pq, const TIn* pk, int32_t* lut, int8_t* sparse_map,
                            int32_t* col_offsets, int32_t* col_index, cudaStream_t st);

template <typename TIn, int D>
static int launch_block_map(const sla_shape* s, const TIn* q, const TIn* k, int32_t* lut, int8_t* sparse_map,
                            int32_t* col_offsets, int32_t* col_index, unsigned char* ws, cudaStream_t st) {
  const int bh = s->B * s->H, L = s->L;
  const int mb = ceil_div(L, s->BLKQ), nb = ceil_div(L, s->BLKK);
  WsBlockMap w = ws_block_map(s);
  float* partial = reinterpret_cast<float*>(ws + w.colsum_partial);
  float* kmean = reinterpret_cast<float*>(ws + w.kmean);
  TIn* pq = reinterpret_cast<TIn*>(ws + w.pooled_q);
  TIn* pk = reinterpret_cast<TIn*>(ws + w.pooled_k);
  const bool want_cols = col_offsets != nullptr && col_index != nullptr;
  if (want_cols && sparse_map == nullptr) sparse_map = reinterpret_cast<int8_t*>(ws + w.map);

  SLA_CUDA_OK(launch_pdl<false>(colsum_kernel<TIn, D>, dim3(w.nch, bh), dim3(256), 0, st, k, partial, L, w.nch));
  SLA_LAUNCH_OK();
  SLA_CUDA_OK(launch_pdl<false>(kmean_finalize_kernel<TIn>, dim3(bh), dim3(D), 0, st, partial, kmean, L, w.nch, D));
  SLA_LAUNCH_OK();
  SLA_CUDA_OK(launch_pdl<false>(pool_kernel<TIn, D>, dim3(ceil_div(max(mb, nb), kPoolWarps), bh, 2),
                                dim3(kPoolWarps * 32), 0, st, q, k, static_cast<const float*>(kmean), pq, pk, L,
                                s->BLKQ, s->BLKK, mb, nb));
  SLA_LAUNCH_OK();
  return score_and_select<TIn, D>(s, pq, pk, lut, sparse_map, col_offsets, col_index, st);
}

// pooled Q, pooled smoothed K (in the input dtype) -> LUT, optional 0/1 map and column lists
template <typename TIn, int D>
static int score_and_select(const sla_shape* s, const TIn* pq, const TIn* pk, int32_t* lut, int8_t* sparse_map,
                            int32_t* col_offsets, int32_t* col_index, cudaStream_t st) {
  const int bh = s->B * s->H, L = s->L;
  const int mb = ceil_div(L, s->BLKQ), nb = ceil_div(L, s->BLKK);
  const bool want_cols = col_offsets != nullptr && col_index != nullptr;
  if (want_cols) SLA_CUDA_OK(cudaMemsetAsync(col_offsets, 0, sizeof(int32_t) * size_t(bh) * (nb + 1), st));
  if constexpr (sizeof(TIn) == 2) {
    const size_t smem = size_t(kMmaRows) * score_key_stride(nb) * 4;
    if (smem > 200 * 1024) return SLA_ERR_BAD_SHAPE;
    auto kern = score_topk_mma_kernel<TIn, D>;
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    SLA_CUDA_OK(launch_pdl<false>(kern, dim3(ceil_div(mb, kMmaRows), bh), dim3(kMmaWarps * 32), smem, st, pq, pk, lut,
                                  sparse_map, want_cols ? col_offsets : nullptr, mb, nb, s->topk));
    SLA_LAUNCH_OK();
  } else {
    // fp32 inputs: the scalar kernel (one sequential fp32 sum per score)
    const size_t smem =
        (size_t(kTopkRows) * (2 * D + nb) * 4 + 15) / 16 * 16 + size_t(kScoreStages) * 2 * kTopkRows * 32 * 16;
    if (smem > 200 * 1024) return SLA_ERR_BAD_SHAPE;
    auto kern = score_topk_kernel<TIn, D>;
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    SLA_CUDA_OK(launch_pdl<false>(kern, dim3(ceil_div(mb, kTopkRows), bh), dim3(kTopkRows * 32), smem, st, pq, pk, lut,
                                  sparse_map, want_cols ? col_offsets : nullptr, mb, nb, s->topk));
    SLA_LAUNCH_OK();
  }
  if (want_cols) {
    SLA_CUDA_OK(launch_pdl<false>(col_scan_kernel, dim3(bh), dim3(1024), 0, st, col_offsets, nb));
    SLA_LAUNCH_OK();
    SLA_CUDA_OK(launch_pdl<false>(col_fill_kernel, dim3(ceil_div(nb, 32), bh), dim3(1024), 0, st,
                           static_cast<const int8_t*>(sparse_map), static_cast<const int32_t*>(col_offsets), col_index,
                           mb, nb, s->topk));
    SLA_LAUNCH_OK();
  }
  return SLA_OK;
}

// Column mean of K per head, rounded to the element type (what k.mean(dim=-2) returns): used by the
// SageSLA path (SageSLA/core.py:102). partial: fp32 [BH][ceil(L/512)][D]; kmean: fp32 [BH][D].
template <typename TIn, int D>
static int k_mean_typed(const sla_shape* s, const TIn* k, float* partial, float* kmean, cudaStream_t st) {
  const int bh = s->B * s->H, nch = ceil_div(s->L, kColsumRows);
  colsum_kernel<TIn, D><<<dim3(nch, bh), 256, 0, st>>>(k, partial, s->L, nch);
  SLA_LAUNCH_OK();
  kmean_finalize_kernel<TIn><<<bh, D, 0, st>>>(partial, kmean, s->L, nch, D);
  SLA_LAUNCH_OK();
  return SLA_OK;
}
int run_k_mean(const sla_shape* s, const void* k, float* partial, float* kmean, cudaStream_t st) {
  if (s->dtype == SLA_BF16)
    return s->D == 64 ? k_mean_typed<__nv_bfloat16, 64>(s, (const __nv_bfloat16*)k, partial, kmean, st)
                      : k_mean_typed<__nv_bfloat16, 128>(s, (const __nv_bfloat16*)k, partial, kmean, st);
  return s->D == 64 ? k_mean_typed<__half, 64>(s, (const __half*)k, partial, kmean, st)
                    : k_mean_typed<__half, 128>(s, (const __half*)k, partial, kmean, st);
}

}  // namespace sla

namespace sla {
// ---- 8. the step before the path: per-head RMS norm and rotary embedding of q and k, with the block sums the mask
// prediction needs taken from the rows while they are in registers ----
// One CTA = one block of rows of one head (z = 0: a query block, z = 1: a KV block). A row is spread over D/8
// threads with 16-byte loads and stores. Per row: y = x * rsqrt(mean(x^2) + eps) * g (skipped when g is NULL), then
// the rotation of each pair by the row's angles (skipped when cos is NULL): pairs are (y[2i], y[2i+1]) when
// `interleaved`, else (y[i], y[i + D/2]). The result is rounded to T, stored, and the ROUNDED values are summed per
// column into sums[bh][block][D] (fp32): the mask prediction then starts from the same bits a separate pooling
// pass over the stored tensor would read.
template <typename T, int D>
__global__ void __launch_bounds__(256) qk_norm_rope_pool_kernel(
    const T* __restrict__ q_in, const T* __restrict__ k_in, const float* __restrict__ gq, const float* __restrict__ gk,
    const float* __restrict__ cs, const float* __restrict__ sn, float eps, int interleaved, T* __restrict__ q_out,
    T* __restrict__ k_out, float* __restrict__ qsum, float* __restrict__ ksum, int L, int blkq, int blkk) {
  constexpr int TPR = D / 8;       // threads per row
  constexpr int RP = 256 / TPR;    // rows per pass
  __shared__ float red[RP][D];
  const bool is_k = blockIdx.z == 1;
  const int blk = is_k ? blkk : blkq;
  const int nblk = (L + blk - 1) / blk;
  if (static_cast<int>(blockIdx.x) >= nblk) return;
  const int bh = blockIdx.y, ib = blockIdx.x;
  const int tid = threadIdx.x, rg = tid / TPR, c = (tid % TPR) * 8;
  const int row0 = ib * blk, row1 = min(L, row0 + blk);
  const T* src = (is_k ? k_in : q_in) + static_cast<size_t>(bh) * L * D;
  T* dst = (is_k ? k_out : q_out) + static_cast<size_t>(bh) * L * D;
  const float* gw = is_k ? gk : gq;
  float g8[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) g8[i] = gw ? gw[c + i] : 1.f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // every thread runs the same number of passes (the shuffles below need the whole row group); rows past the
  // block are computed on zeros and dropped
  const int passes = (blk + RP - 1) / RP;
  for (int it = 0; it < passes; ++it) {
    const int r = row0 + it * RP + rg;
    const bool live = r < row1;
    float x[8];
    if (live) {
      uint4 raw = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * D + c);
      const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = Elem<T>::unpack2(w[i]);
        x[2 * i] = f.x; x[2 * i + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = 0.f;
    }
    if (gw != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
      for (int o = 1; o < TPR; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = x[i] * inv * g8[i];
    }
    if (cs != nullptr) {
      const int rr = live ? r : 0;
      const float* cr = cs + static_cast<size_t>(rr) * (D / 2);
      const float* sr = sn + static_cast<size_t>(rr) * (D / 2);
      if (interleaved) {
        const float4 c4 = *reinterpret_cast<const float4*>(cr + c / 2), s4 = *reinterpret_cast<const float4*>(sr + c / 2);
        const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = x[2 * i], b = x[2 * i + 1];
          x[2 * i] = a * cc[i] - b * sv[i];
          x[2 * i + 1] = a * sv[i] + b * cc[i];
        }
      } else {
        // the partner of column j is column j +- D/2, held by the lane TPR/2 away in the same row group
        const bool upper = c >= D / 2;
        const int j0 = upper ? c - D / 2 : c;
        const float4 ca = *reinterpret_cast<const float4*>(cr + j0), cb = *reinterpret_cast<const float4*>(cr + j0 + 4);
        const float4 sa = *reinterpret_cast<const float4*>(sr + j0), sb = *reinterpret_cast<const float4*>(sr + j0 + 4);
        const float cc[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
        const float sv[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float other = __shfl_xor_sync(0xffffffffu, x[i], TPR / 2);
          x[i] = upper ? x[i] * cc[i] + other * sv[i] : x[i] * cc[i] - other * sv[i];
        }
      }
    }
    uint4 outv;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&outv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ow[i] = Elem<T>::pack2(x[2 * i], x[2 * i + 1]);
      const float2 f = Elem<T>::unpack2(ow[i]);
      if (live) { acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
    }
    if (live) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * D + c) = outv;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[rg][c + i] = acc[i];
  __syncthreads();
  if (tid < D) {
    float sm = 0.f;
#pragma unroll 4
    for (int g = 0; g < RP; ++g) sm += red[g][tid];
    float* out = (is_k ? ksum : qsum) + (static_cast<size_t>(bh) * nblk + ib) * D;
    out[tid] = sm;
  }
}

// Block sums -> what score_topk reads: kmean = round_T(sum_blocks ksum / L); pooled_q = round_T(qsum / nx);
// pooled_k = round_T(ksum / nx - kmean). The last line is where this path departs from utils.py:56 + :40, which
// round every element of k - mean(k) to T before pooling: the block mean of those rounding errors (well below one
// unit in the last place of the pooled value) is not reproduced.
// One CTA per head, 1024 threads = 8 groups of 128 columns: group g sums the blocks j = g (mod 8) with four loads in
// flight, the eight partial sums are added in a fixed order.
template <typename TIn>
__global__ void __launch_bounds__(1024) pooled_kmean_kernel(const float* __restrict__ ksum, float* __restrict__ kmean,
                                                            int L, int nb, int D) {
  __shared__ float part[8][128];
  const int bh = blockIdx.x, d = threadIdx.x & 127, g = threadIdx.x >> 7;
  const float* base = ksum + static_cast<size_t>(bh) * nb * D;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (d < D) {
    int j = g;
    for (; j + 24 < nb; j += 32) {
      s0 += base[static_cast<size_t>(j) * D + d];
      s1 += base[static_cast<size_t>(j + 8) * D + d];
      s2 += base[static_cast<size_t>(j + 16) * D + d];
      s3 += base[static_cast<size_t>(j + 24) * D + d];
    }
    for (; j < nb; j += 8) s0 += base[static_cast<size_t>(j) * D + d];
  }
  part[g][d] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (g == 0 && d < D) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += part[i][d];
    kmean[static_cast<size_t>(bh) * D + d] = round_to<TIn>(s / static_cast<float>(L));
  }
}
template <typename TIn>
__global__ void __launch_bounds__(256) pooled_finalize_kernel(const float* __restrict__ qsum, const float* __restrict__ ksum,
                                                              const float* __restrict__ kmean, TIn* __restrict__ pq,
                                                              TIn* __restrict__ pk, int L, int blkq, int blkk, int D) {
  const bool is_k = blockIdx.z == 1;
  const int blk = is_k ? blkk : blkq;
  const int nblk = (L + blk - 1) / blk;
  const int bh = blockIdx.y;
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i >= nblk * D) return;
  const int ib = i / D, d = i % D;
  const float nx = static_cast<float>(min(L, (ib + 1) * blk) - ib * blk);
  const size_t o = static_cast<size_t>(bh) * nblk * D + i;
  if (is_k) pk[o] = Elem<TIn>::from_f(ksum[o] / nx - kmean[static_cast<size_t>(bh) * D + d]);
  else pq[o] = Elem<TIn>::from_f(qsum[o] / nx);
}

static size_t pooled_sums_bytes(const sla_shape* s) {
  const size_t bh = size_t(s->B) * s->H;
  return ws_round(bh * ceil_div(s->L, s->BLKQ) * s->D * 4) + ws_round(bh * ceil_div(s->L, s->BLKK) * s->D * 4);
}

template <typename T, int D>
static int qk_prepare_typed(const sla_shape* s, const T* q_in, const T* k_in, const float* gq, const float* gk,
                            const float* cs, const float* sn, float eps, int interleaved, T* q_out, T* k_out,
                            unsigned char* sums, cudaStream_t st) {
  const int bh = s->B * s->H, mb = ceil_div(s->L, s->BLKQ), nb = ceil_div(s->L, s->BLKK);
  float* qsum = reinterpret_cast<float*>(sums);
  float* ksum = reinterpret_cast<float*>(sums + ws_round(size_t(bh) * mb * s->D * 4));
  qk_norm_rope_pool_kernel<T, D><<<dim3(max(mb, nb), bh, 2), 256, 0, st>>>(q_in, k_in, gq, gk, cs, sn, eps, interleaved,
                                                                            q_out, k_out, qsum, ksum, s->L, s->BLKQ,
                                                                            s->BLKK);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

template <typename TIn, int D>
static int block_map_pooled_typed(const sla_shape* s, const unsigned char* sums, int32_t* lut, int8_t* sparse_map,
                                  int32_t* col_offsets, int32_t* col_index, unsigned char* ws, cudaStream_t st) {
  const int bh = s->B * s->H, mb = ceil_div(s->L, s->BLKQ), nb = ceil_div(s->L, s->BLKK);
  const float* qsum = reinterpret_cast<const float*>(sums);
  const float* ksum = reinterpret_cast<const float*>(sums + ws_round(size_t(bh) * mb * s->D * 4));
  WsBlockMap w = ws_block_map(s);
  float* kmean = reinterpret_cast<float*>(ws + w.kmean);
  TIn* pq = reinterpret_cast<TIn*>(ws + w.pooled_q);
  TIn* pk = reinterpret_cast<TIn*>(ws + w.pooled_k);
  if (col_offsets != nullptr && sparse_map == nullptr) sparse_map = reinterpret_cast<int8_t*>(ws + w.map);
  pooled_kmean_kernel<TIn><<<bh, 1024, 0, st>>>(ksum, kmean, s->L, nb, D);
  SLA_LAUNCH_OK();
  pooled_finalize_kernel<TIn><<<dim3(ceil_div(max(mb, nb) * D, 256), bh, 2), 256, 0, st>>>(qsum, ksum, kmean, pq, pk, s->L,
                                                                                          s->BLKQ, s->BLKK, D);
  SLA_LAUNCH_OK();
  return score_and_select<TIn, D>(s, pq, pk, lut, sparse_map, col_offsets, col_index, st);
}
}  // namespace sla

extern "C" size_t sla_pooled_sums_bytes(const sla_shape* s) { return s ? sla::pooled_sums_bytes(s) : 0; }

extern "C" int sla_qk_norm_rope_pool(const sla_shape* s, const void* q_in, const void* k_in, const float* gq,
                                     const float* gk, const float* rope_cos, const float* rope_sin, float eps,
                                     int interleaved, void* q_out, void* k_out, void* pooled_sums, size_t sums_bytes,
                                     sla_stream_t stream) {
  using namespace sla;
  if (!s || !q_in || !k_in || !q_out || !k_out || !pooled_sums) return SLA_ERR_NULL;
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) return SLA_ERR_NULL;
  if (s->B < 1 || s->H < 1 || s->L < 1 || (s->D != 64 && s->D != 128)) return SLA_ERR_BAD_SHAPE;
  if (s->BLKQ < 16 || s->BLKK < 16 || s->BLKQ > 1024 || s->BLKK > 1024) return SLA_ERR_BAD_SHAPE;
  if (static_cast<long long>(s->B) * s->H > 65535) return SLA_ERR_BAD_SHAPE;
  if (s->dtype != SLA_BF16 && s->dtype != SLA_FP16) return SLA_ERR_BAD_DTYPE;
  if (!aligned16(q_in) || !aligned16(k_in) || !aligned16(q_out) || !aligned16(k_out) || !aligned16(pooled_sums) ||
      !aligned16(rope_cos) || !aligned16(rope_sin))
    return SLA_ERR_BAD_ALIGN;
  if (sums_bytes < pooled_sums_bytes(s)) return SLA_ERR_WS_TOO_SMALL;
  int rc = check_device_arch();
  if (rc != SLA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* sums = static_cast<unsigned char*>(pooled_sums);
#define SLA_QKP(TT, DD) \
  return qk_prepare_typed<TT, DD>(s, static_cast<const TT*>(q_in), static_cast<const TT*>(k_in), gq, gk, rope_cos, \
                                  rope_sin, eps, interleaved, static_cast<TT*>(q_out), static_cast<TT*>(k_out), sums, st)
  if (s->dtype == SLA_BF16) { if (s->D == 64) SLA_QKP(__nv_bfloat16, 64); SLA_QKP(__nv_bfloat16, 128); }
  if (s->D == 64) SLA_QKP(__half, 64);
  SLA_QKP(__half, 128);
#undef SLA_QKP
}

extern "C" int sla_block_map_pooled(const sla_shape* s, const void* pooled_sums, int32_t* lut, int8_t* sparse_map,
                                    int32_t* col_offsets, int32_t* col_index, void* ws, size_t ws_bytes,
                                    sla_stream_t stream) {
  using namespace sla;
  if (!s || !pooled_sums || !lut || !ws) return SLA_ERR_NULL;
  if (s->B < 1 || s->H < 1 || s->L < 1 || (s->D != 64 && s->D != 128)) return SLA_ERR_BAD_SHAPE;
  if (s->BLKQ < 16 || s->BLKK < 16 || s->BLKQ > 1024 || s->BLKK > 1024) return SLA_ERR_BAD_SHAPE;
  if (static_cast<long long>(s->B) * s->H > 65535) return SLA_ERR_BAD_SHAPE;
  if (s->dtype != SLA_BF16 && s->dtype != SLA_FP16) return SLA_ERR_BAD_DTYPE;
  if (s->topk < 1 || s->topk > ceil_div(s->L, s->BLKK)) return SLA_ERR_BAD_TOPK;
  if ((col_offsets == nullptr) != (col_index == nullptr)) return SLA_ERR_NULL;
  if (!aligned16(pooled_sums) || !aligned16(ws)) return SLA_ERR_BAD_ALIGN;
  if (ws_bytes < ws_block_map(s).total) return SLA_ERR_WS_TOO_SMALL;
  int rc = check_device_arch();
  if (rc != SLA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned char* sums = static_cast<const unsigned char*>(pooled_sums);
  unsigned char* w = static_cast<unsigned char*>(ws);
#define SLA_BMP(TT, DD) \
  return block_map_pooled_typed<TT, DD>(s, sums, lut, sparse_map, col_offsets, col_index, w, st)
  if (s->dtype == SLA_BF16) { if (s->D == 64) SLA_BMP(__nv_bfloat16, 64); SLA_BMP(__nv_bfloat16, 128); }
  if (s->D == 64) SLA_BMP(__half, 64);
  SLA_BMP(__half, 128);
#undef SLA_BMP
}

namespace sla {
// ---- 7. packed block lists: block indices fit 16 bits while N_BLOCKS, M_BLOCKS <= 65536 ----
template <typename TSrc, typename TDst>
__global__ void __launch_bounds__(256) index_convert_kernel(const TSrc* __restrict__ src, TDst* __restrict__ dst,
                                                            size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = static_cast<TDst>(src[i]);
}
}  // namespace sla

extern "C" int sla_index_convert(const void* src, int src_bits, void* dst, int dst_bits, size_t count,
                                 sla_stream_t stream) {
  using namespace sla;
  if (!src || !dst) return SLA_ERR_NULL;
  if (count == 0) return SLA_OK;
  int rc = check_device_arch();
  if (rc != SLA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(count / 1024 + 1 < 148u * 8u ? count / 1024 + 1 : 148u * 8u);
  if (src_bits == 32 && dst_bits == 16)
    index_convert_kernel<int32_t, uint16_t><<<grid, 256, 0, st>>>(static_cast<const int32_t*>(src),
                                                                  static_cast<uint16_t*>(dst), count);
  else if (src_bits == 16 && dst_bits == 32)
    index_convert_kernel<uint16_t, int32_t><<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(src),
                                                                  static_cast<int32_t*>(dst), count);
  else
    return SLA_ERR_UNSUPPORTED;
  SLA_LAUNCH_OK();
  return SLA_OK;
}

extern "C" int sla_column_lists(const sla_shape* s, const int8_t* sparse_map, int32_t* col_offsets,
                                int32_t* col_index, sla_stream_t stream) {
  using namespace sla;
  if (!s || !sparse_map || !col_offsets || !col_index) return SLA_ERR_NULL;
  if (s->B < 1 || s->H < 1 || s->L < 1 || s->BLKQ < 1 || s->BLKK < 1) return SLA_ERR_BAD_SHAPE;
  int rc = check_device_arch();
  if (rc != SLA_OK) return rc;
  const int bh = s->B * s->H, mb = ceil_div(s->L, s->BLKQ), nb = ceil_div(s->L, s->BLKK);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  SLA_CUDA_OK(cudaMemsetAsync(col_offsets, 0, sizeof(int32_t) * size_t(bh) * (nb + 1), st));
  col_count_kernel<<<dim3(ceil_div(nb, 32), bh), 1024, 0, st>>>(sparse_map, col_offsets, mb, nb);
  SLA_LAUNCH_OK();
  col_scan_kernel<<<bh, 1024, 0, st>>>(col_offsets, nb);
  SLA_LAUNCH_OK();
  col_fill_kernel<<<dim3(ceil_div(nb, 32), bh), 1024, 0, st>>>(sparse_map, col_offsets, col_index, mb, nb, s->topk);
  SLA_LAUNCH_OK();
  return SLA_OK;
}

extern "C" int sla_block_map(const sla_shape* s, int in_dtype, const void* q, const void* k, int32_t* lut,
                             int8_t* sparse_map, int32_t* col_offsets, int32_t* col_index, void* ws,
                             size_t ws_bytes, sla_stream_t stream) {
  using namespace sla;
  if (s == nullptr || q == nullptr || k == nullptr || lut == nullptr || ws == nullptr) return SLA_ERR_NULL;
  if (s->B < 1 || s->H < 1 || s->L < 1 || (s->D != 64 && s->D != 128)) return SLA_ERR_BAD_SHAPE;
  if (s->BLKQ < 16 || s->BLKK < 16 || s->BLKQ > 1024 || s->BLKK > 1024) return SLA_ERR_BAD_SHAPE;
  if (static_cast<long long>(s->B) * s->H > 65535) return SLA_ERR_BAD_SHAPE;
  int nb = ceil_div(s->L, s->BLKK);
  if (s->topk < 1 || s->topk > nb) return SLA_ERR_BAD_TOPK;
  if (!aligned16(q) || !aligned16(k) || !aligned16(ws)) return SLA_ERR_BAD_ALIGN;
  if ((col_offsets == nullptr) != (col_index == nullptr)) return SLA_ERR_NULL;
  if (ws_bytes < ws_block_map(s).total) return SLA_ERR_WS_TOO_SMALL;
  int rc = check_device_arch();
  if (rc != SLA_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* w = static_cast<unsigned char*>(ws);
#define SLA_BM(TIn, DD) \
  return launch_block_map<TIn, DD>(s, static_cast<const TIn*>(q), static_cast<const TIn*>(k), lut, sparse_map, \
                                   col_offsets, col_index, w, st)
  switch (in_dtype) {
    case SLA_BF16: if (s->D == 64) SLA_BM(__nv_bfloat16, 64); else SLA_BM(__nv_bfloat16, 128);
    case SLA_FP16: if (s->D == 64) SLA_BM(__half, 64); else SLA_BM(__half, 128);
    case SLA_FP32: if (s->D == 64) SLA_BM(float, 64); else SLA_BM(float, 128);
    default: return SLA_ERR_BAD_DTYPE;
  }
#undef SLA_BM
}
