// Linear-branch state: H = phi(k)^T v (D x D) and z = sum_L phi(k) per (batch, head), following
// sparse_linear_attention/core.py:91,93-94. phi(k) is rounded to the 16-bit compute type before it is
// used (core.py:91); the sums accumulate in fp32 and are rounded once at the end (what a 16-bit
// matmul / torch.sum returns). One streaming pass over K and V: HBM-bound, 2*L*D*2 bytes per head.
//
// Stage 1: a CTA reduces a chunk of rows into an fp32 partial (scratch memory, one slot per chunk).
// Stage 2: partials are summed in a fixed order -> deterministic results.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace sla {

// phi of 8 consecutive elements of a row; the row is spread over 8 consecutive lanes (CPT such pieces
// per lane), reductions run over those 8 lanes.
template <typename T, int FEAT, int N>
__device__ inline void phi_piece(float (&x)[N]) {
  if (FEAT == SLA_PHI_SOFTMAX) {
    float mx = x[0];
#pragma unroll
    for (int i = 1; i < N; ++i) mx = fmaxf(mx, x[i]);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) {
      x[i] = __expf(x[i] - mx);
      s += x[i];
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    s = 1.f / s;
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] *= s;
  } else if (FEAT == SLA_PHI_RELU) {
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = fmaxf(x[i], 0.f);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = x[i] > 0.f ? x[i] + 1.f : __expf(x[i]);
  }
}

// Reduces rows [chunk*rows, (chunk+1)*rows) of one head into partial[(bh*nch + chunk)*(D*D+D)].
// 64-row {K, V} tiles stream through two buffers (the next tile is copied in while this one is worked
// on); phi(k) is computed in place on the K tile, 8 lanes per row, then H += phi(k)^T V on mma.sync with
// warp w owning rows [16w, 16w+16) of H.
template <typename T, int D, int FEAT>
__device__ inline void linear_state_chunk(const T* __restrict__ k, const T* __restrict__ v,
                                          float* __restrict__ partial, int L, int nch, int rows,
                                          unsigned char* smem) {
  constexpr int NW = D / 16, NT = NW * 32;
  constexpr int T64 = 64 * D * 2;
  constexpr int CPT = D / 64;          // 16-byte pieces of a row per lane
  constexpr int RPP = NT / 8;          // rows per pass of the phi step
  float* red = reinterpret_cast<float*>(smem);  // reused at the end: [RPP][D]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ch = blockIdx.x, bh = blockIdx.y;
  const T* kg = k + static_cast<size_t>(bh) * L * D;
  const T* vg = v + static_cast<size_t>(bh) * L * D;

  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float zacc[CPT][8];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) zacc[c][i] = 0.f;

  const int row_begin = ch * rows, row_end = min(L, row_begin + rows);
  auto prefetch = [&](int row0, int buf) {
    const uint32_t a = smem_u32(smem + 2 * buf * T64);
    load_tile_async<D, 64>(a, kg, row0, L, tid, NT);
    load_tile_async<D, 64>(a + T64, vg, row0, L, tid, NT);
    cp_async_commit();
  };
  if (row_begin < row_end) prefetch(row_begin, 0);
  const int e8 = tid & 7, prow = tid >> 3;
  int buf = 0;
  for (int row0 = row_begin; row0 < row_end; row0 += 64, buf ^= 1) {
    unsigned char* sK = smem + 2 * buf * T64;
    const uint32_t sK_a = smem_u32(sK), sV_a = sK_a + T64;
    cp_async_wait<0>();
    __syncthreads();   // this tile has landed, and every warp is done with the other buffer
    if (row0 + 64 < row_end) prefetch(row0 + 64, buf ^ 1);
    // phi(k) in place; rows past the end of the sequence were zero-filled and must stay zero
#pragma unroll
    for (int r0 = 0; r0 < 64; r0 += RPP) {
      const int r = r0 + prow;
      float x[CPT * 8];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const uint4 raw = *reinterpret_cast<const uint4*>(sK + tile_off<D>(r, e8 + 8 * c));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = Elem<T>::unpack2(w[i]);
          x[c * 8 + 2 * i] = f.x;
          x[c * 8 + 2 * i + 1] = f.y;
        }
      }
      phi_piece<T, FEAT, CPT * 8>(x);
      const bool live = row0 + r < L;
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w[i] = live ? Elem<T>::pack2(x[c * 8 + 2 * i], x[c * 8 + 2 * i + 1]) : 0u;
          const float2 f = Elem<T>::unpack2(w[i]);     // phi(k) is rounded to T before it is used (core.py:91)
          zacc[c][2 * i] += f.x;
          zacc[c][2 * i + 1] += f.y;
        }
        *reinterpret_cast<uint4*>(sK + tile_off<D>(r, e8 + 8 * c)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    __syncthreads();
    uint32_t a[4][4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) load_a_frag_trans<D>(a[kk], sK_a, kk * 16, warp * 16, lane);
    gemm_b_kn<T, D, D / 8, 4>(acc, a, sV_a, 0, 0, lane);
  }
  cp_async_wait<0>();
  __syncthreads();

  float* out = partial + (static_cast<size_t>(bh) * nch + ch) * (D * D + D);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    int r0 = warp * 16 + g, c = 8 * j + 2 * t;
    *reinterpret_cast<float2*>(out + r0 * D + c) = make_float2(acc[j][0], acc[j][1]);
    *reinterpret_cast<float2*>(out + (r0 + 8) * D + c) = make_float2(acc[j][2], acc[j][3]);
  }
  // z: lane e8 of row group prow holds columns [8 (e8 + 8c), +8)
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int i = 0; i < 8; ++i) red[prow * D + (e8 + 8 * c) * 8 + i] = zacc[c][i];
  __syncthreads();
  for (int d = tid; d < D; d += NT) {
    float s = 0.f;
#pragma unroll 8
    for (int w = 0; w < RPP; ++w) s += red[w * D + d];
    out[D * D + d] = s;
  }
}

template <typename T, int D, int FEAT>
__global__ void __launch_bounds__(D / 16 * 32) linear_state_kernel(const T* __restrict__ k,
                                                                   const T* __restrict__ v,
                                                                   float* __restrict__ partial, int L,
                                                                   int nch, int rows) {
  extern __shared__ __align__(128) unsigned char smem[];   // two {K, V} buffers of 64 rows
  pdl_wait();
  linear_state_chunk<T, D, FEAT>(k, v, partial, L, nch, rows, smem);
}

// n = D*D + D values per head; the head's record is rec_stride elements long (H, z, then room for H W^T)
template <typename T>
__global__ void linear_state_reduce_kernel(const float* __restrict__ partial, T* __restrict__ state, int nch,
                                           int n, int rec_stride) {
  pdl_wait();
  int bh = blockIdx.y;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* p = partial + static_cast<size_t>(bh) * nch * n + i;
  float s = 0.f;
#pragma unroll 8
  for (int c = 0; c < nch; ++c) s += p[static_cast<size_t>(c) * n];   // loads batched, sum in order
  state[static_cast<size_t>(bh) * rec_stride + i] = Elem<T>::from_f(s);
}

template <typename T, int D>
static int launch_state(const sla_shape* s, const T* k, const T* v, T* state, float* partial, int nch,
                        int rows, cudaStream_t st) {
  int bh = s->B * s->H;
  dim3 grid(nch, bh);
  const int n = D * D + D;
  auto reduce = [&]() -> int {
    SLA_CUDA_OK(launch_pdl<false>(linear_state_reduce_kernel<T>, dim3(ceil_div(n, 256), bh), dim3(256), 0, st,
                                  static_cast<const float*>(partial), state, nch, n, 2 * D * D + D));
    SLA_LAUNCH_OK();
    return SLA_OK;
  };
  if (!(s->flags & SLA_FLAG_LEGACY_MMA)) {
    // tcgen05 kernel (head dim 128, chunks of whole 128-row tiles); anything else takes the mma.sync kernel below
    const int rc_tc = run_linear_state_partials_tc(s, k, v, partial, nch, rows, st);
    if (rc_tc == SLA_OK) return reduce();
    if (rc_tc != SLA_ERR_UNSUPPORTED) return rc_tc;
  }
  const int smem = 4 * 64 * D * 2;
  auto go = [&](auto kern) -> int {
    SLA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    SLA_CUDA_OK(launch_pdl<false>(kern, grid, dim3(D / 16 * 32), smem, st, k, v, partial, s->L, nch, rows));
    SLA_LAUNCH_OK();
    return SLA_OK;
  };
  int rc;
  switch (s->feature_map) {
    case SLA_PHI_SOFTMAX: rc = go(linear_state_kernel<T, D, SLA_PHI_SOFTMAX>); break;
    case SLA_PHI_RELU: rc = go(linear_state_kernel<T, D, SLA_PHI_RELU>); break;
    default: rc = go(linear_state_kernel<T, D, SLA_PHI_ELU>); break;
  }
  if (rc != SLA_OK) return rc;
  return reduce();
}

int run_linear_state(const sla_shape* s, const void* k, const void* v, void* lin_state, float* partial, int nch,
                     int rows, cudaStream_t st) {
  if (s->dtype == SLA_BF16) {
    using T = __nv_bfloat16;
    if (s->D == 64) return launch_state<T, 64>(s, (const T*)k, (const T*)v, (T*)lin_state, partial, nch, rows, st);
    return launch_state<T, 128>(s, (const T*)k, (const T*)v, (T*)lin_state, partial, nch, rows, st);
  }
  using T = __half;
  if (s->D == 64) return launch_state<T, 64>(s, (const T*)k, (const T*)v, (T*)lin_state, partial, nch, rows, st);
  return launch_state<T, 128>(s, (const T*)k, (const T*)v, (T*)lin_state, partial, nch, rows, st);
}

// ---------------------------------------------------------------------------------------------
// Variant for callers that cannot hand over a workspace
// ---------------------------------------------------------------------------------------------
// Scratch for the per-chunk fp32 partials, reserved inside the library image: every GPU that loads the
// library holds these 16 MiB until the process exits. All calls on a device share it.
constexpr size_t kStaticScratchFloats = size_t(4) << 20;   // 4 Mi floats = 16 MiB
static __device__ __align__(256) float g_state_scratch[kStaticScratchFloats];

// In host code `g_state_scratch` is only a handle, not an address a kernel could use: the device
// address is looked up once per device (with that device current) and cached.
static float* static_scratch_for_current_device(int* status) {
  static std::atomic<float*> ptrs[64];     // several host threads may make the first call on a device
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_last_cuda_error(e); *status = SLA_ERR_CUDA; return nullptr; }
  if (dev < 0 || dev >= 64) { *status = SLA_ERR_UNSUPPORTED; return nullptr; }
  float* ptr = ptrs[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_state_scratch);
    if (e != cudaSuccess) { set_last_cuda_error(e); *status = SLA_ERR_CUDA; return nullptr; }
    ptrs[dev].store(ptr, std::memory_order_release);
  }
  *status = SLA_OK;
  return ptr;
}

int run_linear_state_static(const sla_shape* s, const void* k, const void* v, void* lin_state, cudaStream_t st) {
  const size_t rec = size_t(s->D) * s->D + s->D;
  const size_t bh = size_t(s->B) * s->H;
  // as many row chunks per head as fit in the reserved scratch (at least one, at most one per 512 rows)
  size_t max_chunks = kStaticScratchFloats / (bh * rec);
  if (max_chunks < 1) return SLA_ERR_WS_TOO_SMALL;
  int nch = (s->L + 511) / 512;
  if (static_cast<size_t>(nch) > max_chunks) nch = static_cast<int>(max_chunks);
  int rows = ((s->L + nch - 1) / nch + 63) / 64 * 64;
  nch = (s->L + rows - 1) / rows;
  int status = SLA_OK;
  float* scratch = static_scratch_for_current_device(&status);
  if (scratch == nullptr) return status;
  return run_linear_state(s, k, v, lin_state, scratch, nch, rows, st);
}

}  // namespace sla
