// Linear-branch state: H = phi(k)^T v (D x D) and z = sum_L phi(k) per (batch, head), following
// sparse_linear_attention/core.py:91,93-94. phi(k) is rounded to the 16-bit compute type before it is
// used (core.py:91); the sums accumulate in fp32 and are rounded once at the end (what a 16-bit
// matmul / torch.sum returns). One streaming pass over K and V: HBM-bound, 2*L*D*2 bytes per head.
//
// Stage 1: a CTA reduces a chunk of rows into an fp32 partial (scratch memory, one slot per chunk).
// Stage 2: partials are summed in a fixed order -> deterministic results.
#include "common.cuh"
#include "kernels.h"

namespace sla {

template <typename T, int FEAT, int EPL>
__device__ inline void phi_row(float (&x)[EPL]) {
  if (FEAT == SLA_PHI_SOFTMAX) {
    float mx = x[0];
#pragma unroll
    for (int i = 1; i < EPL; ++i) mx = fmaxf(mx, x[i]);
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      x[i] = __expf(x[i] - mx);
      s += x[i];
    }
    s = 1.f / warp_sum(s);
#pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] *= s;
  } else if (FEAT == SLA_PHI_RELU) {
#pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] = fmaxf(x[i], 0.f);
  } else {
#pragma unroll
    for (int i = 0; i < EPL; ++i) x[i] = x[i] > 0.f ? x[i] + 1.f : __expf(x[i]);
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) x[i] = round_to<T>(x[i]);
}

// Reduces rows [chunk*rows, (chunk+1)*rows) of one head into partial[(bh*nch + chunk)*(D*D+D)].
template <typename T, int D, int FEAT>
__device__ inline void linear_state_chunk(const T* __restrict__ k, const T* __restrict__ v,
                                          float* __restrict__ partial, int L, int nch, int rows,
                                          unsigned char* smem) {
  constexpr int NW = D / 16, NT = NW * 32;
  constexpr int EPL = D / 32;  // elements of a row per lane
  unsigned char* sPhi = smem;            // [64][D] T
  unsigned char* sV = smem + 64 * D * 2; // [64][D] T
  float* red = reinterpret_cast<float*>(smem);  // reused at the end: [NW][D]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ch = blockIdx.x, bh = blockIdx.y;
  const T* kg = k + static_cast<size_t>(bh) * L * D;
  const T* vg = v + static_cast<size_t>(bh) * L * D;
  const uint32_t sPhi_a = smem_u32(sPhi), sV_a = smem_u32(sV);

  float acc[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float zacc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) zacc[i] = 0.f;

  const int row_begin = ch * rows, row_end = min(L, row_begin + rows);
  for (int row0 = row_begin; row0 < row_end; row0 += 64) {
    load_tile_async<D, 64>(sV_a, vg, row0, L, tid, NT);
    cp_async_commit();
    // phi(k) for 64 rows, one warp per row
    for (int r = warp; r < 64; r += NW) {
      int gr = row0 + r;
      float x[EPL];
      if (gr < L) {
        const T* src = kg + static_cast<size_t>(gr) * D + lane * EPL;
        if (EPL == 4) {
          uint2 raw = *reinterpret_cast<const uint2*>(src);
          float2 a = Elem<T>::unpack2(raw.x), b = Elem<T>::unpack2(raw.y);
          x[0] = a.x; x[1] = a.y; x[EPL - 2] = b.x; x[EPL - 1] = b.y;
        } else {
          uint32_t raw = *reinterpret_cast<const uint32_t*>(src);
          float2 a = Elem<T>::unpack2(raw);
          x[0] = a.x; x[1] = a.y;
        }
        phi_row<T, FEAT, EPL>(x);
      } else {
#pragma unroll
        for (int i = 0; i < EPL; ++i) x[i] = 0.f;  // rows past the end contribute nothing
      }
#pragma unroll
      for (int i = 0; i < EPL; ++i) zacc[i] += x[i];
      int col = lane * EPL;
      unsigned char* dst = sPhi + tile_off<D>(r, col >> 3) + (col & 7) * 2;
      if (EPL == 4) {
        uint2 pk;
        pk.x = Elem<T>::pack2(x[0], x[1]);
        pk.y = Elem<T>::pack2(x[EPL - 2], x[EPL - 1]);
        *reinterpret_cast<uint2*>(dst) = pk;
      } else {
        *reinterpret_cast<uint32_t*>(dst) = Elem<T>::pack2(x[0], x[1]);
      }
    }
    cp_async_wait<0>();
    __syncthreads();
    uint32_t a[4][4];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) load_a_frag_trans<D>(a[kk], sPhi_a, kk * 16, warp * 16, lane);
    gemm_b_kn<T, D, D / 8, 4>(acc, a, sV_a, 0, 0, lane);
    __syncthreads();
  }

  float* out = partial + (static_cast<size_t>(bh) * nch + ch) * (D * D + D);
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    int r0 = warp * 16 + g, c = 8 * j + 2 * t;
    *reinterpret_cast<float2*>(out + r0 * D + c) = make_float2(acc[j][0], acc[j][1]);
    *reinterpret_cast<float2*>(out + (r0 + 8) * D + c) = make_float2(acc[j][2], acc[j][3]);
  }
#pragma unroll
  for (int i = 0; i < EPL; ++i) red[warp * D + lane * EPL + i] = zacc[i];
  __syncthreads();
  for (int d = tid; d < D; d += NT) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += red[w * D + d];
    out[D * D + d] = s;
  }
}

template <typename T, int D, int FEAT>
__global__ void __launch_bounds__(D / 16 * 32) linear_state_kernel(const T* __restrict__ k,
                                                                   const T* __restrict__ v,
                                                                   float* __restrict__ partial, int L,
                                                                   int nch, int rows) {
  __shared__ __align__(128) unsigned char smem[2 * 64 * D * 2];
  linear_state_chunk<T, D, FEAT>(k, v, partial, L, nch, rows, smem);
}

// n = D*D + D values per head; the head's record is rec_stride elements long (H, z, then room for H W^T)
template <typename T>
__global__ void linear_state_reduce_kernel(const float* __restrict__ partial, T* __restrict__ state, int nch,
                                           int n, int rec_stride) {
  int bh = blockIdx.y;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* p = partial + static_cast<size_t>(bh) * nch * n + i;
  float s = 0.f;
  for (int c = 0; c < nch; ++c) s += p[static_cast<size_t>(c) * n];
  state[static_cast<size_t>(bh) * rec_stride + i] = Elem<T>::from_f(s);
}

template <typename T, int D>
static int launch_state(const sla_shape* s, const T* k, const T* v, T* state, float* partial, int nch,
                        int rows, cudaStream_t st) {
  int bh = s->B * s->H;
  dim3 grid(nch, bh);
  switch (s->feature_map) {
    case SLA_PHI_SOFTMAX:
      linear_state_kernel<T, D, SLA_PHI_SOFTMAX><<<grid, D / 16 * 32, 0, st>>>(k, v, partial, s->L, nch, rows);
      break;
    case SLA_PHI_RELU:
      linear_state_kernel<T, D, SLA_PHI_RELU><<<grid, D / 16 * 32, 0, st>>>(k, v, partial, s->L, nch, rows);
      break;
    default:
      linear_state_kernel<T, D, SLA_PHI_ELU><<<grid, D / 16 * 32, 0, st>>>(k, v, partial, s->L, nch, rows);
      break;
  }
  SLA_LAUNCH_OK();
  int n = D * D + D;
  linear_state_reduce_kernel<T><<<dim3(ceil_div(n, 256), bh), 256, 0, st>>>(partial, state, nch, n, 2 * D * D + D);
  SLA_LAUNCH_OK();
  return SLA_OK;
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
  static float* ptrs[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_last_cuda_error(e); *status = SLA_ERR_CUDA; return nullptr; }
  if (dev < 0 || dev >= 64) { *status = SLA_ERR_UNSUPPORTED; return nullptr; }
  if (ptrs[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_state_scratch);
    if (e != cudaSuccess) { set_last_cuda_error(e); *status = SLA_ERR_CUDA; return nullptr; }
    ptrs[dev] = ptr;
  }
  *status = SLA_OK;
  return ptrs[dev];
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
