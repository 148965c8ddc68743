// Shared device/host helpers for the sla_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sla_b200.h"

namespace sla {

constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
void set_last_cuda_error(cudaError_t e);
int check_device_arch();  // SLA_OK or SLA_ERR_WRONG_ARCH / SLA_ERR_CUDA

#define SLA_CUDA_OK(expr)                     \
  do {                                        \
    cudaError_t _e = (expr);                  \
    if (_e != cudaSuccess) {                  \
      ::sla::set_last_cuda_error(_e);         \
      return SLA_ERR_CUDA;                    \
    }                                         \
  } while (0)

void count_launch();
#define SLA_LAUNCH_OK()                 \
  do {                                  \
    ::sla::count_launch();              \
    SLA_CUDA_OK(cudaGetLastError());    \
  } while (0)

// Programmatic dependent launch: a kernel launched through launch_pdl may be scheduled while its predecessor in
// the stream is still running; it must call pdl_wait() before it touches global memory (the call returns once the
// predecessor has completed and its writes are visible; it is a no-op for a kernel launched the ordinary way).
// pdl_launch_dependents() lets the successor's CTAs take the SMs this kernel's last wave leaves idle. Every kernel
// launched through launch_pdl calls both first thing, so a chain of them keeps stream order for memory while
// the launch latency and the partial last wave of one kernel overlap the start of the next.
// launch_pdl<false> is an ordinary launch through the same interface. The forward path uses it: there the linear-branch
// state runs on a second stream next to the mask prediction, and a kernel that becomes resident early and sits in
// pdl_wait() holds SM slots the other stream's kernels could use; no gain was measured there. The backward is one
// chain of eight kernels on one stream and launches programmatically (about 1 % of the step at L = 32760 with 12
// heads, 5-8 % with one or two heads per GPU).
template <bool Programmatic = true, typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = Programmatic ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#if defined(__CUDACC__)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_entry() { pdl_wait(); pdl_launch_dependents(); }
#endif

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round256(size_t x) { return (x + 255) & ~size_t(255); }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

int validate_shape(const sla_shape* s);  // checks D, BLKQ, BLKK, topk, dtype
inline float softmax_scale(const sla_shape* s) {
  return s->qk_scale != 0.f ? s->qk_scale : 1.0f / sqrtf(static_cast<float>(s->D));
}

// ---------------------------------------------------------------------------------------------
// 16-bit element types
// ---------------------------------------------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
  __device__ static inline float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static inline __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  __device__ static inline uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static inline float2 unpack2(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
  }
  // element-wise product / sum of two packed pairs, each result rounded once to T
  __device__ static inline uint32_t mul2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ static inline uint32_t add2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ static inline uint32_t max2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
};
template <>
struct Elem<__half> {
  __device__ static inline float to_f(__half x) { return __half2float(x); }
  __device__ static inline __half from_f(float x) { return __float2half_rn(x); }
  __device__ static inline uint32_t pack2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static inline float2 unpack2(uint32_t u) {
    __half2 v = *reinterpret_cast<__half2*>(&u);
    return __half22float2(v);
  }
  __device__ static inline uint32_t mul2(uint32_t a, uint32_t b) {
    __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ static inline uint32_t add2(uint32_t a, uint32_t b) {
    __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
  __device__ static inline uint32_t max2(uint32_t a, uint32_t b) {
    __half2 r = __hmax2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
  }
};
template <>
struct Elem<float> {
  __device__ static inline float to_f(float x) { return x; }
  __device__ static inline float from_f(float x) { return x; }
};

// round an fp32 value to T and back (the reference's "tensor of dtype T between two ops")
template <typename T>
__device__ inline float round_to(float x) {
  return Elem<T>::to_f(Elem<T>::from_f(x));
}

// ---------------------------------------------------------------------------------------------
// warp-level MMA m16n8k16 (the legacy tensor path; the tcgen05 kernels live in their own files)
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ inline void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ inline void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ inline void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ inline void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ inline void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}

__device__ inline uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared; `valid == false` writes zeros instead of reading.
__device__ inline void cp_async16(uint32_t saddr, const void* gptr, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(saddr), "l"(gptr), "r"(sz));
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ inline void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ---------------------------------------------------------------------------------------------
// Shared-memory tiles of 16-bit elements: ROWS x COLS, COLS in {64,128}, row pitch COLS*2 bytes,
// 16-byte chunks XOR-swizzled with (row & 7) so that ldmatrix and row-wise stores are
// bank-conflict free.
// ---------------------------------------------------------------------------------------------
template <int COLS>
__device__ inline uint32_t tile_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (COLS * 2) + (((chunk) ^ (row & 7)) << 4));
}

// Copy `rows` x COLS elements starting at global row `row0` of a (L x COLS) matrix into a tile.
// Rows >= L are zero-filled. All `nthreads` threads of the CTA take part.
template <int COLS, int ROWS>
__device__ inline void load_tile_async(uint32_t stile, const void* gbase, int row0, int L, int tid,
                                       int nthreads) {
  constexpr int CH = COLS / 8;
  const char* g = reinterpret_cast<const char*>(gbase);
  for (int i = tid; i < ROWS * CH; i += nthreads) {
    int r = i / CH, c = i % CH;
    int gr = row0 + r;
    bool ok = gr < L;
    const char* src = g + (static_cast<size_t>(ok ? gr : 0) * COLS + c * 8) * 2;
    cp_async16(stile + tile_off<COLS>(r, c), src, ok);
  }
}

// A fragments (16 x 16*KS) of rows [m0, m0+16) from a tile stored [m][k].
template <int COLS, int KS>
__device__ inline void load_a_frags(uint32_t (&a)[KS][4], uint32_t stile, int m0, int k0, int lane) {
  int row = m0 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    int chunk = (k0 >> 3) + kk * 2 + (lane >> 4);
    ldmatrix_x4(a[kk], stile + tile_off<COLS>(row, chunk));
  }
}
// One A fragment (16x16) of A = X^T where X is stored [k][m]: rows k0.., columns m0..m0+15.
template <int COLS>
__device__ inline void load_a_frag_trans(uint32_t (&a)[4], uint32_t stile, int k0, int m0, int lane) {
  int row = k0 + (lane & 7) + (lane >> 4) * 8;
  int chunk = (m0 >> 3) + ((lane >> 3) & 1);
  ldmatrix_x4_trans(a, stile + tile_off<COLS>(row, chunk));
}

// acc(16 x 8*NT) += A(16 x 16*KS) * B, B read from a tile stored [n][k] (n = output column).
template <typename T, int COLS, int NT, int KS>
__device__ inline void gemm_b_nk(float (&acc)[NT][4], const uint32_t (&a)[KS][4], uint32_t stile,
                                 int n0, int k0, int lane) {
  int rsel = (lane & 7) + (lane >> 4) * 8;
  int csel = (lane >> 3) & 1;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4(b, stile + tile_off<COLS>(n0 + np * 16 + rsel, (k0 >> 3) + kk * 2 + csel));
      mma16816<T>(acc[2 * np], a[kk], b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], a[kk], b[2], b[3]);
    }
  }
}
// acc(16 x 8*NT) += A(16 x 16*KS) * B, B read from a tile stored [k][n].
template <typename T, int COLS, int NT, int KS>
__device__ inline void gemm_b_kn(float (&acc)[NT][4], const uint32_t (&a)[KS][4], uint32_t stile,
                                 int k0, int n0, int lane) {
  int rsel = (lane & 7) + ((lane >> 3) & 1) * 8;
  int csel = lane >> 4;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, stile + tile_off<COLS>(k0 + kk * 16 + rsel, (n0 >> 3) + np * 2 + csel));
      mma16816<T>(acc[2 * np], a[kk], b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], a[kk], b[2], b[3]);
    }
  }
}

// Turn an accumulator block (16 x 16*KS fp32, MMA C layout) into A fragments of type T.
template <typename T, int KS>
__device__ inline void acc_to_a_frags(uint32_t (&a)[KS][4], const float (&acc)[2 * KS][4]) {
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    a[kk][0] = Elem<T>::pack2(acc[2 * kk][0], acc[2 * kk][1]);
    a[kk][1] = Elem<T>::pack2(acc[2 * kk][2], acc[2 * kk][3]);
    a[kk][2] = Elem<T>::pack2(acc[2 * kk + 1][0], acc[2 * kk + 1][1]);
    a[kk][3] = Elem<T>::pack2(acc[2 * kk + 1][2], acc[2 * kk + 1][3]);
  }
}

// Store a 16-row accumulator block (MMA C layout, fp32) as T into a tile [m][n] at rows m0...
template <typename T, int COLS, int NT>
__device__ inline void store_acc_to_tile(unsigned char* tile, const float (&acc)[NT][4], int m0,
                                         int lane) {
  int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    int r0 = m0 + g, r1 = m0 + g + 8;
    *reinterpret_cast<uint32_t*>(tile + tile_off<COLS>(r0, j) + t * 4) =
        Elem<T>::pack2(acc[j][0], acc[j][1]);
    *reinterpret_cast<uint32_t*>(tile + tile_off<COLS>(r1, j) + t * 4) =
        Elem<T>::pack2(acc[j][2], acc[j][3]);
  }
}
// Store A-fragment registers (16 x 16*KS of T) into a tile [m][k] at rows m0.., columns k0...
template <int COLS, int KS>
__device__ inline void store_a_frags_to_tile(unsigned char* tile, const uint32_t (&a)[KS][4], int m0,
                                             int k0, int lane) {
  int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    int c = (k0 >> 3) + 2 * kk;
    *reinterpret_cast<uint32_t*>(tile + tile_off<COLS>(m0 + g, c) + t * 4) = a[kk][0];
    *reinterpret_cast<uint32_t*>(tile + tile_off<COLS>(m0 + g + 8, c) + t * 4) = a[kk][1];
    *reinterpret_cast<uint32_t*>(tile + tile_off<COLS>(m0 + g, c + 1) + t * 4) = a[kk][2];
    *reinterpret_cast<uint32_t*>(tile + tile_off<COLS>(m0 + g + 8, c + 1) + t * 4) = a[kk][3];
  }
}

// Write rows [0, rows) of a tile [m][COLS] to global rows row0.. (< L), 16 bytes per thread-step.
template <int COLS, int ROWS>
__device__ inline void store_tile_to_global(void* gbase, const unsigned char* tile, int row0, int L,
                                            int tid, int nthreads) {
  constexpr int CH = COLS / 8;
  char* g = reinterpret_cast<char*>(gbase);
  for (int i = tid; i < ROWS * CH; i += nthreads) {
    int r = i / CH, c = i % CH;
    int gr = row0 + r;
    if (gr < L) {
      uint4 v = *reinterpret_cast<const uint4*>(tile + tile_off<COLS>(r, c));
      *reinterpret_cast<uint4*>(g + (static_cast<size_t>(gr) * COLS + c * 8) * 2) = v;
    }
  }
}

__device__ inline float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  return v;
}
__device__ inline float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}
__device__ inline float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---------------------------------------------------------------------------------------------
// Feature maps phi (sparse_linear_attention/core.py:43-57) on A-fragment registers: a thread holds,
// for rows g and g+8 of a 16-row slab, the columns {16kk + 2t, +1, 16kk + 8 + 2t, +1}.
// in: x fragments (T). out: phi(x) fragments rounded to T (core.py:90-91).
// ---------------------------------------------------------------------------------------------
template <typename T, int KS, int FEAT>
__device__ inline void feature_map_frags(uint32_t (&out)[KS][4], const uint32_t (&x)[KS][4]) {
  if (FEAT == SLA_PHI_SOFTMAX) {
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      float2 a = Elem<T>::unpack2(x[kk][0]), b = Elem<T>::unpack2(x[kk][1]);
      float2 c = Elem<T>::unpack2(x[kk][2]), d = Elem<T>::unpack2(x[kk][3]);
      mx0 = fmaxf(mx0, fmaxf(fmaxf(a.x, a.y), fmaxf(c.x, c.y)));
      mx1 = fmaxf(mx1, fmaxf(fmaxf(b.x, b.y), fmaxf(d.x, d.y)));
    }
    mx0 = quad_max(mx0);
    mx1 = quad_max(mx1);
    float s0 = 0.f, s1 = 0.f;
    float e[KS][8];
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      float2 a = Elem<T>::unpack2(x[kk][0]), b = Elem<T>::unpack2(x[kk][1]);
      float2 c = Elem<T>::unpack2(x[kk][2]), d = Elem<T>::unpack2(x[kk][3]);
      e[kk][0] = __expf(a.x - mx0); e[kk][1] = __expf(a.y - mx0);
      e[kk][2] = __expf(b.x - mx1); e[kk][3] = __expf(b.y - mx1);
      e[kk][4] = __expf(c.x - mx0); e[kk][5] = __expf(c.y - mx0);
      e[kk][6] = __expf(d.x - mx1); e[kk][7] = __expf(d.y - mx1);
      s0 += e[kk][0] + e[kk][1] + e[kk][4] + e[kk][5];
      s1 += e[kk][2] + e[kk][3] + e[kk][6] + e[kk][7];
    }
    s0 = 1.f / quad_sum(s0);
    s1 = 1.f / quad_sum(s1);
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      out[kk][0] = Elem<T>::pack2(e[kk][0] * s0, e[kk][1] * s0);
      out[kk][1] = Elem<T>::pack2(e[kk][2] * s1, e[kk][3] * s1);
      out[kk][2] = Elem<T>::pack2(e[kk][4] * s0, e[kk][5] * s0);
      out[kk][3] = Elem<T>::pack2(e[kk][6] * s1, e[kk][7] * s1);
    }
  } else {
#pragma unroll
    for (int kk = 0; kk < KS; ++kk)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float2 a = Elem<T>::unpack2(x[kk][r]);
        if (FEAT == SLA_PHI_RELU) {
          a.x = fmaxf(a.x, 0.f);
          a.y = fmaxf(a.y, 0.f);
        } else {  // elu(x) + 1
          a.x = a.x > 0.f ? a.x + 1.f : __expf(a.x);
          a.y = a.y > 0.f ? a.y + 1.f : __expf(a.y);
        }
        out[kk][r] = Elem<T>::pack2(a.x, a.y);
      }
  }
}

// Backward of phi on fragments: given phi(x) (T fragments) and dphi (fp32, MMA C layout:
// acc[2kk][0..1] <-> frag[kk][0], acc[2kk][2..3] <-> frag[kk][1], acc[2kk+1][0..1] <-> frag[kk][2],
// acc[2kk+1][2..3] <-> frag[kk][3]) overwrite dphi with dx. Only phi is needed: for relu x > 0 iff
// phi > 0, and for elu+1 x > 0 iff phi > 1 (derivative 1), otherwise the derivative exp(x) = phi.
template <typename T, int KS, int FEAT>
__device__ inline void feature_map_bwd_frags(float (&dphi)[2 * KS][4], const uint32_t (&phi)[KS][4]) {
  if (FEAT == SLA_PHI_SOFTMAX) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      float2 p0 = Elem<T>::unpack2(phi[kk][0]), p1 = Elem<T>::unpack2(phi[kk][1]);
      float2 p2 = Elem<T>::unpack2(phi[kk][2]), p3 = Elem<T>::unpack2(phi[kk][3]);
      s0 += dphi[2 * kk][0] * p0.x + dphi[2 * kk][1] * p0.y + dphi[2 * kk + 1][0] * p2.x +
            dphi[2 * kk + 1][1] * p2.y;
      s1 += dphi[2 * kk][2] * p1.x + dphi[2 * kk][3] * p1.y + dphi[2 * kk + 1][2] * p3.x +
            dphi[2 * kk + 1][3] * p3.y;
    }
    s0 = quad_sum(s0);
    s1 = quad_sum(s1);
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      float2 p0 = Elem<T>::unpack2(phi[kk][0]), p1 = Elem<T>::unpack2(phi[kk][1]);
      float2 p2 = Elem<T>::unpack2(phi[kk][2]), p3 = Elem<T>::unpack2(phi[kk][3]);
      dphi[2 * kk][0] = p0.x * (dphi[2 * kk][0] - s0);
      dphi[2 * kk][1] = p0.y * (dphi[2 * kk][1] - s0);
      dphi[2 * kk][2] = p1.x * (dphi[2 * kk][2] - s1);
      dphi[2 * kk][3] = p1.y * (dphi[2 * kk][3] - s1);
      dphi[2 * kk + 1][0] = p2.x * (dphi[2 * kk + 1][0] - s0);
      dphi[2 * kk + 1][1] = p2.y * (dphi[2 * kk + 1][1] - s0);
      dphi[2 * kk + 1][2] = p3.x * (dphi[2 * kk + 1][2] - s1);
      dphi[2 * kk + 1][3] = p3.y * (dphi[2 * kk + 1][3] - s1);
    }
  } else {
#pragma unroll
    for (int kk = 0; kk < KS; ++kk)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float2 pv = Elem<T>::unpack2(phi[kk][r]);
        int j = 2 * kk + (r >> 1);
        int c = (r & 1) * 2;
        if (FEAT == SLA_PHI_RELU) {
          dphi[j][c] = pv.x > 0.f ? dphi[j][c] : 0.f;
          dphi[j][c + 1] = pv.y > 0.f ? dphi[j][c + 1] : 0.f;
        } else {
          dphi[j][c] = pv.x > 1.f ? dphi[j][c] : dphi[j][c] * pv.x;
          dphi[j][c + 1] = pv.y > 1.f ? dphi[j][c + 1] : dphi[j][c + 1] * pv.y;
        }
      }
  }
}

// acc(16 x 8*NT) += A * B with A (rows m0.. of a tile [m][k]) fetched per k-step and B read from a
// tile stored [k][n].
template <typename T, int COLS, int NT, int KS>
__device__ inline void gemm_at_b_kn(float (&acc)[NT][4], uint32_t sA, int m0, uint32_t sB, int lane) {
  int arow = m0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int rsel = (lane & 7) + ((lane >> 3) & 1) * 8;
  int csel = lane >> 4;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, sA + tile_off<COLS>(arow, kk * 2 + (lane >> 4)));
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, sB + tile_off<COLS>(kk * 16 + rsel, np * 2 + csel));
      mma16816<T>(acc[2 * np], a, b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// acc(16 x 8*NT) += X^T * B for rows m0..m0+15 of X^T, X stored [k][m], B stored [k][n]; K = 16*KS.
template <typename T, int COLS, int NT, int KS>
__device__ inline void gemm_atrans_b_kn(float (&acc)[NT][4], uint32_t sX, int m0, uint32_t sB, int lane) {
  int rsel = (lane & 7) + ((lane >> 3) & 1) * 8;
  int csel = lane >> 4;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    uint32_t a[4];
    load_a_frag_trans<COLS>(a, sX, kk * 16, m0, lane);
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, sB + tile_off<COLS>(kk * 16 + rsel, np * 2 + csel));
      mma16816<T>(acc[2 * np], a, b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// acc(16 x 8*NT) += A * B with A (rows m0..m0+15 of a tile [m][k]) fetched per k-step and B read
// from a tile stored [n][k].
template <typename T, int COLS, int NT, int KS>
__device__ inline void gemm_at_b_nk(float (&acc)[NT][4], uint32_t sA, int m0, uint32_t sB, int lane) {
  int arow = m0 + (lane & 7) + ((lane >> 3) & 1) * 8;
  int rsel = (lane & 7) + (lane >> 4) * 8;
  int csel = (lane >> 3) & 1;
#pragma unroll
  for (int kk = 0; kk < KS; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, sA + tile_off<COLS>(arow, kk * 2 + (lane >> 4)));
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldmatrix_x4(b, sB + tile_off<COLS>(np * 16 + rsel, kk * 2 + csel));
      mma16816<T>(acc[2 * np], a, b[0], b[1]);
      mma16816<T>(acc[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// Write 16 staged rows (tile rows m0.., T) to global rows grow0.., optionally adding what is there.
template <typename T, int D>
__device__ inline void flush16(const unsigned char* tile, int m0, T* gbase, int grow0, int L, int lane,
                               bool accumulate) {
  constexpr int CH = D / 8;
  __syncwarp();
  for (int i = lane; i < 16 * CH; i += 32) {
    int r = i / CH, c = i % CH;
    int gr = grow0 + r;
    if (gr < L) {
      uint4 v4 = *reinterpret_cast<const uint4*>(tile + tile_off<D>(m0 + r, c));
      uint4* dst = reinterpret_cast<uint4*>(gbase + static_cast<size_t>(gr) * D + c * 8);
      if (accumulate) {
        uint4 old = *dst;
        uint32_t* a = reinterpret_cast<uint32_t*>(&v4);
        uint32_t* b = reinterpret_cast<uint32_t*>(&old);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 x = Elem<T>::unpack2(a[e]), y = Elem<T>::unpack2(b[e]);
          a[e] = Elem<T>::pack2(x.x + y.x, x.y + y.y);
        }
      }
      *dst = v4;
    }
  }
  __syncwarp();
}

}  // namespace sla
