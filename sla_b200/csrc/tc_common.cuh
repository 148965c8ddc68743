// PTX wrappers for the Blackwell (sm_100a) async machinery used by the tcgen05 kernels:
// mbarriers with bounded waits, TMA tiled copies, tensor memory allocation / load / store, and
// tcgen05.mma with shared-memory and tensor-memory operands.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sla {
namespace tc {

// Every kernel gets a pointer to a device-wide control block (TcControl): word 0 is the error word, 0 = fine,
// otherwise the code of the first bounded wait that ran out. Once it is non-zero every CTA of the tcgen05
// kernels leaves as soon as it notices. Word 1 is a test hook (see sparse_fwd_tc.cu), the 64-bit word behind
// them the limit of every wait in nanoseconds.
struct TcControl {
  int error;
  int drop_first_k_tile;             // test hook: CTA (0,0) of the forward never requests its first K tile
  unsigned long long wait_limit_ns;
};
constexpr unsigned long long kDefaultWaitLimitNs = 2000000000ull;   // 2 s: far above any legitimate wait (microseconds)

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Non-blocking probe of a phase (cheap when the phase has already completed).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait. Returns false (after recording `code`) if the phase did not complete within the control block's
// wait limit of wall-clock time or another CTA has already reported a failure. The bound is on elapsed time, not on the
// number of polls: a try_wait on a pending phase may itself suspend the thread for a while.
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code, int* err) {
  if (mbar_test(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 15u) == 15u) {       // the control block is only looked at while the wait is already long
      if (*reinterpret_cast<volatile int*>(err) != 0) return false;
      if (global_timer_ns() - t0 > reinterpret_cast<volatile TcControl*>(err)->wait_limit_ns) break;
    }
  }
  atomicCAS(err, 0, code);
  return false;
}

// Wait of the abort path: a copy this CTA requested earlier must land before its shared memory goes away. The
// error word is already set at that point, so it is not consulted; the time limit still holds.
__device__ __forceinline__ void mbar_wait_drain(uint32_t bar, uint32_t parity, int* err) {
  if (mbar_test(bar, parity)) return;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t it = 0;; ++it) {
    if (mbar_try(bar, parity)) return;
    if ((it & 15u) == 15u &&
        global_timer_ns() - t0 > reinterpret_cast<volatile TcControl*>(err)->wait_limit_ns) return;
  }
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 3-D tiled load global -> shared (no multicast), completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// 3-D tiled store shared -> global (rows outside the tensor are clipped).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];\n"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// Same, but the tile is ADDED to what global memory holds (element type of the tensor map).
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];\n"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }
// Enough before the CTA's shared memory goes away: the copy engine has READ the staged tiles (the writes to global
// memory complete in the background; kernel completion makes them visible).
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }

// One arrival per warp instead of 32: every lane's earlier writes (shared memory, or tensor memory behind a
// tcgen05.wait + fence::before_thread_sync) are ordered before the warp barrier, and the arrival of lane 0
// releases them. The barrier is initialised with the number of WARPS.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// ---- union of two ascending index lists, by one warp ----
// out = ascending union of a[0, na) and b[0, nb) (each strictly ascending); an element carries flag_a, flag_b or both.
// Every lane of the warp calls this; ranks come from binary searches in the other list, so the cost is
// O(log n) shared-memory round trips per 32 elements instead of one per element for a serial merge.
__device__ __forceinline__ int lower_bound_i32(const int32_t* x, int n, int v) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (x[mid] < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}
__device__ inline bool warp_is_ascending(const int32_t* x, int n, int lane) {
  bool ok = true;
  for (int i = lane; i + 1 < n; i += 32) ok = ok && x[i] < x[i + 1];
  return __all_sync(0xffffffffu, ok);
}
__device__ inline int warp_union_lists(const int32_t* a, int na, const int32_t* b, int nb, int32_t* out,
                                       int32_t flag_a, int32_t flag_b, int lane) {
  if (!warp_is_ascending(a, na, lane) || !warp_is_ascending(b, nb, lane)) {
    // Lists in arbitrary order (torch.topk(sorted=False) gives no order, utils.py:64): a two-pointer walk by
    // one lane still emits every element of both lists, possibly once per list; the flags keep that correct.
    int n = 0;
    if (lane == 0) {
      int i = 0, j = 0;
      while (i < na || j < nb) {
        const int va = i < na ? a[i] : 0x7fffffff, vb = j < nb ? b[j] : 0x7fffffff;
        if (va == vb) { out[n++] = va | flag_a | flag_b; ++i; ++j; }
        else if (va < vb) { out[n++] = va | flag_a; ++i; }
        else { out[n++] = vb | flag_b; ++j; }
      }
    }
    n = __shfl_sync(0xffffffffu, n, 0);
    __syncwarp();
    return n;
  }
  const uint32_t lt = (1u << lane) - 1u;
  if (na <= 32 && nb <= 32) {
    // short lists (the usual top-k): one element of each list per lane, all-pairs comparison through shuffles
    const int va = lane < na ? a[lane] : 0x7fffffff, vb = lane < nb ? b[lane] : 0x7fffffff;
    int less_b = 0, less_a = 0;
    bool dup_a = false, dup_b = false;
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
      const int bj = __shfl_sync(0xffffffffu, vb, j), aj = __shfl_sync(0xffffffffu, va, j);
      less_b += (j < nb && bj < va);
      dup_a = dup_a || (j < nb && bj == va);
      less_a += (j < na && aj < vb);
      dup_b = dup_b || (j < na && aj == vb);
    }
    const uint32_t ma = __ballot_sync(0xffffffffu, lane < na && dup_a);
    const uint32_t mb = __ballot_sync(0xffffffffu, lane < nb && dup_b);
    if (lane < na) out[lane + less_b - __popc(ma & lt)] = va | (dup_a ? (flag_a | flag_b) : flag_a);
    if (lane < nb && !dup_b) out[less_a + lane - __popc(mb & lt)] = vb | flag_b;
    __syncwarp();
    return na + nb - __popc(ma);
  }
  int dups = 0;                                   // elements of a seen so far that are also in b
  for (int base = 0; base < na; base += 32) {
    const int i = base + lane;
    const bool valid = i < na;
    const int va = valid ? a[i] : 0x7fffffff;
    const int lb = valid ? lower_bound_i32(b, nb, va) : 0;
    const bool dup = valid && lb < nb && b[lb] == va;
    const uint32_t m = __ballot_sync(0xffffffffu, dup);
    // rank = elements of a below va + elements of b below va that are not in a
    if (valid) out[i + lb - dups - __popc(m & lt)] = va | (dup ? (flag_a | flag_b) : flag_a);
    dups += __popc(m);
  }
  int dups_b = 0;                                 // elements of b seen so far that are also in a
  for (int base = 0; base < nb; base += 32) {
    const int i = base + lane;
    const bool valid = i < nb;
    const int vb = valid ? b[i] : 0x7fffffff;
    const int la = valid ? lower_bound_i32(a, na, vb) : 0;
    const bool dup = valid && la < na && a[la] == vb;
    const uint32_t m = __ballot_sync(0xffffffffu, dup);
    if (valid && !dup) out[la + i - dups_b - __popc(m & lt)] = vb | flag_b;
    dups_b += __popc(m);
  }
  __syncwarp();
  return na + nb - dups;
}

// ---- tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

#include "tc_ldst.inc"

// True in exactly one lane of a converged warp. The MMA-issuing warp runs its control flow in all 32
// lanes and predicates only the tcgen05 instructions on this: with a divergent `lane == 0` branch
// around the whole loop the compiler keeps descriptors in vector registers and pays a transfer to the
// uniform datapath for every operand of every MMA (measured: 45 vs 32 cycles per N=64 MMA).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ bool warp_all(bool ok) { return __all_sync(0xffffffffu, ok) != 0; }

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}

// ---- descriptors ----
// Shared-memory matrix descriptor, 128-byte swizzle. Bits [0,14) address>>4, [16,30) leading byte
// offset>>4, [32,46) stride byte offset>>4, [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor for kind::f16 (fp32 accumulate). fmt: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t idesc_f16(int fmt, int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
// The issuing thread is a serial resource: descriptors are kept as 32-bit halves so that stepping
// through a tile costs one integer add per operand. hi is the same for every 128B-swizzled tile
// with 1024-byte 8-row groups: SBO = 1024 >> 4, version 1 (bit 46), layout SWIZZLE_128B (bits 61-63).
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}

// 8-bit kinds (K = 32 per instruction): kind::i8 (s8 x s8 -> s32) and kind::f8f6f4 (e4m3 x e4m3 -> f32)
__device__ __forceinline__ void mma_ss_i8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void mma_ts_f8(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %3, p;\n\t}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}
// instruction descriptors: s8 x s8 -> s32, both K-major; e4m3 x e4m3 -> f32 with an MN-major B
__host__ __device__ constexpr uint32_t idesc_i8(int M, int N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_e4m3(int M, int N, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

}  // namespace tc

// host: encode a 3-D tensor map (D, L, BH) of 16-bit elements with a (64, box_rows, 1) box and
// 128-byte swizzle. Returns SLA_OK or SLA_ERR_CUDA.
int make_tmap_3d(CUtensorMap* out, const void* base, int dtype, int D, int L, int BH, int box_rows);
int make_tmap_rows(CUtensorMap* out, const void* base, int dtype, int D, int L, int BH, size_t head_stride_bytes,
                   int box_rows);
// host: same for 8-bit elements, rows of `row_bytes` (<= 128) bytes, box = (row_bytes, box_rows, 1).
int make_tmap_3d_u8(CUtensorMap* out, const void* base, int row_bytes, int L, int BH, int box_rows);
// host: address of the current device's control block, i.e. of its error word (looked up once per device), or
// nullptr.
int* tc_error_word();
// host: set the wait limit / the test hook of the current device's control block (synchronous copies).
int set_tc_wait_limit(unsigned long long ns);
int set_tc_drop_first_k_tile(int on);

}  // namespace sla
