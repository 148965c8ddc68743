// extern "C" entry points of the attention operators: argument checks, workspace carving, launches.
#include <cuda.h>
#include <initializer_list>
#include <string.h>

#include "common.cuh"
#include "kernels.h"
#include "tc_common.cuh"
#include "workspace.h"

using namespace sla;

namespace {

int check_common(const sla_shape* s) {
  int rc = validate_shape(s);
  if (rc != SLA_OK) return rc;
  if (!(softmax_scale(s) > 0.f)) return SLA_ERR_UNSUPPORTED;   // the kernels take row maxima before scaling
  return check_device_arch();
}

bool all_aligned(std::initializer_list<const void*> ps) {
  for (const void* p : ps)
    if (p != nullptr && !aligned16(p)) return false;
  return true;
}

FwdParams make_fwd(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
                   void* o, void* o_s, float* lse, const void* lin_state, const void* wbits) {
  FwdParams p;
  p.q = q; p.k = k; p.v = v; p.lut = lut; p.o = o; p.o_s = o_s; p.lse = lse;
  p.lin_state = lin_state; p.wbits = wbits;
  p.L = s->L; p.mb = ceil_div(s->L, s->BLKQ); p.topk = s->topk;
  p.scale_log2 = softmax_scale(s) * kLog2e;
  return p;
}

// Sparse forward (with the fused linear read-out when `lin`): the tcgen05 kernel, or the mma.sync kernel when the
// caller asks for it or when the entry list of a query tile does not fit the tcgen05 kernel's shared memory.
int run_sparse_fwd(const sla_shape* s, const FwdParams& p, bool lin, cudaStream_t st) {
  if (!(s->flags & SLA_FLAG_LEGACY_MMA)) {
    int rc = run_sparse_fwd_tc(s, p, st);
    if (rc != SLA_ERR_BAD_SHAPE) return rc;
  }
  return run_sparse_fwd_mma(s, p, lin, st);
}

}  // namespace

extern "C" {

int sla_sparse_fwd(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
                   void* o_s, float* lse, sla_stream_t stream) {
  if (!q || !k || !v || !lut || !o_s || !lse) return SLA_ERR_NULL;
  int rc = check_common(s);
  if (rc != SLA_OK) return rc;
  if (!all_aligned({q, k, v, o_s})) return SLA_ERR_BAD_ALIGN;
  FwdParams p = make_fwd(s, q, k, v, lut, o_s, nullptr, lse, nullptr, nullptr);
  return run_sparse_fwd(s, p, false, static_cast<cudaStream_t>(stream));
}

int sla_kernel_path(const sla_shape* s, int op) {
  int rc = validate_shape(s);
  if (rc != SLA_OK) return rc;
  const bool legacy = (s->flags & SLA_FLAG_LEGACY_MMA) != 0;
  switch (op) {
    case SLA_OP_FWD: return (legacy || !sparse_fwd_tc_fits(s)) ? 1 : 0;
    case SLA_OP_BWD:
    case SLA_OP_SPARSE_BWD: return (legacy || !sparse_bwd_tc_fits(s)) ? 1 : 0;
    case SLA_OP_SAGE_FWD: return 0;
    default: return SLA_ERR_UNSUPPORTED;
  }
}

int sla_debug_set_trace(void* device_buffer) {
  set_trace_buffer(static_cast<long long*>(device_buffer));
  return SLA_OK;
}

int sla_poll_device_error(int* code, int clear) {
  if (!code) return SLA_ERR_NULL;
  int rc = read_tc_error(code, clear != 0);
  if (rc != SLA_OK) return rc;
  return *code != 0 ? SLA_ERR_TIMEOUT : SLA_OK;
}

int sla_debug_set_wait_limit_ns(unsigned long long ns) {
  int rc = check_device_arch();
  if (rc != SLA_OK) return rc;
  return set_tc_wait_limit(ns == 0 ? tc::kDefaultWaitLimitNs : ns);
}

int sla_debug_drop_first_k_tile(int on) {
  int rc = check_device_arch();
  if (rc != SLA_OK) return rc;
  return set_tc_drop_first_k_tile(on != 0 ? 1 : 0);
}

int sla_linear_state(const sla_shape* s, const void* k, const void* v, void* lin_state, void* ws,
                     size_t ws_bytes, sla_stream_t stream) {
  if (!k || !v || !lin_state || !ws) return SLA_ERR_NULL;
  int rc = check_common(s);
  if (rc != SLA_OK) return rc;
  if (!all_aligned({k, v, lin_state, ws})) return SLA_ERR_BAD_ALIGN;
  WsLinearState w = ws_linear_state(s);
  if (ws_bytes < w.total) return SLA_ERR_WS_TOO_SMALL;
  return run_linear_state(s, k, v, lin_state, reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + w.partial),
                          w.nch, w.rows, static_cast<cudaStream_t>(stream));
}

int sla_linear_state_static(const sla_shape* s, const void* k, const void* v, void* lin_state,
                            sla_stream_t stream) {
  if (!k || !v || !lin_state) return SLA_ERR_NULL;
  int rc = check_common(s);
  if (rc != SLA_OK) return rc;
  if (!all_aligned({k, v, lin_state})) return SLA_ERR_BAD_ALIGN;
  return run_linear_state_static(s, k, v, lin_state, static_cast<cudaStream_t>(stream));
}

int sla_fwd_prepare(const sla_shape* s, const void* k, const void* v, const float* w, const float* bias,
                    void* lin_state, void* ws, size_t ws_bytes, sla_stream_t stream) {
  if (!k || !v || !w || !lin_state || !ws) return SLA_ERR_NULL;
  int rc = check_common(s);
  if (rc != SLA_OK) return rc;
  if (!all_aligned({k, v, lin_state, ws})) return SLA_ERR_BAD_ALIGN;
  if (s->flags & SLA_FLAG_SPARSE_ONLY) return SLA_ERR_UNSUPPORTED;
  WsLinearState wl = ws_linear_state(s);
  if (ws_bytes < ws_fwd_total(s)) return SLA_ERR_WS_TOO_SMALL;
  unsigned char* base = static_cast<unsigned char*>(ws);
  void* wbits = base + wl.total;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = convert_proj(s, w, bias, wbits, st);
  if (rc != SLA_OK) return rc;
  rc = run_linear_state(s, k, v, lin_state, reinterpret_cast<float*>(base + wl.partial), wl.nch, wl.rows, st);
  if (rc != SLA_OK) return rc;
  return run_state_proj(s, lin_state, wbits, st);
}

static int fwd_impl(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
                    const float* w, const float* bias, void* o, void* o_s, float* lse, void* lin_state, void* ws,
                    size_t ws_bytes, void* const* gather_dst, int n_gather, sla_stream_t stream) {
  if (!q || !k || !v || !lut || !o || !lse) return SLA_ERR_NULL;
  int rc = check_common(s);
  if (rc != SLA_OK) return rc;
  if (n_gather < 0 || n_gather > 8 || (n_gather > 0 && gather_dst == nullptr)) return SLA_ERR_UNSUPPORTED;
  for (int g = 0; g < n_gather; ++g) {
    if (gather_dst[g] == nullptr) return SLA_ERR_NULL;
    if (!aligned16(gather_dst[g])) return SLA_ERR_BAD_ALIGN;
  }
  // the copies are written by the tcgen05 kernel's epilogue only
  if (n_gather > 0 && ((s->flags & (SLA_FLAG_LEGACY_MMA | SLA_FLAG_LINEAR_UNSELECTED)) || !sparse_fwd_tc_fits(s)))
    return SLA_ERR_UNSUPPORTED;
  auto with_gather = [&](FwdParams p) {
    p.n_gather = n_gather;
    for (int g = 0; g < n_gather; ++g) p.gather_dst[g] = gather_dst[g];
    return p;
  };
  if (!all_aligned({q, k, v, o, o_s, lin_state, ws})) return SLA_ERR_BAD_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool legacy = (s->flags & SLA_FLAG_LEGACY_MMA) != 0;
  if (s->flags & SLA_FLAG_SPARSE_ONLY) {
    FwdParams p = with_gather(make_fwd(s, q, k, v, lut, o, nullptr, lse, nullptr, nullptr));
    return run_sparse_fwd(s, p, false, st);
  }
  if (!w || !lin_state || !ws) return SLA_ERR_NULL;
  WsLinearState wl = ws_linear_state(s);
  if (ws_bytes < ws_fwd_total(s)) return SLA_ERR_WS_TOO_SMALL;
  unsigned char* base = static_cast<unsigned char*>(ws);
  void* wbits = base + wl.total;
  const bool unselected = (s->flags & SLA_FLAG_LINEAR_UNSELECTED) != 0;
  if (unselected && legacy) return SLA_ERR_UNSUPPORTED;
  if (!(s->flags & SLA_FLAG_STATE_READY)) {
    rc = convert_proj(s, w, bias, wbits, st);
    if (rc != SLA_OK) return rc;
    rc = run_linear_state(s, k, v, lin_state, reinterpret_cast<float*>(base + wl.partial), wl.nch, wl.rows, st);
    if (rc != SLA_OK) return rc;
    rc = run_state_proj(s, lin_state, wbits, st);
    if (rc != SLA_OK) return rc;
  }
  FwdParams p = with_gather(make_fwd(s, q, k, v, lut, o, o_s, lse, lin_state, wbits));
  if (unselected) {
    // sparse branch; then the same block lists once more without softmax on (phi(q), phi(k), v) for the
    // selected blocks' share of the linear state, which the read-out takes off the all-token state
    unsigned char* ub = base + wl.total + ws_fwd_extra(s);
    WsUnselected wu = ws_unselected(s);
    void* os_buf = o_s ? o_s : o;
    FwdParams ps = make_fwd(s, q, k, v, lut, os_buf, nullptr, lse, nullptr, nullptr);
    rc = run_sparse_fwd_tc(s, ps, st);
    if (rc == SLA_ERR_BAD_SHAPE) return SLA_ERR_UNSUPPORTED;   // this scope has no mma.sync path
    if (rc != SLA_OK) return rc;
    rc = run_feature_map(s, q, ub + wu.phiq, st);
    if (rc != SLA_OK) return rc;
    rc = run_feature_map(s, k, ub + wu.phik, st);
    if (rc != SLA_OK) return rc;
    FwdParams pc = make_fwd(s, ub + wu.phiq, ub + wu.phik, v, lut, ub + wu.cnum, nullptr,
                            reinterpret_cast<float*>(ub + wu.cden), nullptr, nullptr);
    pc.plain = 1;
    rc = run_sparse_fwd_tc(s, pc, st);
    if (rc != SLA_OK) return rc;
    FwdParams pr = make_fwd(s, ub + wu.phiq, k, v, lut, o, os_buf, lse, lin_state, wbits);
    return run_linear_readout_unselected(s, pr, ub + wu.cnum, reinterpret_cast<const float*>(ub + wu.cden), st);
  }
  // sparse branch with the linear read-out, proj_l and the final sum fused into its epilogue
  return run_sparse_fwd(s, p, true, st);
}

int sla_fwd(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
            const float* w, const float* bias, void* o, void* o_s, float* lse, void* lin_state, void* ws,
            size_t ws_bytes, sla_stream_t stream) {
  return fwd_impl(s, q, k, v, lut, w, bias, o, o_s, lse, lin_state, ws, ws_bytes, nullptr, 0, stream);
}

int sla_fwd_gather(const sla_shape* s, const void* q, const void* k, const void* v, const int32_t* lut,
                   const float* w, const float* bias, void* o, void* o_s, float* lse, void* lin_state, void* ws,
                   size_t ws_bytes, void* const* gather_dst, int n_gather, sla_stream_t stream) {
  return fwd_impl(s, q, k, v, lut, w, bias, o, o_s, lse, lin_state, ws, ws_bytes, gather_dst, n_gather, stream);
}

int sla_enable_peer_access(int peer_device) {
  int dev = 0;
  SLA_CUDA_OK(cudaGetDevice(&dev));
  if (peer_device == dev) return SLA_OK;
  int can = 0;
  SLA_CUDA_OK(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return SLA_ERR_UNSUPPORTED;
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return SLA_OK; }
  SLA_CUDA_OK(e);
  return SLA_OK;
}

int sla_ipc_export(const void* ptr, void* handle64, size_t* offset) {
  if (!ptr || !handle64 || !offset) return SLA_ERR_NULL;
  // the handle names the whole allocation `ptr` lies in: find its base
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  SLA_CUDA_OK(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
  if (qres != cudaDriverEntryPointSuccess || fn == nullptr) return SLA_ERR_UNSUPPORTED;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) {
    set_last_cuda_error(cudaErrorInvalidValue);
    return SLA_ERR_CUDA;
  }
  cudaIpcMemHandle_t h;
  SLA_CUDA_OK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle64, &h, sizeof(h));
  *offset = reinterpret_cast<CUdeviceptr>(ptr) - base;
  return SLA_OK;
}

int sla_ipc_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return SLA_ERR_NULL;
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) == 64, "CUDA IPC handles are 64 bytes");
  memcpy(&h, handle64, sizeof(h));
  // opened with the ACCESSING device current: the mapping (and, lazily, peer access to the owning GPU) is set up for
  // this device's kernels. A handle opened under the owner's device index is only usable by that device.
  SLA_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return SLA_OK;
}

int sla_ipc_close(void* ptr) {
  if (!ptr) return SLA_ERR_NULL;
  SLA_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return SLA_OK;
}

static int sparse_bwd_impl(const sla_shape* s, const void* q, const void* k, const void* v, const void* o_s,
                           const float* lse, const void* do_s, const int32_t* lut, const int32_t* col_offsets,
                           const int32_t* col_index, void* dq, void* dk, void* dv, unsigned char* ws,
                           int accumulate_legacy, cudaStream_t st, const void* lin_dh = nullptr,
                           const float* lin_dz = nullptr) {
  WsSparseBwd w = ws_sparse_bwd(s);
  BwdParams p;
  p.q = q; p.k = k; p.v = v; p.o_s = o_s; p.d_o = do_s; p.lse = lse;
  p.delta = reinterpret_cast<float*>(ws + w.delta); p.lut = lut;
  p.col_offsets = col_offsets; p.col_index = col_index; p.dq = dq; p.dk = dk; p.dv = dv;
  p.L = s->L; p.mb = ceil_div(s->L, s->BLKQ); p.nb = ceil_div(s->L, s->BLKK); p.topk = s->topk;
  p.scale = softmax_scale(s); p.scale_log2 = p.scale * kLog2e; p.accumulate = accumulate_legacy;
  p.lin_dh = lin_dh; p.lin_dz = lin_dz;
  if (!(s->flags & SLA_FLAG_LEGACY_MMA)) {
    int rc = run_sparse_bwd_tc(s, p, ws + w.stats, st);
    if (rc != SLA_ERR_BAD_SHAPE) return rc;   // lists too long for the tcgen05 kernel's shared memory
  }
  return run_sparse_bwd_mma(s, p, st);
}

// Backward of sla_fwd with SLA_FLAG_LINEAR_UNSELECTED (algebra: linear_bwd_unselected.cu). `base` is the workspace of
// sla_bwd: the all-token regions, the sparse backward's, then ws_bwd_unselected; its 16-bit W has been written.
static int bwd_unselected(const sla_shape* s, const void* q, const void* k, const void* v, const void* o_s,
                          const float* lse, const void* d_o, const int32_t* lut, const int32_t* col_offsets,
                          const int32_t* col_index, const float* w, const void* lin_state, void* dq, void* dk,
                          void* dv, float* dw, float* dbias, unsigned char* base, cudaStream_t st) {
  const WsBwd wb = ws_bwd(s);
  unsigned char* sparse_ws = base + wb.total;
  unsigned char* ub = sparse_ws + ws_sparse_bwd(s).total;
  const WsBwdUnselected wu = ws_bwd_unselected(s);
  const int nb = ceil_div(s->L, s->BLKK), Lpad = ceil_div(s->L, 128) * 128;
  const size_t bh = size_t(s->B) * s->H;
  int rc;
  // the forward's intermediates again: phi(q), phi(k), and the selected blocks' share C_num, C_den
  if ((rc = run_feature_map(s, q, ub + wu.phiq, st)) != SLA_OK) return rc;
  if ((rc = run_feature_map(s, k, ub + wu.phik, st)) != SLA_OK) return rc;
  FwdParams pc = make_fwd(s, ub + wu.phiq, ub + wu.phik, v, lut, ub + wu.cnum, nullptr,
                          reinterpret_cast<float*>(ub + wu.cden), nullptr, nullptr);
  pc.plain = 1;
  if ((rc = run_sparse_fwd_tc(s, pc, st)) != SLA_OK) return rc;
  // row pass: -dN, dden, the all-token part of dphi_q (into dq), and the partials of G, dz, db, G2
  SLA_CUDA_OK(cudaMemsetAsync(ub + wu.stats, 0, bh * Lpad * sizeof(float2), st));
  UnselBwdParams up;
  up.phiq = ub + wu.phiq; up.d_o = d_o; up.cnum = ub + wu.cnum;
  up.cden = reinterpret_cast<const float*>(ub + wu.cden);
  up.lin_state = lin_state; up.wbits = base + wb.wbits;
  up.dn_neg = ub + wu.dn_neg; up.dphi = dq;
  up.stats = reinterpret_cast<float2*>(ub + wu.stats);
  up.g_partial = reinterpret_cast<float*>(ub + wu.g_partial);
  up.L = s->L; up.Lpad = Lpad; up.nch = wb.nch; up.rows = wb.rows; up.all_selected = s->topk >= nb ? 1 : 0;
  if ((rc = run_linear_bwd_unselected_rows(s, up, st)) != SLA_OK) return rc;
  LinBwdParams lp;
  lp.q = q; lp.k = k; lp.v = v; lp.d_o = d_o; lp.lin_state = lin_state; lp.wbits = base + wb.wbits; lp.w = w;
  lp.dq = dq; lp.dk = dk; lp.dv = dv;
  lp.g_partial = up.g_partial;
  lp.g_sum = reinterpret_cast<float*>(ub + wu.g_sum);
  lp.dh = base + wb.dh;
  lp.dz = reinterpret_cast<float*>(base + wb.dz);
  lp.dw_part = reinterpret_cast<float*>(base + wb.dw_part);
  lp.dw = dw; lp.dbias = dbias; lp.L = s->L; lp.nch = wb.nch; lp.rows = wb.rows;
  lp.g_stride = 2 * s->D * s->D + 2 * s->D; lp.has_g2 = 1;
  if ((rc = run_linear_bwd_reductions(s, lp, st)) != SLA_OK) return rc;
  // the product without softmax over the selected blocks, on (phi(q), phi(k), v) with dO = -dN, delta = dden:
  // dq += dS phi(k) (still a gradient of phi(q)); dk = phi'(k)(v dH^T + dz + dS^T phi(q)); dv = phi(k) dH + P^T dO
  BwdParams bp;
  bp.q = ub + wu.phiq; bp.k = ub + wu.phik; bp.v = v; bp.o_s = nullptr; bp.d_o = ub + wu.dn_neg; bp.lse = nullptr;
  bp.delta = nullptr; bp.lut = lut; bp.col_offsets = col_offsets; bp.col_index = col_index;
  bp.dq = dq; bp.dk = dk; bp.dv = dv;
  bp.L = s->L; bp.mb = ceil_div(s->L, s->BLKQ); bp.nb = nb; bp.topk = s->topk;
  bp.scale = 1.0f; bp.scale_log2 = 1.0f; bp.accumulate = 1;
  bp.lin_dh = lp.dh; bp.lin_dz = lp.dz; bp.plain = 1;
  if ((rc = run_sparse_bwd_tc(s, bp, ub + wu.stats, st)) != SLA_OK) return rc;
  if ((rc = run_feature_map_bwd(s, ub + wu.phiq, dq, st)) != SLA_OK) return rc;   // dq = phi'(q) dphi_q
  // the softmax branch adds its dq, dk, dv
  return sparse_bwd_impl(s, q, k, v, o_s, lse, d_o, lut, col_offsets, col_index, dq, dk, dv, sparse_ws, 1, st);
}

int sla_sparse_bwd(const sla_shape* s, const void* q, const void* k, const void* v, const void* o_s,
                   const float* lse, const void* do_s, const int32_t* lut, const int32_t* col_offsets,
                   const int32_t* col_index, void* dq, void* dk, void* dv, void* ws, size_t ws_bytes,
                   sla_stream_t stream) {
  if (!q || !k || !v || !o_s || !lse || !do_s || !lut || !col_offsets || !col_index || !dq || !dk || !dv || !ws)
    return SLA_ERR_NULL;
  int rc = check_common(s);
  if (rc != SLA_OK) return rc;
  if (!all_aligned({q, k, v, o_s, do_s, dq, dk, dv, ws})) return SLA_ERR_BAD_ALIGN;
  if (ws_bytes < ws_sparse_bwd(s).total) return SLA_ERR_WS_TOO_SMALL;
  return sparse_bwd_impl(s, q, k, v, o_s, lse, do_s, lut, col_offsets, col_index, dq, dk, dv,
                         static_cast<unsigned char*>(ws), 0, static_cast<cudaStream_t>(stream));
}

int sla_bwd(const sla_shape* s, const void* q, const void* k, const void* v, const void* o_s, const float* lse,
            const void* d_o, const int32_t* lut, const int32_t* col_offsets, const int32_t* col_index,
            const float* w, const void* lin_state, void* dq, void* dk, void* dv, float* dw, float* dbias,
            void* ws, size_t ws_bytes, sla_stream_t stream) {
  const bool linear_only = s && (s->flags & SLA_FLAG_LINEAR_ONLY) != 0;
  if (!q || !k || !v || !d_o || !dq || !dk || !dv || !ws) return SLA_ERR_NULL;
  if (!linear_only && (!o_s || !lse || !lut || !col_offsets || !col_index)) return SLA_ERR_NULL;
  int rc = check_common(s);
  if (rc != SLA_OK) return rc;
  if (!all_aligned({q, k, v, o_s, d_o, dq, dk, dv, lin_state, ws})) return SLA_ERR_BAD_ALIGN;
  if (linear_only && (s->flags & SLA_FLAG_SPARSE_ONLY)) return SLA_ERR_UNSUPPORTED;
  WsBwd wb = ws_bwd(s);
  if (ws_bytes < ws_bwd_total(s)) return SLA_ERR_WS_TOO_SMALL;
  unsigned char* base = static_cast<unsigned char*>(ws);
  unsigned char* sparse_ws = base + wb.total;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (s->flags & SLA_FLAG_SPARSE_ONLY)
    return sparse_bwd_impl(s, q, k, v, o_s, lse, d_o, lut, col_offsets, col_index, dq, dk, dv, sparse_ws, 0, st);
  if (!w || !lin_state || !dw || !dbias) return SLA_ERR_NULL;
  const bool legacy = (s->flags & SLA_FLAG_LEGACY_MMA) != 0;
  rc = convert_proj(s, w, nullptr, base + wb.wbits, st);
  if (rc != SLA_OK) return rc;
  if (s->flags & SLA_FLAG_LINEAR_UNSELECTED) {
    if (legacy || linear_only || !sparse_bwd_tc_fits(s) || !sparse_fwd_tc_fits(s)) return SLA_ERR_UNSUPPORTED;
    return bwd_unselected(s, q, k, v, o_s, lse, d_o, lut, col_offsets, col_index, w, lin_state, dq, dk, dv, dw,
                          dbias, base, st);
  }
  LinBwdParams lp;
  lp.q = q; lp.k = k; lp.v = v; lp.d_o = d_o; lp.lin_state = lin_state; lp.wbits = base + wb.wbits; lp.w = w;
  lp.dq = dq; lp.dk = dk; lp.dv = dv;
  lp.g_sum = reinterpret_cast<float*>(base + wb.g_sum);
  lp.g_partial = reinterpret_cast<float*>(base + wb.g_partial);
  lp.dh = base + wb.dh;
  lp.dz = reinterpret_cast<float*>(base + wb.dz);
  lp.dw_part = reinterpret_cast<float*>(base + wb.dw_part);
  lp.dw = dw; lp.dbias = dbias; lp.L = s->L; lp.nch = wb.nch; lp.rows = wb.rows;
  // Linear branch first (plain stores), then the sparse kernels add their part: the tcgen05 dQ kernel through TMA
  // reduce-add stores, the mma.sync kernels by reading the tile back. With the tcgen05 kernels the linear
  // branch's dk, dv are not a pass of their own: the dK/dV kernel computes them in its epilogue from dH and dz.
  const bool fuse_kv = !linear_only && !legacy && sparse_bwd_tc_fits(s);
  lp.accumulate = 0;
  lp.skip_kv = fuse_kv ? 1 : 0;
  lp.tc_pass_a = legacy ? 0 : 1;
  rc = run_linear_bwd(s, lp, st);
  if (rc != SLA_OK || linear_only) return rc;
  return sparse_bwd_impl(s, q, k, v, o_s, lse, d_o, lut, col_offsets, col_index, dq, dk, dv, sparse_ws, 1, st,
                         fuse_kv ? lp.dh : nullptr, fuse_kv ? lp.dz : nullptr);
}

}  // extern "C"
