// Housekeeping entry points of the C ABI: version, status text, shape validation, workspace sizes.
#include <atomic>
#include <math.h>
#include <stdio.h>

#include "common.cuh"
#include "workspace.h"

namespace sla {

static thread_local char g_last_error[256] = "";
static std::atomic<long long> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_last_cuda_error(cudaError_t e) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
}

int check_device_arch() {
  int dev = 0;
  SLA_CUDA_OK(cudaGetDevice(&dev));
  int major = 0;
  SLA_CUDA_OK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  return major == 10 ? SLA_OK : SLA_ERR_WRONG_ARCH;
}

int validate_shape(const sla_shape* s) {
  if (s == nullptr) return SLA_ERR_NULL;
  if (s->B < 1 || s->H < 1 || s->L < 1) return SLA_ERR_BAD_SHAPE;
  if (s->D != 64 && s->D != 128) return SLA_ERR_BAD_SHAPE;
  if (s->BLKQ != 64 && s->BLKQ != 128) return SLA_ERR_BAD_SHAPE;  // kernel.py:247
  if (s->BLKK != 64) return SLA_ERR_BAD_SHAPE;                    // kernel.py:248
  if (s->dtype != SLA_BF16 && s->dtype != SLA_FP16) return SLA_ERR_BAD_DTYPE;
  if (s->feature_map < SLA_PHI_SOFTMAX || s->feature_map > SLA_PHI_ELU) return SLA_ERR_UNSUPPORTED;
  int nb = ceil_div(s->L, s->BLKK);
  if (s->topk < 1 || s->topk > nb) return SLA_ERR_BAD_TOPK;
  if (static_cast<long long>(s->B) * s->H > 65535) return SLA_ERR_BAD_SHAPE;  // gridDim.y
  return SLA_OK;
}

}  // namespace sla

extern "C" {

int sla_version(void) { return 100; }

long long sla_launch_count(void) { return sla::g_launches.load(std::memory_order_relaxed); }

const char* sla_status_string(int status) {
  switch (status) {
    case SLA_OK: return "ok";
    case SLA_ERR_BAD_SHAPE: return "unsupported shape (D in {64,128}, BLKQ in {64,128}, BLKK == 64)";
    case SLA_ERR_BAD_DTYPE: return "unsupported dtype";
    case SLA_ERR_BAD_ALIGN: return "tensor pointer not 16-byte aligned";
    case SLA_ERR_BAD_TOPK: return "topk must be in [1, N_BLOCKS]";
    case SLA_ERR_WS_TOO_SMALL: return "workspace too small (see sla_workspace_bytes)";
    case SLA_ERR_WRONG_ARCH: return "device is not compute capability 10.x (B200)";
    case SLA_ERR_CUDA: return "CUDA runtime error (see sla_last_cuda_error)";
    case SLA_ERR_TIMEOUT: return "bounded device-side wait ran out";
    case SLA_ERR_NULL: return "required pointer is NULL";
    case SLA_ERR_UNSUPPORTED: return "unsupported option";
    default: return "unknown status";
  }
}

const char* sla_last_cuda_error(void) { return sla::g_last_error; }

int sla_topk_count(int n_blocks, double topk_ratio) {
  // Python: min(K, int(topk_ratio * K)) -- int() truncates toward zero, product in double.
  double prod = topk_ratio * static_cast<double>(n_blocks);
  int t = static_cast<int>(prod);
  return t < n_blocks ? t : n_blocks;
}

size_t sla_workspace_bytes(const sla_shape* s, int op) {
  if (s == nullptr) return 0;
  switch (op) {
    case SLA_OP_BLOCK_MAP: return sla::ws_block_map(s).total;
    case SLA_OP_LINEAR_STATE: return sla::ws_linear_state(s).total;
    case SLA_OP_FWD: return sla::ws_fwd_total(s);
    case SLA_OP_BWD: return sla::ws_bwd_total(s);
    case SLA_OP_SPARSE_BWD: return sla::ws_sparse_bwd(s).total;
    case SLA_OP_SAGE_FWD: return sla::ws_sage(s).total;
    default: return 0;
  }
}

}  // extern "C"
