// Internal launch interfaces shared by the translation units of libsla_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sla_b200.h"

namespace sla {

struct FwdParams {
  const void *q, *k, *v;
  const int32_t* lut;
  void* o;                // final output (or o_s when the linear branch is skipped)
  void* o_s;              // optional copy of the sparse branch output (needed by the backward)
  float* lse;
  const void* lin_state;  // [BH][2*D*D + D] 16-bit: H, z, then H W^T
  const void* wbits;      // [D*D + D] 16-bit: W then bias
  int L, mb, topk;
  float scale_log2;       // softmax scale * log2(e)
  int plain = 0;          // tcgen05 forward only: P = S without softmax, unnormalised O, row sums in `lse`
  // tcgen05 forward only: further copies of the output, written tile by tile from the epilogue with plain 16-byte
  // stores. Each pointer addresses a (B, H, L, D) block laid out like `o`; it may be memory of another GPU mapped
  // into this process (peer access enabled), which makes the forward its own all-gather.
  void* gather_dst[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n_gather = 0;
};

struct BwdParams {
  const void *q, *k, *v, *o_s, *d_o;
  const float* lse;
  float* delta;
  const int32_t* lut;
  const int32_t* col_offsets;
  const int32_t* col_index;
  void *dq, *dk, *dv;
  int L, mb, nb, topk;
  float scale, scale_log2;
  int accumulate;         // dq/dk/dv already hold the linear branch's contribution
  // tcgen05 path only: compute the linear branch's dk, dv in the epilogue of the dK/dV kernel (then dk, dv are
  // plainly stored, whatever `accumulate` says). lin_dh: [BH][D*D] 16-bit dH, lin_dz: [BH][D] fp32.
  const void* lin_dh = nullptr;
  const float* lin_dz = nullptr;
  // tcgen05 path only: differentiate the block-sparse product WITHOUT softmax, sum_{j in sel(i)} (q_i k_j^T) v_j and
  // its row sums (the selected blocks' share of the linear state in the "unselected" scope): P = S, dS = T2 - delta
  // with `delta` given by the caller in the row statistics (no pre-pass), no softmax scale. With lin_dh set, q and k
  // are feature maps already and dk = phi'(k) (v dH^T + dz + dK), dv = phi(k) dH + dV.
  int plain = 0;
};

struct LinBwdParams {
  const void *q, *k, *v, *d_o;
  const void* lin_state;  // H, z (16-bit)
  const void* wbits;      // W (16-bit)
  const float* w;         // W fp32
  void *dq, *dk, *dv;     // written (not accumulated) with the linear branch's gradients
  float* g_partial;       // [BH][NCH][D*D + 2D]
  float* g_sum;           // [BH][D*D + 2D]
  void* dh;               // [BH][D*D] 16-bit
  float* dz;              // [BH][D]
  float* dw_part;         // [BH][D*D + D]
  float *dw, *dbias;
  int L, nch, rows;
  int accumulate;         // add to what dq/dk/dv already hold instead of overwriting
  int skip_kv = 0;        // stop after dq and the per-head reductions (dk, dv are produced elsewhere)
  int tc_pass_a = 0;      // run pass A (dq, G, dz, db) as the tcgen05 kernel where it applies
  // "unselected" linear scope (linear_bwd_unselected.cu): per-chunk partials and per-head sums are records of
  // g_stride floats {G, dz, db, G2}, and the head's dW is G H - G2
  int g_stride = 0;       // 0: the default record D*D + 2*D
  int has_g2 = 0;
};

// Row pass of the backward of the "unselected" linear scope.
struct UnselBwdParams {
  const void *phiq, *d_o, *cnum;   // (BH, L, D) 16-bit: phi(q), dY, C_num
  const float* cden;               // (BH, L)
  const void* lin_state;           // H, z, H W^T
  const void* wbits;               // W 16-bit [n][k]
  void* dn_neg;                    // out (BH, L, D) 16-bit: -dY W / den
  void* dphi;                      // out (BH, L, D) 16-bit: the all-token part of dphi_q
  float2* stats;                   // out (BH, Lpad): {unused, dden}
  float* g_partial;                // out [BH][NCH][2*D*D + 2*D]
  int L, Lpad, nch, rows, all_selected;
};
int run_linear_bwd_unselected_rows(const sla_shape* s, const UnselBwdParams& p, cudaStream_t st);
int run_feature_map_bwd(const sla_shape* s, const void* phi, void* dphi_to_dx, cudaStream_t st);
int run_linear_bwd_reductions(const sla_shape* s, const LinBwdParams& p, cudaStream_t st);

int convert_proj(const sla_shape* s, const float* w, const float* bias, void* out, cudaStream_t st);
int run_sparse_fwd_mma(const sla_shape* s, const FwdParams& p, bool lin, cudaStream_t st);
int run_sparse_fwd_tc(const sla_shape* s, const FwdParams& p, cudaStream_t st);
int run_feature_map(const sla_shape* s, const void* x, void* out, cudaStream_t st);
int run_linear_readout_unselected(const sla_shape* s, const FwdParams& p, const void* cnum, const float* cden,
                                  cudaStream_t st);
int run_state_proj(const sla_shape* s, void* lin_state, const void* wbits, cudaStream_t st);
int read_tc_error(int* out, bool clear);
void set_trace_buffer(long long* p);
long long* trace_buffer();
int run_sparse_bwd_tc(const sla_shape* s, const BwdParams& p, void* stats, cudaStream_t st);
bool sparse_bwd_tc_fits(const sla_shape* s);
bool sparse_bwd_dq_pair_fits(const sla_shape* s);
bool sparse_fwd_tc_fits(const sla_shape* s);
// softmax variant: fills `stats` ({lse, delta} per row) itself; no-softmax variant (p.plain): reads it
int run_sparse_bwd_dq_pair(const sla_shape* s, const BwdParams& p, void* stats, int Lpad, cudaStream_t st);
int run_linear_state(const sla_shape* s, const void* k, const void* v, void* lin_state, float* partial,
                     int nch, int rows, cudaStream_t st);
int run_linear_state_static(const sla_shape* s, const void* k, const void* v, void* lin_state, cudaStream_t st);
int run_k_mean(const sla_shape* s, const void* k, float* partial, float* kmean, cudaStream_t st);
int run_sparse_bwd_mma(const sla_shape* s, const BwdParams& p, cudaStream_t st);
int run_linear_bwd(const sla_shape* s, const LinBwdParams& p, cudaStream_t st);
int run_linear_bwd_q_tc(const sla_shape* s, const LinBwdParams& p, cudaStream_t st);
// tcgen05 kernel for the per-chunk partials of the linear state (linear_state_tc.cu); SLA_ERR_UNSUPPORTED unless
// head dim 128 and rows % 128 == 0
int run_linear_state_partials_tc(const sla_shape* s, const void* k, const void* v, float* partial, int nch, int rows,
                                 cudaStream_t st);

}  // namespace sla
