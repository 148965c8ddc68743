// Layout of the caller-provided workspaces. Every region starts on a 256-byte boundary.
#pragma once
#include <stddef.h>

#include "../../include/sla_b200.h"

namespace sla {

inline size_t ws_round(size_t x) { return (x + 255) & ~size_t(255); }
inline int ws_ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- block-mask prediction ----
constexpr int kColsumRows = 512;  // rows of K summed by one CTA of the column-sum kernel
struct WsBlockMap {
  size_t colsum_partial;  // fp32 [BH][NCH][D]
  size_t kmean;           // fp32 [BH][D]
  size_t pooled_q;        // in-dtype [BH][M_BLOCKS][D]
  size_t pooled_k;        // in-dtype [BH][N_BLOCKS][D]
  size_t map;             // int8 [BH][M_BLOCKS][N_BLOCKS] (used when the caller passes no sparse_map)
  size_t total;
  int nch;
};
inline WsBlockMap ws_block_map(const sla_shape* s) {
  WsBlockMap w;
  size_t bh = size_t(s->B) * s->H;
  int mb = ws_ceil_div(s->L, s->BLKQ), nb = ws_ceil_div(s->L, s->BLKK);
  w.nch = ws_ceil_div(s->L, kColsumRows);
  size_t o = 0;
  w.colsum_partial = o; o += ws_round(bh * w.nch * s->D * 4);
  w.kmean = o;          o += ws_round(bh * s->D * 4);
  w.pooled_q = o;       o += ws_round(bh * mb * s->D * 4);
  w.pooled_k = o;       o += ws_round(bh * nb * s->D * 4);
  w.map = o;            o += ws_round(bh * mb * size_t(nb));
  w.total = o;
  return w;
}

// ---- linear-branch state: partial H (D x D) and z (D) per chunk of rows, fp32 ----
struct WsLinearState {
  size_t partial;  // fp32 [BH][NCH][D*D + D]
  size_t total;
  int nch;         // chunks per head
  int rows;        // rows per chunk (multiple of 128)
};
inline WsLinearState ws_linear_state(const sla_shape* s) {
  WsLinearState w;
  size_t bh = size_t(s->B) * s->H;
  // The split of a head's rows into chunks fixes the order of the fp32 sums. It depends on L alone, never on
  // B or H, so a (batch, head) unit gives the same bits whatever else is in the batch and however the units are
  // sharded over GPUs: at most 64 chunks per head, at least 512 rows per chunk.
  int nch = ws_ceil_div(s->L, 512);
  if (nch > 64) nch = 64;
  int rows = (ws_ceil_div(s->L, nch) + 127) / 128 * 128;
  w.rows = rows;
  w.nch = ws_ceil_div(s->L, rows);
  w.partial = 0;
  w.total = ws_round(bh * w.nch * (size_t(s->D) * s->D + s->D) * 4);
  return w;
}

// extra bytes the fused forward needs after the linear-state workspace: proj weight + bias in 16 bit
inline size_t ws_fwd_extra(const sla_shape* s) { return ws_round(size_t(s->D) * s->D * 2 + s->D * 2); }

// the "unselected blocks" scope of the linear branch: phi(q), phi(k), C_num as 16-bit (B,H,L,D), C_den fp32 (B,H,L)
struct WsUnselected {
  size_t phiq, phik, cnum, cden, total;
};
inline WsUnselected ws_unselected(const sla_shape* s) {
  WsUnselected w;
  size_t n = size_t(s->B) * s->H * s->L;
  size_t o = 0;
  w.phiq = o; o += ws_round(n * s->D * 2);
  w.phik = o; o += ws_round(n * s->D * 2);
  w.cnum = o; o += ws_round(n * s->D * 2);
  w.cden = o; o += ws_round(n * 4);
  w.total = o;
  return w;
}
inline size_t ws_fwd_total(const sla_shape* s) {
  size_t t = ws_linear_state(s).total + ws_fwd_extra(s);
  if (s->flags & SLA_FLAG_LINEAR_UNSELECTED) t += ws_unselected(s).total;
  return t;
}

// ---- backward ----
struct WsBwd {
  size_t wbits;     // 16-bit copy of W [D][D]
  size_t g_partial; // fp32 [BH][NCH][D*D + 2*D]: G, dz, db partials of the linear backward
  size_t dh;        // 16-bit [BH][D*D] dH, then fp32 [BH][D] dz
  size_t dz;
  size_t dw_part;   // fp32 [BH][D*D + D] per-head dW and db
  size_t g_sum;     // fp32 [BH][D*D + 2*D]
  size_t total;
  int nch, rows;
};
inline WsBwd ws_bwd(const sla_shape* s) {
  WsBwd w;
  size_t bh = size_t(s->B) * s->H;
  // chunks of the linear backward's row passes: a function of L alone, like ws_linear_state
  int nch = ws_ceil_div(s->L, 512);
  if (nch > 64) nch = 64;
  int rows = (ws_ceil_div(s->L, nch) + 127) / 128 * 128;
  w.rows = rows;
  w.nch = ws_ceil_div(s->L, rows);
  size_t dd = size_t(s->D) * s->D;
  size_t o = 0;
  w.wbits = o;     o += ws_round(dd * 2);
  w.g_partial = o; o += ws_round(bh * w.nch * (dd + 2 * s->D) * 4);
  w.dh = o;        o += ws_round(bh * dd * 2);
  w.dz = o;        o += ws_round(bh * s->D * 4);
  w.dw_part = o;   o += ws_round(bh * (dd + s->D) * 4);
  w.g_sum = o;     o += ws_round(bh * (dd + 2 * s->D) * 4);
  w.total = o;
  return w;
}

// ---- sparse backward: padded row statistics {lse, delta} and the plain delta array ----
struct WsSparseBwd {
  size_t stats;   // float2 [BH][Lpad], Lpad = ceil(L/128)*128
  size_t delta;   // fp32 [BH][L]
  size_t total;
};
inline WsSparseBwd ws_sparse_bwd(const sla_shape* s) {
  WsSparseBwd w;
  size_t bh = size_t(s->B) * s->H;
  size_t lpad = size_t(ws_ceil_div(s->L, 128)) * 128;
  size_t o = 0;
  w.stats = o; o += ws_round(bh * lpad * 8);
  w.delta = o; o += ws_round(bh * size_t(s->L) * 4);
  w.total = o;
  return w;
}

// ---- backward of the "unselected" linear scope (behind the two regions above) ----
struct WsBwdUnselected {
  size_t phiq, phik, cnum, dn_neg;   // 16-bit [BH][L][D]: phi(q), phi(k), C_num (recomputed), -dN
  size_t cden;                       // fp32 [BH][L]
  size_t stats;                      // float2 [BH][Lpad] {unused, dden}
  size_t g_partial;                  // fp32 [BH][NCH][2*D*D + 2*D]
  size_t g_sum;                      // fp32 [BH][2*D*D + 2*D]
  size_t total;
};
inline WsBwdUnselected ws_bwd_unselected(const sla_shape* s) {
  WsBwdUnselected w;
  const size_t bh = size_t(s->B) * s->H, n = bh * s->L;
  const size_t lpad = size_t(ws_ceil_div(s->L, 128)) * 128;
  const size_t rec = 2 * size_t(s->D) * s->D + 2 * s->D;
  const int nch = ws_bwd(s).nch;
  size_t o = 0;
  w.phiq = o;      o += ws_round(n * s->D * 2);
  w.phik = o;      o += ws_round(n * s->D * 2);
  w.cnum = o;      o += ws_round(n * s->D * 2);
  w.dn_neg = o;    o += ws_round(n * s->D * 2);
  w.cden = o;      o += ws_round(n * 4);
  w.stats = o;     o += ws_round(bh * lpad * 8);
  w.g_partial = o; o += ws_round(bh * nch * rec * 4);
  w.g_sum = o;     o += ws_round(bh * rec * 4);
  w.total = o;
  return w;
}
inline size_t ws_bwd_total(const sla_shape* s) {
  size_t t = ws_bwd(s).total + ws_sparse_bwd(s).total;
  if (s->flags & SLA_FLAG_LINEAR_UNSELECTED) t += ws_bwd_unselected(s).total;
  return t;
}

// ---- SageSLA quantized forward ----
struct WsSage {
  size_t lin;      // linear-state partials (same layout as WsLinearState)
  size_t wbits;    // 16-bit W + bias
  size_t kmean;    // fp32 [BH][D]
  size_t colsum;   // fp32 [BH][NCH][D] partial column sums of K, then [BH][NCH][D] column abs-max of V
  size_t q8;       // int8 [BH][L][128] (rows padded to one 128-byte swizzle atom when D = 64)
  size_t k8;       // int8 [BH][L][128]
  size_t v8;       // e4m3 [BH][L][128]
  size_t qscale;   // fp32 [BH][M_BLOCKS]
  size_t kscale;   // fp32 [BH][N_BLOCKS]
  size_t vscale;   // fp32 [BH][D]
  size_t lse;      // fp32 [BH][L]
  size_t total;
  int nch;
};
inline WsSage ws_sage(const sla_shape* s) {
  WsSage w;
  size_t bh = size_t(s->B) * s->H;
  int mb = ws_ceil_div(s->L, s->BLKQ), nb = ws_ceil_div(s->L, s->BLKK);
  w.nch = ws_ceil_div(s->L, kColsumRows);
  size_t o = 0;
  w.lin = o;    o += ws_linear_state(s).total;
  w.wbits = o;  o += ws_fwd_extra(s);
  w.kmean = o;  o += ws_round(bh * s->D * 4);
  w.colsum = o; o += ws_round(bh * w.nch * s->D * 4 * 2);
  w.q8 = o;     o += ws_round(bh * size_t(s->L) * 128);
  w.k8 = o;     o += ws_round(bh * size_t(s->L) * 128);
  w.v8 = o;     o += ws_round(bh * size_t(s->L) * 128);
  w.qscale = o; o += ws_round(bh * mb * 4);
  w.kscale = o; o += ws_round(bh * nb * 4);
  w.vscale = o; o += ws_round(bh * s->D * 4);
  w.lse = o;    o += ws_round(bh * size_t(s->L) * 4);
  w.total = o;
  return w;
}

}  // namespace sla
