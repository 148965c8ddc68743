/*
 * sla_b200 -- C ABI of the B200 (sm_100a) implementation of the SLA attention hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle. The caller owns
 * all memory (inputs, outputs and workspaces); except where an entry point says otherwise the
 * library allocates nothing, keeps no pointer after returning, enqueues all work on the given
 * stream and never synchronises. Return value: SLA_OK (0) or a negative sla_status.
 *
 * Tensor layouts (all contiguous, row-major):
 *   q, k, v, o, o_s, do, dq, dk, dv : (B, H, L, D)     16-bit float given by sla_shape.dtype
 *   lse, delta                      : (B, H, L)        fp32, log2 units of the scaled score
 *   lut                             : (B, H, M_BLOCKS, topk) int32, ascending inside a row
 *   sparse_map                      : (B, H, M_BLOCKS, N_BLOCKS) int8 0/1
 *   col_offsets                     : (B, H, N_BLOCKS + 1) int32   } per-KV-block list of the
 *   col_index                       : (B, H, M_BLOCKS * topk) int32 } query blocks that selected it
 *   lin_state                       : (B, H, 2*D*D + D) 16-bit: H = phi(k)^T v, z = sum phi(k), then H W^T
 *                                     (sla_linear_state fills H and z; sla_fwd also the last part)
 *   w, bias                         : (D, D), (D)      fp32 (nn.Linear parameters of proj_l)
 * with M_BLOCKS = ceil(L / BLKQ), N_BLOCKS = ceil(L / BLKK).
 *
 * "Replaces" comments name the reference (thu-ml/SLA) interface each entry point stands in for,
 * by path inside that project.
 */
#ifndef SLA_B200_H_
#define SLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* sla_stream_t; /* a cudaStream_t / CUstream */

#if defined(__GNUC__)
#define SLA_API __attribute__((visibility("default")))
#else
#define SLA_API
#endif

enum sla_status {
  SLA_OK = 0,
  SLA_ERR_BAD_SHAPE = -1,   /* unsupported D / BLKQ / BLKK / empty tensor */
  SLA_ERR_BAD_DTYPE = -2,
  SLA_ERR_BAD_ALIGN = -3,   /* a tensor pointer is not 16-byte aligned */
  SLA_ERR_BAD_TOPK = -4,    /* topk < 1 or topk > N_BLOCKS (the reference divides 0/0 there) */
  SLA_ERR_WS_TOO_SMALL = -5,
  SLA_ERR_WRONG_ARCH = -6,  /* the current device is not compute capability 10.x */
  SLA_ERR_CUDA = -7,        /* a CUDA runtime call failed; see sla_last_cuda_error() */
  SLA_ERR_TIMEOUT = -8,     /* a bounded device-side wait ran out */
  SLA_ERR_NULL = -9,        /* a required pointer is NULL */
  SLA_ERR_UNSUPPORTED = -10
};

enum sla_dtype { SLA_BF16 = 0, SLA_FP16 = 1, SLA_FP32 = 2 };
enum sla_feature { SLA_PHI_SOFTMAX = 0, SLA_PHI_RELU = 1, SLA_PHI_ELU = 2 };
enum sla_op { SLA_OP_BLOCK_MAP = 0, SLA_OP_FWD = 1, SLA_OP_BWD = 2, SLA_OP_LINEAR_STATE = 3,
              SLA_OP_SAGE_FWD = 4, SLA_OP_SPARSE_BWD = 5 };
enum sla_flags {
  SLA_FLAG_SPARSE_ONLY = 1, /* skip the linear branch and proj_l (the `_attention` operator) */
  SLA_FLAG_LEGACY_MMA = 2,  /* use the mma.sync kernels instead of the tcgen05 ones */
  SLA_FLAG_LINEAR_UNSELECTED = 4, /* sla_fwd, sla_bwd: the linear branch of query block i sums over the KV blocks
                                    that block did NOT select (the scope drawn in assets/overview_of_SLA.png)
                                    instead of over all tokens (core.py:92-96). tcgen05 kernels only. */
  SLA_FLAG_LINEAR_ONLY = 16,     /* sla_bwd only: differentiate the linear branch and proj_l alone, the sparse branch
                                    being a constant of the graph (the quantized forward of SageSLA/core.py:114-146
                                    has no backward; core.py:148-158 after it is ordinary autograd). o_s, lse, lut and
                                    the column lists are not read and may be NULL. */
  SLA_FLAG_STATE_READY = 8       /* sla_fwd / sage_sla_fwd only: sla_fwd_prepare / sage_sla_prepare has already run
                                    for this shape on the same inputs, lin_state and workspace (and has completed,
                                    or is ordered before this call on the stream) */
};

typedef struct sla_shape {
  int32_t B, H, L, D;     /* D in {64, 128} */
  int32_t BLKQ, BLKK;     /* BLKQ in {64, 128}, BLKK == 64 (kernel.py:247-248) */
  int32_t topk;           /* selected KV blocks per query block, see sla_topk_count */
  int32_t dtype;          /* SLA_BF16 or SLA_FP16: element type of q,k,v,o and of the MMAs */
  int32_t feature_map;    /* sla_feature */
  int32_t flags;          /* sla_flags */
  float qk_scale;         /* softmax scale; 0 selects D^-0.5 (kernel.py:251-252) */
} sla_shape;

SLA_API int sla_version(void);
SLA_API const char* sla_status_string(int status);
/* Text of the last CUDA runtime error seen by the calling thread inside this library. */
SLA_API const char* sla_last_cuda_error(void);
/* The tcgen05 kernels bound every device-side wait; when one runs out the kernel records a code in
 * a device word and stops working: that launch and every later tcgen05 launch on the device leave their
 * outputs unwritten until the word is cleared. This call synchronises the device, stores the code
 * (0 = none) in *code, optionally clears it, and returns SLA_ERR_TIMEOUT when the code is non-zero.
 * Poll it where the host synchronises anyway (once per step). */
SLA_API int sla_poll_device_error(int* code, int clear);
/* Diagnostic: the limit of every device-side wait on the current device, in nanoseconds (default 2 s;
 * 0 restores the default). A synchronous copy to the device. */
SLA_API int sla_debug_set_wait_limit_ns(unsigned long long ns);
/* Test hook for the time-out path: while set, the first CTA of the tcgen05 forward never requests its first
 * K tile, so its waits run out, it records a code and leaves through the same teardown as a real time-out
 * (shared-memory copies drained, tensor memory freed). Nothing faults; clear it and the error word afterwards. */
SLA_API int sla_debug_drop_first_k_tile(int on);
/* Diagnostic: give the backward tcgen05 kernels a device buffer of 2 x 1024 int64 into which the
 * first CTA of each kernel records SM-clock timestamps of its pipeline events; NULL switches it off. */
SLA_API int sla_debug_set_trace(void* device_buffer);
/* Diagnostic: number of kernels this library has launched in the process so far. */
SLA_API long long sla_launch_count(void);

/* Which kernels serve `op` (SLA_OP_FWD, SLA_OP_BWD, SLA_OP_SPARSE_BWD, SLA_OP_SAGE_FWD) for `shape`: 0 = the
 * tcgen05 kernels, 1 = the mma.sync kernels (asked for with SLA_FLAG_LEGACY_MMA, or taken automatically when a
 * tile's block list does not fit the tcgen05 kernels' shared memory: forward top-k above about 8,000 at D = 128;
 * backward M_BLOCKS above 1,536 or top-k above 2,100 at D = 128, M_BLOCKS above 5,500 at D = 64), or a negative
 * sla_status. No counterpart in the reference, which has one set of kernels. */
SLA_API int sla_kernel_path(const sla_shape* shape, int op);

/* Replaces sparse_linear_attention/utils.py:61-62: min(n_blocks, int(topk_ratio * n_blocks)). */
SLA_API int sla_topk_count(int n_blocks, double topk_ratio);

/* Bytes of caller-provided workspace `op` needs for `shape` (a multiple of 256). */
SLA_API size_t sla_workspace_bytes(const sla_shape* shape, int op);

/*
 * Replaces sparse_linear_attention/utils.py:55-67 get_block_map (with mean_pool / compress_kernel,
 * utils.py:21-52). q and k are in `in_dtype` (any sla_dtype: the reference predicts the mask on the
 * tensors as given, core.py:83). Writes lut (required); sparse_map, col_offsets + col_index are
 * optional (NULL to skip; the column lists need sparse_map or workspace room for it).
 * Ties at the k-th score go to the lower block index.
 */
SLA_API int sla_block_map(const sla_shape* shape, int in_dtype, const void* q, const void* k,
                  int32_t* lut, int8_t* sparse_map, int32_t* col_offsets, int32_t* col_index,
                  void* ws, size_t ws_bytes, sla_stream_t stream);

/* The step before the path, fused with the first pass of the mask prediction. The attention layer of a video DiT
 * produces q and k, normalises each head's rows (RMS norm with a learned gain) and rotates them (rotary position
 * embedding) before it calls the operator (the caller of sparse_linear_attention/core.py:69); sla_block_map then reads q
 * once and k twice again. This entry point applies
 *     y = x * rsqrt(mean_D(x^2) + eps) * gain            (skipped for a NULL gain)
 *     (a, b) -> (a cos - b sin, a sin + b cos) per pair  (skipped for NULL tables; rope_cos, rope_sin: (L, D/2) fp32;
 *                                                         pairs (y[2i], y[2i+1]) if `interleaved`, else (y[i], y[i+D/2]))
 * to q_in, k_in (shape.dtype, 16-bit), writes q_out, k_out (may alias the inputs) and leaves in `pooled_sums`
 * (sla_pooled_sums_bytes) the fp32 per-block column sums of the rows it wrote. sla_block_map_pooled finishes the
 * prediction from those sums without touching q or k. No counterpart in the reference. */
SLA_API size_t sla_pooled_sums_bytes(const sla_shape* shape);
SLA_API int sla_qk_norm_rope_pool(const sla_shape* shape, const void* q_in, const void* k_in, const float* gain_q,
                                  const float* gain_k, const float* rope_cos, const float* rope_sin, float eps,
                                  int interleaved, void* q_out, void* k_out, void* pooled_sums, size_t sums_bytes,
                                  sla_stream_t stream);
/* sla_block_map from the block sums of sla_qk_norm_rope_pool (workspace: sla_workspace_bytes(shape, SLA_OP_BLOCK_MAP);
 * shape.dtype is the dtype q and k were written in). One rounding point differs from utils.py:56 + :40: the reference
 * rounds every element of k - mean(k) to the tensor dtype before pooling, this takes round(block mean - mean(k)). The
 * pooled K values differ by a fraction of a unit in the last place, so a row's selection can differ from
 * sla_block_map's where two scores are within rounding of each other at the k-th place. */
SLA_API int sla_block_map_pooled(const sla_shape* shape, const void* pooled_sums, int32_t* lut, int8_t* sparse_map,
                                 int32_t* col_offsets, int32_t* col_index, void* ws, size_t ws_bytes,
                                 sla_stream_t stream);

/* Builds the per-KV-block query-block lists from a 0/1 block map. Stands in for the way
 * sparse_linear_attention/kernel.py:208-210 consults k_block_id inside the dK/dV kernel: callers
 * that bring their own sparse_map (the `_attention.apply` signature, kernel.py:242) convert it once. */
SLA_API int sla_column_lists(const sla_shape* shape, const int8_t* sparse_map, int32_t* col_offsets,
                             int32_t* col_index, sla_stream_t stream);

/* Converts `count` block indices between the 32-bit form every entry point here reads and writes (lut,
 * col_index) and an unsigned 16-bit form, for callers that keep block maps across calls (the reference's own
 * benchmark predicts the map once, evaluate/bench_kernel.py:79, and a diffusion sampler may reuse it over several
 * steps): (src_bits, dst_bits) = (32, 16) packs, (16, 32) unpacks. Indices must be below 65,536 (L < 4 Mi tokens).
 * The reference keeps its LUT as int64 (utils.py:64); no counterpart there. */
SLA_API int sla_index_convert(const void* src, int src_bits, void* dst, int dst_bits, size_t count,
                              sla_stream_t stream);

/* Replaces sparse_linear_attention/kernel.py:242-274 _attention.forward (+ _attn_fwd :21-82). */
SLA_API int sla_sparse_fwd(const sla_shape* shape, const void* q, const void* k, const void* v,
                   const int32_t* lut, void* o_s, float* lse, sla_stream_t stream);

/* Replaces sparse_linear_attention/kernel.py:277-320 _attention.backward (+ kernels :85-237).
 * Workspace: sla_workspace_bytes(shape, SLA_OP_SPARSE_BWD) (row statistics: delta of
 * kernel.py:102-105 next to lse). dq, dk, dv are overwritten. */
SLA_API int sla_sparse_bwd(const sla_shape* shape, const void* q, const void* k, const void* v,
                   const void* o_s, const float* lse, const void* do_s, const int32_t* lut,
                   const int32_t* col_offsets, const int32_t* col_index, void* dq, void* dk,
                   void* dv, void* ws, size_t ws_bytes, sla_stream_t stream);

/* Replaces the feature map on k and the two state reductions of
 * sparse_linear_attention/core.py:91,93-94 (kvsum, ksum). Writes lin_state. */
SLA_API int sla_linear_state(const sla_shape* shape, const void* k, const void* v, void* lin_state,
                     void* ws, size_t ws_bytes, sla_stream_t stream);

/* Same result as sla_linear_state, for callers that cannot supply a workspace. No counterpart in the
 * reference. Some hosts fix their device-memory budget at start-up -- an inference server that gives
 * the whole GPU to its own pool, a plugin host that treats a cudaMalloc in steady state as an error --
 * and so have nothing to pass as `ws`. This entry point allocates nothing (no cudaMalloc, cudaFree or
 * allocating library call): its scratch is a 16 MiB array reserved inside the library image, which
 * every GPU that loads the library holds until the process exits.
 *   - Limit: B*H*(D*D + D)*4 bytes must fit in those 16 MiB (B*H <= 254 at D = 128, <= 1008 at
 *     D = 64); larger shapes return SLA_ERR_WS_TOO_SMALL. Long sequences use fewer, longer row chunks.
 *   - The first call on each device looks up the array's device address (a one-time, synchronous
 *     query); make that first call before starting any stream capture.
 *   - All calls on a device share the array and it keeps the previous call's contents; every slot a
 *     call reads is first overwritten by that call, so nothing needs clearing, but two calls whose
 *     kernels overlap on the GPU (different streams) race on it. Serialise them.
 */
SLA_API int sla_linear_state_static(const sla_shape* shape, const void* k, const void* v,
                                    void* lin_state, sla_stream_t stream);

/* Replaces sparse_linear_attention/core.py:88-100 (everything in SparseLinearAttention.forward
 * after get_block_map and the dtype casts): sparse branch, feature maps, linear branch, proj_l and
 * the final sum. o_s may be NULL when no backward will follow. lin_state and lse are outputs. */
SLA_API int sla_fwd(const sla_shape* shape, const void* q, const void* k, const void* v,
            const int32_t* lut, const float* w, const float* bias, void* o, void* o_s, float* lse,
            void* lin_state, void* ws, size_t ws_bytes, sla_stream_t stream);

/* sla_fwd whose epilogue also writes the output tile by tile into up to 8 further buffers, each laid out like `o`
 * (a (B, H, L, D) block): gather_dst[i] is the address, in THIS process's address space, of the place in
 * destination i where this call's o belongs. A destination may be memory of another GPU of the node mapped into
 * this process (CUDA IPC, peer access enabled: sla_enable_peer_access): every rank of a (batch x head)-sharded run
 * then leaves its slice of o in every peer's full-size buffer, and the forward is its own all-gather, written
 * over NVLink with plain stores while the kernel computes (no TMA and no multicast touch peer memory). Stands in for
 * the all-gather a caller of sparse_linear_attention/core.py:69 runs after the module when heads are sharded over
 * GPUs; no counterpart in the reference, which is single-GPU. The copies are complete when the stream has reached
 * the end of this call; readers on other GPUs need their own synchronisation with it (a barrier between the ranks).
 * tcgen05 kernels only: SLA_ERR_UNSUPPORTED with SLA_FLAG_LEGACY_MMA, SLA_FLAG_LINEAR_UNSELECTED or a top-k
 * beyond the tcgen05 forward's list budget. */
SLA_API int sla_fwd_gather(const sla_shape* shape, const void* q, const void* k, const void* v, const int32_t* lut,
                   const float* w, const float* bias, void* o, void* o_s, float* lse, void* lin_state, void* ws,
                   size_t ws_bytes, void* const* gather_dst, int n_gather, sla_stream_t stream);
/* Helpers for sla_fwd_gather (no counterpart in the reference). sla_ipc_export: the 64-byte CUDA IPC handle of the
 * device allocation `ptr` lies in (cudaMalloc memory, e.g. a PyTorch tensor without expandable segments) and ptr's
 * offset inside it; send both to the other processes of the node. sla_ipc_open maps such an allocation into this
 * process FOR THE CURRENT DEVICE: call it with the GPU current whose kernels will write the buffer, not the GPU that
 * owns it; *ptr is the allocation's base (add the offset). sla_ipc_close unmaps it. */
SLA_API int sla_ipc_export(const void* ptr, void* handle64, size_t* offset);
SLA_API int sla_ipc_open(const void* handle64, void** ptr);
SLA_API int sla_ipc_close(void* ptr);
/* Enables access from the current device to `peer_device`'s memory (cudaDeviceEnablePeerAccess; fine if it already
 * is). SLA_ERR_UNSUPPORTED when the two GPUs have no peer path. */
SLA_API int sla_enable_peer_access(int peer_device);

/* The part of sla_fwd that depends on k, v and proj_l only (core.py:91,93-94 and the 16-bit copy of the
 * projection): a caller may run it on a second stream next to sla_block_map, which depends on q and k only,
 * and then call sla_fwd with SLA_FLAG_STATE_READY and the same lin_state and workspace. No counterpart in the
 * reference, where PyTorch runs these operators one after the other. */
SLA_API int sla_fwd_prepare(const sla_shape* shape, const void* k, const void* v, const float* w,
                    const float* bias, void* lin_state, void* ws, size_t ws_bytes, sla_stream_t stream);

/* Replaces the autograd backward of sparse_linear_attention/core.py:88-100 (kernel.py:277-320 for
 * the sparse branch; PyTorch autograd of core.py:90-100 for the rest). dw (D,D) and dbias (D) are
 * fp32 and are OVERWRITTEN with this call's gradient. */
SLA_API int sla_bwd(const sla_shape* shape, const void* q, const void* k, const void* v, const void* o_s,
            const float* lse, const void* d_o, const int32_t* lut, const int32_t* col_offsets,
            const int32_t* col_index, const float* w, const void* lin_state, void* dq, void* dk,
            void* dv, float* dw, float* dbias, void* ws, size_t ws_bytes, sla_stream_t stream);

/* Replaces SageSLA/core.py:100-158 (SageSparseLinearAttention.forward after get_block_map and the
 * casts): INT8 Q.K^T with per-block scales and K-mean smoothing, FP8 e4m3 P.V, then the same
 * linear branch and proj_l. BLKQ must be 128 and BLKK 64 (SageSLA/README.md:16-17), D 64 or 128
 * (SageSLA/core.py:112). */
SLA_API int sage_sla_fwd(const sla_shape* shape, const void* q, const void* k, const void* v,
                 const int32_t* lut, const float* w, const float* bias, void* o, void* lin_state,
                 void* ws, size_t ws_bytes, sla_stream_t stream);

/* sage_sla_fwd with the gather destinations of sla_fwd_gather (same meaning, same limits: up to 8 further
 * (B, H, L, D) blocks, peers' memory allowed, written from the kernel's epilogue with plain stores). */
SLA_API int sage_sla_fwd_gather(const sla_shape* shape, const void* q, const void* k, const void* v,
                        const int32_t* lut, const float* w, const float* bias, void* o, void* lin_state, void* ws,
                        size_t ws_bytes, void* const* gather_dst, int n_gather, sla_stream_t stream);

/* The part of sage_sla_fwd that does not need the block map: the linear-branch state and the quantized copies of
 * q, k, v (SageSLA/core.py:102-108,127-129). A caller may run it on a second stream next to sla_block_map and then
 * call sage_sla_fwd with SLA_FLAG_STATE_READY and the same lin_state and workspace. */
SLA_API int sage_sla_prepare(const sla_shape* shape, const void* q, const void* k, const void* v, const float* w,
                     const float* bias, void* lin_state, void* ws, size_t ws_bytes, sla_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SLA_B200_H_ */
