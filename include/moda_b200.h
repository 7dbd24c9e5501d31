/*
 * moda_b200 — C ABI of the B200 (sm_100a) MoDA attention hot path.
 *
 * The reference (hustvl/MoDA) has no native layer: its operators are Python functions
 * that launch Triton kernels.  Each entry point below names the reference function
 * whose device work it replaces; the Python mirror of those functions
 * (moda_b200/ops.py) binds this library with ctypes.
 *
 * Conventions
 *   - Tensors are 4-D [B, T, H, D] with arbitrary element strides for B, T, H and a
 *     contiguous innermost D (moda_tensor4).  Pointers are DEVICE pointers, 16-byte
 *     aligned; the stride of every dimension of extent > 1 must be a positive multiple
 *     of 8 elements (zero or negative strides, as of expanded or flipped views, are
 *     refused with MODA_ERR_ALIGNMENT; a dimension of extent 1 may carry any stride).
 *     Inputs are never written.
 *   - Queries are folded the reference's way (moda_v14.py:2839-2852): q is
 *     [B, T_kv*G, H, D]; query row r belongs to base position t = r / G.
 *   - depth_k / depth_v are [B, T_kv*L, H, D]; row t*L + l is layer l at position t
 *     (moda_v14.py:1944-1945).  L == 0 means "no depth KV" (pass NULL tensors).
 *     With moda_problem.depth_rows_per_pos = Lmax > L they are instead the first L layers
 *     of an in-place layer cache [B, T_kv, Lmax, H, D] (row t*Lmax + l), see
 *     moda_b200_depth_append; the depth gradients use the same layout as the inputs.
 *   - lse is fp32 [B, T_kv*G, H] contiguous, in base-2 units (moda_v14.py:372-374).
 *   - Every call is asynchronous on `stream` (a cudaStream_t), never synchronises,
 *     never allocates device memory, and returns a moda_status (0 = success).
 *     Nothing is launched when a non-zero status is returned from validation.
 */
#ifndef MODA_B200_H_
#define MODA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum moda_status {
  MODA_OK = 0,
  MODA_ERR_NULL = 1,        /* required pointer is NULL */
  MODA_ERR_SHAPE = 2,       /* B/T/H/G/L out of range, T_q != T_kv*G ... */
  MODA_ERR_HEAD_DIM = 3,    /* D not in {64, 128} */
  MODA_ERR_DTYPE = 4,       /* dtype not bf16/fp16 */
  MODA_ERR_ALIGNMENT = 5,   /* pointer not 16-byte aligned, or a stride not a positive multiple of 8 */
  MODA_ERR_MODE = 6,        /* unknown mode / mode-argument mismatch */
  MODA_ERR_CHUNK = 7,       /* chunk_rows not a positive multiple of G */
  MODA_ERR_WORKSPACE = 8,   /* workspace NULL or too small */
  MODA_ERR_CUDA = 9,        /* a CUDA runtime / driver call failed (see moda_b200_last_cuda_error) */
  MODA_ERR_UNSUPPORTED = 10,/* requested kernel path cannot run this problem */
  MODA_ERR_TOO_LARGE = 11   /* problem exceeds a fixed capacity of the entry point */
} moda_status;

typedef enum moda_mode {
  MODA_CAUSAL = 0,        /* parallel_moda(is_causal=True)            moda_v14.py:2792 */
  MODA_NONCAUSAL = 1,     /* parallel_moda(is_causal=False)           moda_v14.py:2792 */
  MODA_CHUNK_VISIBLE = 2, /* parallel_moda_chunk_visible              moda_v16.py:3614 */
  MODA_DEPTH_ONLY = 3     /* parallel_fda (no sequence k/v)           fda_v12.py:1346  */
} moda_mode;

typedef enum moda_dtype { MODA_BF16 = 0, MODA_FP16 = 1 } moda_dtype;

/* Kernel path selector (moda_problem.path). */
typedef enum moda_path {
  MODA_PATH_AUTO = 0,    /* tcgen05 kernels where they apply (scale > 0), otherwise the mma.sync
                            kernels; the bandwidth kernels for MODA_DEPTH_ONLY and for the
                            own-position depth rows of MODA_CAUSAL / MODA_NONCAUSAL at G = 1
                            (whose partial result the attention kernel merges in its epilogue) */
  MODA_PATH_SIMT_MMA = 1,/* warp-level mma.sync kernels (every shape) */
  MODA_PATH_TCGEN05 = 2, /* tcgen05/TMEM/TMA kernels; MODA_ERR_UNSUPPORTED if they do not apply */
  /* As MODA_PATH_TCGEN05, with the forward kernel fixed instead of chosen by grid size: one
     128-row query tile per CTA (two CTAs per SM), or two query tiles per CTA (one CTA per SM).
     Both give bit-identical results; the values exist so that each can be tested on any shape. */
  MODA_PATH_TCGEN05_ONE_TILE = 3,
  MODA_PATH_TCGEN05_TWO_TILES = 4,
  /* As MODA_PATH_TCGEN05, with the backward over the sequence keys run as ONE key-stationary kernel
     that executes the five matmuls once each and sums dq in fixed point (D = 128 only; otherwise as
     MODA_PATH_TCGEN05).  The default is a query-parallel dq kernel plus a key-parallel dk/dv kernel
     (the reference's structure, seven executed matmuls), which measures no slower; the fused form
     needs more workspace (moda_b200_bwd_workspace_bytes accounts for the path). */
  MODA_PATH_TCGEN05_FUSED_BWD = 5
} moda_path;

typedef struct moda_tensor4 {
  void *data;        /* device pointer, 16-byte aligned                       */
  int64_t stride_b;  /* element strides; innermost (D) stride is 1            */
  int64_t stride_t;
  int64_t stride_h;
} moda_tensor4;

typedef struct moda_problem {
  int32_t B;          /* batch                                                     */
  int32_t T_kv;       /* base sequence length; T_q = T_kv * G                      */
  int32_t H;          /* KV heads (== q heads in the folded layout)                */
  int32_t D;          /* head dim of q/k and of v (64 or 128)                      */
  int32_t G;          /* moda_group_num                                            */
  int32_t L;          /* depth layers per position (0 = none)                      */
  int32_t mode;       /* moda_mode                                                 */
  int32_t chunk_rows; /* chunk-visible: query rows per chunk (the reference fixes
                         64: moda_v16.py:581-585); ignored otherwise              */
  int32_t dtype;      /* moda_dtype of q/k/v/depth/o/grads                         */
  int32_t path;       /* moda_path                                                 */
  float scale;        /* softmax scale (reference default D**-0.5)                 */
  int32_t device;     /* CUDA device ordinal the pointers live on                  */
  int32_t depth_rows_per_pos;     /* memory rows per position of depth_k/v and d_depth_k/v: 0 or L
                                     = packed [B, T_kv*L, H, D]; Lmax > L = in-place layer cache
                                     [B, T_kv, Lmax, H, D] of which the first L layers are valid   */
  int32_t accumulate_depth_grads; /* backward: non-zero adds d_depth_k/v to what the buffers hold
                                     (a gradient cache several layers share) instead of overwriting;
                                     each depth row has one owning thread block, so the result does
                                     not depend on scheduling                                       */
} moda_problem;

/*
 * Forward: o, lse = attention(q, k, v, depth_k, depth_v).
 * Replaces parallel_moda_fwd (moda_v14.py:381-522), parallel_moda_chunk_visible_fwd
 * (moda_v16.py:498-633) and parallel_fda_fwd (fda_v12.py:261-400).
 * k, v may be NULL only for MODA_DEPTH_ONLY; depth_k, depth_v NULL iff L == 0.
 */
int moda_b200_fwd(const moda_problem *prob, const moda_tensor4 *q, const moda_tensor4 *k,
                  const moda_tensor4 *v, const moda_tensor4 *depth_k,
                  const moda_tensor4 *depth_v, const moda_tensor4 *o, float *lse,
                  void *stream);

/*
 * Bytes of scratch moda_b200_bwd needs (delta [B,T_q,H] fp32, plus per-path extras).
 * Replaces the reference's internal torch.empty/torch.zeros scratch
 * (moda_v14.py:1609,1715-1716).
 */
int moda_b200_bwd_workspace_bytes(const moda_problem *prob, size_t *bytes);

/*
 * Backward: dq, dk, dv, d_depth_k, d_depth_v from (inputs, o, lse, dout).
 * Replaces parallel_moda_bwd (moda_v14.py:1470-1842), parallel_moda_chunk_visible_bwd
 * (moda_v16.py:2099-2343) and parallel_fda_bwd (fda_v12.py:881-1135).
 * `workspace` is caller-owned device scratch of at least
 * moda_b200_bwd_workspace_bytes() bytes, 256-byte aligned; contents are undefined
 * on entry and exit.  Gradients are fully overwritten (no pre-zeroing needed) and are
 * computed without atomics: two runs on the same inputs are bit-identical.
 */
int moda_b200_bwd(const moda_problem *prob, const moda_tensor4 *q, const moda_tensor4 *k,
                  const moda_tensor4 *v, const moda_tensor4 *depth_k,
                  const moda_tensor4 *depth_v, const moda_tensor4 *o, const float *lse,
                  const moda_tensor4 *dout, const moda_tensor4 *dq, const moda_tensor4 *dk,
                  const moda_tensor4 *dv, const moda_tensor4 *d_depth_k,
                  const moda_tensor4 *d_depth_v, void *workspace, size_t workspace_bytes,
                  void *stream);

/*
 * Backward for callers that cannot hand the library a scratch buffer.
 *
 * Some hosts of this operator have no way to allocate device memory at the point where
 * the backward runs: code replaying inside a region where cudaMalloc is forbidden or
 * would synchronise the device (a latency-critical serving loop, a plugin callback
 * that is only given its input and output buffers, a framework whose allocator is
 * locked while gradients are produced).  For them this entry point does exactly what
 * moda_b200_bwd does, but takes no workspace: the scratch (the per-row delta and, on
 * the tcgen05 path, the transposed lse/delta copies) lives in a fixed device array of
 * MODA_B200_STATIC_SCRATCH_BYTES that is part of the library image.  It calls no
 * cudaMalloc/cudaFree and no allocating library routine.
 *
 *  - Limit: problems whose moda_b200_bwd_workspace_bytes() exceeds
 *    MODA_B200_STATIC_SCRATCH_BYTES are refused with MODA_ERR_TOO_LARGE and nothing is
 *    launched.  Every GPU that loads the library holds the array until the process
 *    exits, which is why it is kept modest.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device made current) and caches it; make that
 *    first call outside any stream capture.  The cache covers device ordinals 0..63;
 *    a larger ordinal is refused with MODA_ERR_SHAPE.
 *  - All calls on a device share the one array and it keeps the previous call's
 *    contents.  The backward writes every scratch word before reading it, so nothing
 *    needs clearing between calls; but two calls whose kernels overlap on the GPU
 *    (different streams, no ordering between them) race on it.  Order such calls, or
 *    use moda_b200_bwd with separate workspaces.
 *
 * It has no counterpart in the reference, whose backward allocates its scratch with
 * torch (moda_v14.py:1609-1652,1715-1716).
 */
#define MODA_B200_STATIC_SCRATCH_BYTES (8u << 20)
int moda_b200_bwd_static_scratch(const moda_problem *prob, const moda_tensor4 *q,
                                 const moda_tensor4 *k, const moda_tensor4 *v,
                                 const moda_tensor4 *depth_k, const moda_tensor4 *depth_v,
                                 const moda_tensor4 *o, const float *lse,
                                 const moda_tensor4 *dout, const moda_tensor4 *dq,
                                 const moda_tensor4 *dk, const moda_tensor4 *dv,
                                 const moda_tensor4 *d_depth_k, const moda_tensor4 *d_depth_v,
                                 void *stream);

/*
 * In-place depth-KV cache: copies one layer's k and v ([B, T_kv, H, D], any supported strides)
 * into slot `layer` of the caches cache_k / cache_v, given as [B, T_kv*Lmax, H, D] tensors with
 * Lmax = prob->depth_rows_per_pos (row t*Lmax + layer).  Later layers pass the same cache
 * tensors as depth_k / depth_v with L = number of layers appended so far.  Replaces the reference
 * caller's rebuild of the depth cache before every layer (torch.stack + reshape + contiguous over
 * all earlier layers: vision_tasks/deit/models.py:361-375).  Uses B, T_kv, H, D, dtype, device
 * and depth_rows_per_pos of `prob`; 0 <= layer < Lmax.
 */
int moda_b200_depth_append(const moda_problem *prob, const moda_tensor4 *k, const moda_tensor4 *v,
                           const moda_tensor4 *cache_k, const moda_tensor4 *cache_v, int32_t layer,
                           void *stream);

/*
 * Validation only (no launch): the status moda_b200_fwd / moda_b200_bwd would return
 * for this problem's shape fields.  Mirrors the reference's shape assertions
 * (moda_v14.py:404-408,476-478,487,2839-2862).
 */
int moda_b200_check_problem(const moda_problem *prob);

/* Which kernel path MODA_PATH_AUTO resolves to for this problem's forward (is_bwd=0)
 * or backward (is_bwd=1): MODA_PATH_SIMT_MMA or MODA_PATH_TCGEN05; <0 on bad input. */
int moda_b200_resolve_path(const moda_problem *prob, int is_bwd);

/*
 * Per-kernel device timing.  Between profile_begin and profile_end every kernel this
 * library launches is bracketed by cudaEvents on its launch stream; profile_end waits
 * for them and returns, per kernel id that ran, its launch count and summed duration.
 * Replaces the reference's torch.cuda.Event timing loops (moda_v14.py:3054-3078), at
 * kernel granularity.  Not for use inside stream capture.
 */
int moda_b200_profile_begin(void);
int moda_b200_profile_end(int max_entries, int *n_entries, int *kernel_ids, int *launches,
                          float *total_ms);
const char *moda_b200_kernel_name(int kernel_id);

/*
 * Device-side status of the tcgen05 kernels.  Every wait inside those kernels (on an
 * mbarrier fed by TMA, by the tensor core or by other warps) is bounded; a wait that
 * expires records (1 << 8 | barrier id) in a status word, the CTA releases its TMEM and
 * returns, and the remaining CTAs of that launch return at once, leaving outputs
 * unwritten.  The word is sticky: launches never clear it, it keeps the FIRST failure
 * since it was last read, and this call returns it and resets it to 0.  A caller that
 * wants to know that its results are valid reads it at its next synchronisation point
 * (0 = every launch since the previous read ran to completion).  SYNCHRONISES the
 * device.  The reference has no counterpart (Triton kernels do not spin on barriers
 * they could miss).
 */
int moda_b200_device_status(int *status);

/*
 * Measurement aid (no reference counterpart): clocks per tcgen05.mma instruction (kind::f16, bf16,
 * M = 128, K = 16; issue of 64 back-to-back instructions to completion, one CTA) for the six
 * shapes the attention kernels are built from, written to clocks_per_mma[6] (DEVICE memory) in the
 * order SS N=64, SS N=128, SS N=256, TS N=64, TS N=128, TS N=256 (SS: A and B operands in shared
 * memory; TS: A in TMEM).  The nominal rate would be N/2 clocks.  bench.py turns these into the
 * tensor-pipe time a kernel's instruction mix needs per tile, which is the ceiling its measured
 * time is compared with.  A value of -1 means the bounded wait of the probe expired.  Asynchronous
 * on `stream`.
 */
int moda_b200_tensor_pipe_rates(int device, float *clocks_per_mma, void *stream);

/* Number of kernel launches the last successful call on this host thread issued. */
int moda_b200_last_launch_count(void);

/* cudaError_t value recorded by the last MODA_ERR_CUDA on this host thread. */
int moda_b200_last_cuda_error(void);

/* Static, human-readable name of a moda_status. */
const char *moda_b200_status_string(int status);

/* Library version: major*10000 + minor*100 + patch. */
int moda_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MODA_B200_H_ */
