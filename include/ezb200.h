/*
 * ezb200 -- C ABI of the B200 (sm_100a) kernels for the Qwen3 dense-decode
 * path of ez-ops.  One entry point per operator of that path; each comment
 * names the reference interface the entry point stands in for (file:line,
 * paths relative to the ez-ops project root).
 *
 * Conventions
 *   - All pointers are device pointers unless the name ends in _host.
 *   - "bf16" buffers are passed as void* / const void* (2 bytes per element).
 *   - The library never allocates or frees device memory.  Operators that need
 *     scratch take a workspace pointer and size; the matching
 *     *_workspace_bytes() query gives the size.  A workspace must be zero-filled
 *     once before its first use; every call leaves it ready for the next one.
 *     One workspace serves one stream at a time.
 *   - Work is enqueued on `stream` and the call returns without synchronising,
 *     so calls can be captured into a CUDA graph.  The kernels of one call are
 *     chained with programmatic dependent launch: a kernel may start while its
 *     predecessor drains and request WEIGHT tiles early, but reads activations
 *     and the KV cache only after the predecessor has finished.  The first kernel
 *     of a call is ordered against earlier work on the stream in the usual way,
 *     unless EZB_TUNE_PDL_ACROSS_CALLS is set; set it only when the weight
 *     tensors are not written by work enqueued shortly before the call (a decode
 *     loop over resident weights), since early weight requests then overlap the
 *     tail of the previous call.
 *   - Return value: EZB_OK or a negative EZB_ERR_* code.  ezb_strerror() names
 *     the code, ezb_last_error_message() gives the detail of the last failure
 *     on the calling thread.  Arguments are validated before anything is
 *     launched; a rejected call has no effect.
 *   - Device-side waits are bounded.  A kernel that gives up on a wait records
 *     a code in a per-device status word, finishes without hanging, and leaves
 *     its outputs unspecified; ezb_device_status() reads the word.
 */
#ifndef EZB200_H
#define EZB200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ezb_stream_t; /* same type as cudaStream_t */

#define EZB_OK 0
#define EZB_ERR_INVALID_ARGUMENT (-1) /* null / misaligned pointer, non-positive size */
#define EZB_ERR_UNSUPPORTED_SHAPE (-2) /* shape outside what the kernels cover          */
#define EZB_ERR_CUDA (-3)              /* a CUDA runtime call failed                    */
#define EZB_ERR_WORKSPACE (-4)         /* workspace missing or too small                */
#define EZB_ERR_DEVICE_FAULT (-5)      /* ezb_device_status() found a recorded fault    */

/* Tuning knobs for ezb_set_tuning / ezb_get_tuning (process-wide, read at launch). */
#define EZB_TUNE_PDL 0              /* 1: chain kernels with programmatic dependent launch (default 1) */
#define EZB_TUNE_GEMV_SMEM_KB 1     /* shared-memory budget per CTA of the weight-streaming kernel      */
#define EZB_TUNE_GEMV_PREFETCH 2    /* weight stages requested before the dependency wait (0 = all; default 1) */
#define EZB_TUNE_GEMV_CTAS_PER_SM 3 /* persistent CTAs per SM of the weight-streaming kernel            */
#define EZB_TUNE_ATTN_MIN_CHUNK 4   /* smallest KV split, in keys (multiple of 64)                      */
#define EZB_TUNE_ATTN_WAVES 5       /* target number of KV splits per SM                                */
#define EZB_TUNE_GEMV_KC 6          /* k-chunk length of a weight stage (0 = automatic)                 */
#define EZB_TUNE_GEMV_ROWS8 7       /* 1: batch <= 8 uses the whole-row small-batch kernel (default 1)   */
#define EZB_TUNE_PDL_ACROSS_CALLS 8 /* 1: the first kernel of a call may also start early (default 0)    */
#define EZB_TUNE_L2_PREFETCH 9      /* 1: kernels of a chain pull the next kernel's first weights into L2 (default 1) */
#define EZB_TUNE_L2_PREFETCH_KB 10  /* KB per CTA of a following large weight pulled ahead (default 192)                 */
#define EZB_TUNE_GEMV_WINDOW 11     /* stages that may be requested but not landed, small-batch kernel (0 = ring depth) */
#define EZB_TUNE_L2_PREFETCH_ATTN_KB 12 /* KB per CTA of the gate/up weights that the attention kernel pulls ahead (default 0) */
#define EZB_TUNE_TC 13              /* 1: batched projections run on tcgen05 tensor cores (default 1)                   */
#define EZB_TUNE_ATTN_WAVES_UNIFORM 14 /* rows of equal length: 0 (default) = as many splits as fit in one resident wave; n > 0 = as ATTN_WAVES */
#define EZB_TUNE_TP_POLL_ALL 15       /* fused exchange prologue: 0 = by world size (all ranks at once when > 2), 1 = always, 2 = never */
#define EZB_TUNE_TP_PULL 16           /* fused exchange direction: 0 = push (default), 1 = pull (consumers read the peers' buffers) */
#define EZB_TUNE_MEGA 17              /* 1: the batch-1 decode layer runs as one persistent kernel when the shape allows (default 1) */
#define EZB_TUNE_MEGA_L2_STAGES 18    /* single-kernel layer: stages a producer with a full ring may pull into L2 ahead (default 0) */
#define EZB_TUNE_WAIT_LIMIT_MS 19     /* budget of one device-side wait in the single-kernel layer and the cross-rank waits, ms at 2 GHz (default 1000) */
#define EZB_TUNE_MEGA_STAGES 20       /* single-kernel layer: cap on the ring depth (0 = as many as fit)                            */
#define EZB_TUNE_MEGA_INFLIGHT 21     /* single-kernel layer: stages that may be requested but not yet landed (0 = whole ring; default 2) */
#define EZB_TUNE_MEGA_GATE 22         /* single-kernel layer, bit mask: a producer stops 1 = behind its K/V stages until the QKV barrier is passed (default), 2 = behind Wo until the barrier after o_proj, 4 = behind gate/up until the barrier after it */
#define EZB_TUNE_TP_WAIT_LIMIT_MS 23   /* fused exchange: budget of one wait for the peers' partial sums, ms at 2 GHz (default 5000)      */
#define EZB_TUNE_TP_STRONG_STORES 24   /* fused exchange: 1 = publish cells with st.relaxed.sys instead of plain stores (default 0) */
#define EZB_TUNE_STREAM_EVICT_FIRST 25 /* weight streams carry the L2 evict-first policy: 0 = off, 1 = weights (default), 2 = also K/V in the single-kernel layer */
#define EZB_TUNE_COUNT 26

int ezb_version(void);
const char* ezb_strerror(int code);
const char* ezb_last_error_message(void);
int ezb_set_tuning(int key, int value);
int ezb_get_tuning(int key);

/* Reads (and with clear != 0 resets) the status word of the current device.
 * Synchronises the device.  *status_out == 0 means no kernel gave up a wait. */
int ezb_device_status(unsigned int* status_out_host, int clear);

/* Timeline tracing for performance work (no counterpart in the reference; its
 * tracing is an ncu wrapper, scripts/ncu_profile.py).  After this call, one
 * thread per CTA of the streaming and attention kernels appends a record of six
 * 64-bit words {kernel id, block, t_entry, t_after_dependency, t_first_data,
 * t_exit} (GPU nanoseconds) at records[6 * atomicAdd(cursor, 1)], while fewer
 * than `capacity` records exist.  Both buffers are device memory owned by the
 * caller; pass nulls to switch tracing off.  Not for use during timed runs. */
int ezb_trace_enable(void* records, unsigned int* cursor, unsigned int capacity);

/* y[N] = W[N,K] . x[K], bf16 in, fp32 accumulate, bf16 out.
 * Replaces the host entries gemv_cu(A,B,C) (ezops/kernels/gemv/gemv_cu.cu:71)
 * and gemv_ws_cu(A,B,C) (ezops/kernels/gemv/gemv_ws_cu.cu:211) behind
 * GemvOp.forward (ezops/ops/gemv.py:26-27).  K % 16 == 0. */
int ezb_gemv_bf16(const void* x, const void* W, void* y, int N, int K, ezb_stream_t stream);

/* Batched form of the same kernel: Y[b, :] = W[N,K] . X[b, :] for b < B <= 64,
 * X [B,K], Y [B,N]; the weight is still streamed once for the whole batch.
 * (The reference op is batch 1 only; its fused ops hold the batched
 * projections, e.g. ezops/ops/qwen3_dense_decode.py:157.)  For B >= 2 the
 * workspace of ezb_gemv_workspace_bytes() is required (zero-filled once): larger
 * batches run on the tensor cores with a split over K that parks partial tiles
 * there. */
size_t ezb_gemv_workspace_bytes(int B, int N, int K);
int ezb_gemv_batched_bf16(const void* X, const void* W, void* Y, void* workspace, size_t workspace_bytes, int B, int N,
                          int K, ezb_stream_t stream);

/* Out = X * rsqrt(mean(X^2) + eps), fp32 rows, no weight.
 * Replaces rmsnorm_cu(X,Out,eps) (ezops/kernels/rmsnorm/rmsnorm_cu.cu:51)
 * behind RmsNormOp.forward (ezops/ops/rmsnorm.py:26-27). */
int ezb_rmsnorm_f32(const float* X, float* Out, int rows, int dim, float eps, ezb_stream_t stream);

/* bf16 rows with optional bf16 weight (null = unit weight): fp32 statistics,
 * (x * rsqrt(var+eps) * w) in fp32, one rounding.  The norm that the reference
 * has only inside its fused ops (ezops/ops/fused_o_proj_ffn.py:107-110,
 * ezops/ops/qwen3_dense_decode.py:137-140), exposed as an operator. dim % 8 == 0. */
int ezb_rmsnorm_bf16(const void* X, const void* w_or_null, void* Out, int rows, int dim, float eps,
                     ezb_stream_t stream);

/* Per-head RMSNorm(w) + rotate-half RoPE of q and k, and the KV-cache write
 * K_cache[b,:,pos]=k_out, V_cache[b,:,pos]=v.  Replaces the kernel objects
 * behind FusedQkNormRopeOp.forward (ezops/ops/fused_qk_norm_rope.py:95-107;
 * the reference has Triton/TileLang backends only,
 * ezops/kernels/fused_qk_norm_rope/fused_qk_norm_rope_triton.py:53-102).
 * q,q_out [B,NQ,D]; k,v,k_out [B,NKV,D]; qw,kw [D]; cos,sin [S,D];
 * K_cache,V_cache [B,NKV,S,D].  positions_or_null: int32[B] device array with
 * one slot per batch row; when null every row uses `position`.  D is a power of
 * two in [8, 512]. */
int ezb_qk_norm_rope(const void* q, const void* k, const void* v, const void* qw, const void* kw, const void* cos,
                     const void* sin, void* K_cache, void* V_cache, void* q_out, void* k_out, int B, int NQ, int NKV,
                     int D, int S, int position, const int* positions_or_null, float eps, ezb_stream_t stream);

/* Single-query GQA attention, split over the KV length with a log-sum-exp
 * combine.  Replaces attn_decode_cu(Q,K,V,Out)
 * (ezops/kernels/attn_decode/attn_decode_cu.cu:140, MHA only) and the
 * flash_decode_tilelang_gqa* kernels (ezops/kernels/attn_decode/attn_decode_tl.py:25-657)
 * behind AttnDecodeOp.forward (ezops/ops/attn_decode.py:55-56).
 * Q,Out [B,H,1,D]; K,V [B,NKV,S,D]; seq_lens_or_null int32[B] (1 <= len <= S).
 * D in {64, 128}; H % NKV == 0. */
size_t ezb_attn_decode_workspace_bytes(int B, int H, int NKV, int S, int D);
int ezb_attn_decode(const void* Q, const void* K, const void* V, void* Out, void* workspace, size_t workspace_bytes,
                    int B, int H, int NKV, int S, int D, const int* seq_lens_or_null, ezb_stream_t stream);

/* The same attention for callers that cannot allocate device memory (a plugin
 * inside a framework that owns the device heap and passes only inputs and
 * outputs; a serving loop that must never hit cudaMalloc's device sync).  It has
 * no counterpart in the reference.  The scratch lives in a fixed array of
 * EZB_ATTN_STATIC_SCRATCH_BYTES inside the library (held by every GPU that
 * loads it, until exit); larger shapes are refused with EZB_ERR_WORKSPACE.
 * Nothing is allocated or freed.  The first call on a device resolves the
 * array's address and should happen outside stream capture.  All calls on a
 * device share the array (its zero-initialised part is cleared on `stream`
 * before every launch), so calls that may overlap on the GPU must be
 * serialised by the caller. */
#define EZB_ATTN_STATIC_SCRATCH_BYTES (8u << 20)
int ezb_attn_decode_static(const void* Q, const void* K, const void* V, void* Out, int B, int H, int NKV, int S, int D,
                           const int* seq_lens_or_null, ezb_stream_t stream);

/* x2 = residual + attn Wo^T ; out = x2 + (silu(xn Wg^T) * (xn Wu^T)) Wd^T with
 * xn = rmsnorm(x2) * post_norm_w.  Replaces the kernel objects behind
 * FusedOProjFfnOp.forward (ezops/ops/fused_o_proj_ffn.py:84-94; reference
 * backends ezops/kernels/fused_o_proj_ffn/fused_o_proj_ffn_triton.py:31-231).
 * attn [B,Q]; residual,out [B,H]; Wo [H,Q]; post_norm_w [H]; Wg,Wu [I,H];
 * Wd [H,I].  Q, H, I multiples of 16; B in [1, 64]. */
size_t ezb_o_proj_ffn_workspace_bytes(int B, int H, int I, int Q);
int ezb_o_proj_ffn(const void* attn, const void* residual, const void* Wo, const void* post_norm_w, const void* Wg,
                   const void* Wu, const void* Wd, void* out, void* workspace, size_t workspace_bytes, int B, int H,
                   int I, int Q, float eps, ezb_stream_t stream);

/* One decode step of a Qwen3 dense layer (no RoPE, unit-weight norms), new
 * k / v written to cache slot S-1.  Replaces the kernel objects behind
 * Qwen3DenseDecodeOp.forward (ezops/ops/qwen3_dense_decode.py:110-120;
 * reference backends under ezops/kernels/qwen3_dense_decode/).
 * hidden,out [B,H]; K_cache,V_cache [B,NKV,S,D]; Wqkv [(NH+2NKV)D,H];
 * Wo [H,NH*D]; Wgu [2I,H] (gate rows then up rows); Wd [H,I].
 * D in {64,128}; NH/NKV <= 16; H, I multiples of 16; B in [1, 64]. */
size_t ezb_qwen3_decode_layer_workspace_bytes(int B, int S, int H, int I, int NH, int NKV, int D);
int ezb_qwen3_decode_layer(const void* hidden, void* K_cache, void* V_cache, const void* Wqkv, const void* Wo,
                           const void* Wgu, const void* Wd, void* out, void* workspace, size_t workspace_bytes, int B,
                           int S, int H, int I, int NH, int NKV, int D, float eps, ezb_stream_t stream);

/* Tensor-parallel form of the same layer for one rank holding NH_local query
 * heads, NKV_local kv heads and I_local FFN columns (no counterpart in the
 * reference, which is single-GPU; the split follows the usual row/column
 * scheme: Wqkv_local [(NH_local+2NKV_local)D,H], Wo_local [H,NH_local*D],
 * Wgu_local [2*I_local,H], Wd_local [H,I_local]).  The layer is cut at its two
 * exchange points; the caller sums the fp32 partials over ranks in between
 * (NCCL all-reduce):
 *   part 1: rmsnorm, QKV, attention, o_proj         -> partial_o   [B,H] fp32
 *   part 2: x2 = hidden + sum(partial_o), rmsnorm, gate/up, SwiGLU, down
 *                                                   -> x2 [B,H] bf16, partial_d [B,H] fp32
 *   part 3: out = x2 + sum(partial_d)               -> out [B,H] bf16
 * Part 1 takes a workspace of ezb_qwen3_decode_layer_workspace_bytes() for the
 * local sizes; part 2 takes a separate one of
 * ezb_o_proj_ffn_workspace_bytes(B, H, I_local, 16).  Neither may be shared
 * with the other part. */
int ezb_qwen3_decode_layer_tp_attn(const void* hidden, void* K_cache, void* V_cache, const void* Wqkv_local,
                                   const void* Wo_local, float* partial_o, void* workspace, size_t workspace_bytes,
                                   int B, int S, int H, int NH_local, int NKV_local, int D, float eps,
                                   ezb_stream_t stream);
int ezb_qwen3_decode_layer_tp_ffn(const void* hidden, const float* summed_o, const void* Wgu_local,
                                  const void* Wd_local, void* x2, float* partial_d, void* workspace,
                                  size_t workspace_bytes, int B, int H, int I_local, float eps, ezb_stream_t stream);
int ezb_residual_add_f32(const void* x2, const float* summed_d, void* out, int B, int H, ezb_stream_t stream);

/* A stack of decode layers in one call, with what a model has and the
 * reference's layer operator leaves out (ezops/ops/qwen3_dense_decode.py:27-29:
 * "RoPE excluded by design", unit norm weights): per-layer norm weights and the
 * rotary embedding of the new token's q and k, applied exactly as the
 * stand-alone operator does (ezops/ops/fused_qk_norm_rope.py:149-169: norm,
 * weight and rotate-half in fp32, one bf16 rounding) inside the attention
 * kernel.  This is the multi-layer decode loop the reference lists as not yet
 * implemented (README.md:16).  Layer l reads layer l-1's output from a
 * ping-pong buffer in the workspace; all kernels of all layers form one
 * programmatic-dependent-launch chain, and the last kernel of a layer starts
 * pulling the next layer's Wqkv into L2.  Any of the four norm-weight pointers
 * may be NULL (unit weight); rope_cos / rope_sin are [>= rope_position + 1, D]
 * bf16 tables in the reference's layout (halves repeated) or both NULL (no
 * rotation).  As in the layer operator every cache has S slots and the new
 * token goes to slot S - 1 - unless seq_lens (device, [B] int32, each 1..S) is
 * given: then row b's token goes to slot seq_lens[b] - 1, attends to its
 * first seq_lens[b] keys and is rotated with the table row of that slot
 * (rope_position is ignored; the tables must have S rows).  That is the
 * per-row position a serving loop with sequences of different lengths needs.
 * `layers` is a host array, read during the call. */
typedef struct ezb_layer_t {
    void* K_cache;
    void* V_cache;
    const void* Wqkv;
    const void* Wo;
    const void* Wgu;
    const void* Wd;
    const void* input_norm_w; /* [H] */
    const void* post_norm_w;  /* [H] */
    const void* q_norm_w;     /* [D] */
    const void* k_norm_w;     /* [D] */
} ezb_layer_t;
size_t ezb_qwen3_decode_stack_workspace_bytes(int B, int S, int H, int I, int NH, int NKV, int D);
int ezb_qwen3_decode_stack(const void* hidden, void* out, const ezb_layer_t* layers, int n_layers, const void* rope_cos,
                           const void* rope_sin, int rope_position, const int* seq_lens, void* workspace,
                           size_t workspace_bytes, int B, int S, int H, int I, int NH, int NKV, int D, float eps,
                           ezb_stream_t stream);

/* The reference's three teaching operators, for API completeness.
 * C = A + B over n fp32 elements (ezops/ops/vector_add.py:19-30;
 * kernels/vector_add/vector_add_cu.cu).  Softmax over the last dimension of an
 * fp32 [rows, dim] matrix (ezops/ops/softmax.py:24-36): one CTA per row, the
 * row staged in shared memory when dim <= 12288.  Sum of n fp32 elements into
 * Out[0] (ezops/ops/reduce.py:23-33): per-CTA partial sums, added in CTA order
 * by the last CTA to finish, so two calls give the same bits; the workspace
 * (ezb_reduce_workspace_bytes(), zero-filled once) holds the partials. */
int ezb_vector_add_f32(const float* A, const float* B, float* C, long long n, ezb_stream_t stream);

/* Host buffers at the boundary.  The reference's operators take the step's tensors where the caller has them
 * (ezops/ops/base.py forward(*args)); a host application holds a decode step's input and result in host memory.
 * ezb_copy_pinned moves `bytes` (a positive multiple of 16, both pointers 16-byte aligned) between PINNED host
 * memory and device memory - either direction, or device to device - with a small kernel instead of a copy engine,
 * so that {copy in, ezb_qwen3_decode_layer, copy out} on one stream is one programmatic-dependent-launch chain (and
 * one CUDA graph without engine hand-overs): the layer streams its weights while the input crosses PCIe.  Pageable
 * host memory is refused with EZB_ERR_INVALID_ARGUMENT (it has no device address).  The host may read a copied-out
 * buffer after synchronising the stream.  No counterpart in the reference (its benchmarks keep tensors on the GPU). */
int ezb_copy_pinned(void* dst, const void* src, size_t bytes, ezb_stream_t stream);
int ezb_softmax_f32(const float* X, float* Out, int rows, int dim, ezb_stream_t stream);
size_t ezb_reduce_workspace_bytes(void);
int ezb_reduce_sum_f32(const float* A, float* Out, long long n, void* workspace, size_t workspace_bytes, ezb_stream_t stream);

/* Two chained fp32 GEMMs, y[M,N] = x[M,K] . W1[K,N] and z[M,P] = y . W2[N,P] (row-major, TF32 tensor-core
 * arithmetic with fp32 accumulation), the reference's demonstration of programmatic dependent launch.  Replaces
 * pdl_gemm_baseline_cu (use_pdl = 0; ezops/kernels/pdl_gemm/pdl_gemm_cu.cu:163-196) and pdl_gemm_pdl_cu (use_pdl = 1;
 * :202-248) behind PdlGemmOp.forward (ezops/ops/pdl_gemm.py:49-57).  With use_pdl the second GEMM is launched with
 * the programmatic-serialization attribute: its CTAs request their W2 tiles while the first GEMM drains and read y
 * only after it has finished.  Both settings give the same bits.  K, N, P divisible by 4. */
int ezb_pdl_gemm_f32(const float* x, const float* W1, const float* W2, float* y, float* z, int M, int K, int N, int P, int use_pdl,
                     ezb_stream_t stream);

/* Kernel launches issued by the library in this process so far (every kernel of
 * the library goes through one launch helper).  A diagnostic with no
 * counterpart in the reference: benchmarks report launches per step from it
 * instead of a hand-kept constant. */
unsigned long long ezb_launch_count(void);

/* Paged KV caches (the format a serving stack hands over; the reference's caches
 * are contiguous [B, NKV, S, D], ezops/ops/attn_decode.py:52-56): K and V live
 * in page pools [pages, NKV, page_size, D]; page_table [B, max_pages] (device
 * int32) names the pool page of every page_size keys of a row, seq_lens [B]
 * the valid lengths.  page_size is a power of two >= 64, so a 64-key tile of
 * the kernel never straddles pages and paging costs one table lookup per tile.
 * Workspace as for S = max_pages * page_size.  The stack form takes the pools
 * through ezb_layer_t.K_cache / V_cache (one pool pair per layer, one page
 * table for all layers); the new token of row b goes to the page slot of
 * position seq_lens[b] - 1, which the caller has mapped.  num_pages is the
 * number of pages in each pool: a table entry outside [0, num_pages) inside a
 * row's valid length (a stale id, or -1 for "unallocated") is never
 * dereferenced - the kernel zero-fills that tile, skips the cache write,
 * records fault 0x302 in the status word (ezb_device_status) and carries on. */
int ezb_attn_decode_paged(const void* Q, const void* K_pool, const void* V_pool, const int* page_table, void* Out,
                          void* workspace, size_t workspace_bytes, int B, int H, int NKV, int max_pages, int page_size, int D,
                          int num_pages, const int* seq_lens, ezb_stream_t stream);
int ezb_qwen3_decode_stack_paged(const void* hidden, void* out, const ezb_layer_t* layers, int n_layers, const void* rope_cos,
                                 const void* rope_sin, const int* seq_lens, const int* page_table, int page_size,
                                 int max_pages, int num_pages, void* workspace, size_t workspace_bytes, int B, int H, int I,
                                 int NH, int NKV, int D, float eps, ezb_stream_t stream);

/* The stack of layers, tensor parallel with the exchange fused into the kernels:
 * ezb_qwen3_decode_stack on this rank's shards (as ezb_qwen3_decode_layer_tp_fused
 * takes them), one call for all layers.  A layer's second sum is folded into
 * the next layer's QKV prologue, so a layer costs five launches and only the
 * last one ends with the small kernel that adds the final sum.  Same rules for
 * the communication buffers; no counterpart in the reference. */
size_t ezb_qwen3_decode_stack_tp_fused_workspace_bytes(int B, int S, int H, int I_local, int NH_local, int NKV_local, int D);
int ezb_qwen3_decode_stack_tp_fused(const void* hidden, void* out, const ezb_layer_t* layers_local, int n_layers,
                                    const void* rope_cos, const void* rope_sin, int rope_position, const int* seq_lens,
                                    void* workspace, size_t workspace_bytes, void* const* comm_bases_host, int world, int rank,
                                    int B, int S, int H, int I_local, int NH_local, int NKV_local, int D, float eps,
                                    ezb_stream_t stream);

/* Bandwidth calibration for the roofline profile of a GPU: one pass of a
 * STREAM-style kernel over n_vec4 128-bit elements; op 0 reads b, 1 writes a, 2
 * copies b to a, 3 is the triad a = b + scalar*c.  Replaces the stand-alone
 * calibrator the reference compiles at run time
 * (benchmarks/hardware/memory/hbm_saturation.cu:49-93, driven by
 * benchmarks/hardware/memory/hbm_bandwidth.py:52-75); the caller times it
 * with events.  Grid = blocks_per_sm x SM count, block_size threads. */
int ezb_hbm_stream(int op, const void* b, const void* c, void* a, long long n_vec4, float scalar, int block_size,
                   int blocks_per_sm, ezb_stream_t stream);

/* The same tensor-parallel layer as ONE call with the two sums over ranks done
 * inside the kernels, over peer memory instead of NCCL (no counterpart in the
 * reference).  Every rank owns a communication buffer of ezb_tp_comm_bytes(B, H)
 * (ezb_tp_comm_alloc zero-fills it; this is the one place where the library
 * allocates, at set-up time) and maps the buffers of all ranks (ezb_ipc_export /
 * ezb_ipc_open, one process per GPU on one node); comm_bases_host[r] is rank r's
 * buffer as seen from this process.  o_proj and down_proj store every fp32
 * output of their partial [B,H], tagged with an epoch in the same 64-bit word,
 * into the caller's slot of an inbox on every rank; the consuming kernel polls
 * its own inbox (bounded, about one second, then records a device fault) until
 * every word carries the expected epoch and adds the slots in rank order, so
 * all ranks get identical bits.  Ranks must make the same sequence of calls; a
 * buffer serves one stream.  Up to batch 8 the gather and the push live in the
 * resident-activation kernel; for larger batches the row kernel in front of a
 * projection gathers and the tensor-core kernel's epilogue pushes.  Shapes that
 * neither covers return EZB_ERR_UNSUPPORTED_SHAPE (use the three-part form with
 * NCCL then). */
size_t ezb_tp_comm_bytes(int B, int H);

/* The sum over ranks between the three local parts as a kernel of this library instead of an NCCL all-reduce (no
 * counterpart in the reference): buf (device, fp32 [B, H], 16-byte aligned) is summed IN PLACE over the ranks, in
 * rank order, identical bits on every rank.  Uses the communication buffers of the fused exchange (same
 * ezb_tp_comm_bytes(B, H), same mapping) and its epoch-tagged cells: two-shot (every rank sums the slice of elements
 * it owns and hands the result to the others), 64 CTAs, plain peer stores, polls of local memory only, no flag and no
 * fence.  Every rank calls it on its stream behind the part that wrote the partial; when the kernel has finished,
 * buf holds the sum.  Ranks must make the same sequence of calls and alternate `which` (0: the sum after o_proj, 1:
 * the sum after down); B * H a multiple of 4; waits are bounded (EZB_TUNE_TP_WAIT_LIMIT_MS, then fault 0x201).
 * A communication buffer serves EITHER this entry point OR the fused entry points above, never both: the two keep
 * separate epoch counters, and a cell left by one could carry the tag the other waits for. */
int ezb_tp_allreduce_f32(void* buf, void* const* comm_bases_host, int world, int rank, int which, int B, int H,
                         ezb_stream_t stream);
int ezb_tp_comm_alloc(size_t bytes, void** out_host);
int ezb_tp_comm_free(void* buffer);
int ezb_ipc_export(void* buffer, void* handle64_host);
int ezb_ipc_open(const void* handle64_host, void** out_host);
int ezb_ipc_close(void* mapped);
int ezb_qwen3_decode_layer_tp_fused(const void* hidden, void* K_cache, void* V_cache, const void* Wqkv_local,
                                    const void* Wo_local, const void* Wgu_local, const void* Wd_local, void* out,
                                    void* workspace, size_t workspace_bytes, void* const* comm_bases_host, int world,
                                    int rank, int B, int S, int H, int I_local, int NH_local, int NKV_local, int D,
                                    float eps, ezb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* EZB200_H */
