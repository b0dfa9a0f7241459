// Host-side argument blocks and launch functions shared by the .cu files of
// this library.  Launch functions validate nothing: the C-ABI layer (api.cu)
// checks arguments before it fills these blocks.
#pragma once

#include "common.cuh"

namespace ezb {

// ------------------------------------------------------------------ GEMV ---
enum GemvPrologue : int {
    PRO_NONE = 0,         // x is used as given
    PRO_RMSNORM = 1,      // x <- bf16(x * rsqrt(mean(x^2)+eps) [* w])
    PRO_ADD_RMSNORM = 2,  // s = bf16(x + bf16(x_add)); CTA 0 stores s; x <- rmsnorm(s)
};
enum GemvEpilogue : int {
    EPI_STORE = 0,      // out = bf16(acc)
    EPI_RESIDUAL = 1,   // out = bf16(residual + bf16(acc))
    EPI_SWIGLU = 2,     // out = bf16(bf16(silu(bf16(acc_gate))) * bf16(acc_up))
    EPI_STORE_F32 = 3,  // out = acc (fp32)
    EPI_PUSH_F32 = 4,   // acc (fp32) stored into this rank's slot of an inbox on every rank (see TpLink)
};

struct GemvArgs {
    const bf16* W0 = nullptr;  // [N, ldw]: row n produces output n (gate rows when W1 is set)
    const bf16* W1 = nullptr;  // [N, ldw]: up rows (EPI_SWIGLU only)
    long long ldw = 0;
    int N = 0, K = 0, B = 0;
    const bf16* x = nullptr;  // [B, ldx]
    long long ldx = 0;
    const float* x_add = nullptr;  // PRO_ADD_RMSNORM: [B, ldadd] fp32
    long long ldadd = 0;
    bf16* x_sum_out = nullptr;  // PRO_ADD_RMSNORM: [B, ldsum] bf16
    long long ldsum = 0;
    const bf16* norm_w = nullptr;  // optional [K]
    float eps = 1e-6f;
    int prologue = PRO_NONE;
    int epilogue = EPI_STORE;
    const bf16* residual = nullptr;  // EPI_RESIDUAL: [B, ldres]
    long long ldres = 0;
    void* out = nullptr;  // [B, ldout] bf16 (fp32 for EPI_STORE_F32)
    long long ldout = 0;
    bf16* xn_scratch = nullptr;  // [B, K] bf16: needed when the prologue cannot be fused (see gemv_needs_scratch)
    PrefetchList next = {};  // what the following kernels stream first (optional)
    int trace_id = 0;  // label in timeline traces
    void* tc_workspace = nullptr;  // gemm_tc_workspace_bytes(): enables the tensor-core path for batch >= 2
    TpLink link = {0, 0, {}, {}, 0, -1, -1, -1};  // fused tensor-parallel exchange (small-batch kernel only)
};
bool gemv_small_batch_eligible(int B, int K);  // true when launch_gemv would run the small-batch kernel

// Tensor-core (tcgen05) path for batched projections, see gemm_tc.cu.
bool gemm_tc_supported(int B, int K);
bool gemm_tc_fits(int N, bool pair);  // tile count within the fixed ticket-counter region
size_t gemm_tc_workspace_bytes(int B, int N, bool pair);
cudaError_t launch_gemm_tc(const GemvArgs& a, const bf16* x, long long ldx, void* workspace, cudaStream_t stream);

// Prefetch descriptors for the operands of a following kernel.
PrefetchPlan prefetch_plan_rows(const bf16* W0, const bf16* W1, int N, int K, int cap_rows, int skip_rows = 0);  // a GEMV's weight rows
PrefetchPlan prefetch_plan_flat(const void* a, const void* b, size_t bytes_each);            // whole regions

// True when the activation block is too large to stay resident in shared memory
// next to the weight ring, so a prologue has to run as a kernel of its own
// writing to xn_scratch.
bool gemv_needs_scratch(int B, int K);
cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t stream);

// -------------------------------------------------------------- row prep ---
// s = x (+ bf16(add));  optionally store s;  y = rmsnorm(s) [* w] or y = s.
struct RowPrepArgs {
    const bf16* x = nullptr;
    long long ldx = 0;
    const float* add = nullptr;  // optional fp32 [rows, ldadd]
    long long ldadd = 0;
    bf16* sum_out = nullptr;  // optional
    long long ldsum = 0;
    const bf16* w = nullptr;  // optional
    bf16* y = nullptr;        // optional normalised output
    long long ldy = 0;
    int rows = 0, dim = 0;
    float eps = 1e-6f;
    int normalize = 1;
    TpLink link = {0, 0, {}, {}, 0, -1, -1, -1};  // gather_inbox >= 0: `add` is the sum of that inbox's slots
};
cudaError_t launch_row_prep(const RowPrepArgs& a, cudaStream_t stream);
// In-place sum over ranks of a local fp32 buffer of n elements (n % 4 == 0, n <= link.slot_elems) through inbox
// `which` of the ranks' communication buffers (tp_allreduce.cu).
cudaError_t launch_tp_allreduce(float* buf, const TpLink& link, int which, long long n, cudaStream_t stream);
// dst <- src, `bytes` a multiple of 16, both device-visible (device memory or the device alias of pinned host memory)
cudaError_t launch_pinned_copy(void* dst, const void* src, size_t bytes, bool to_host, cudaStream_t stream);
cudaError_t launch_rmsnorm_f32(const float* X, float* Out, int rows, int dim, float eps, cudaStream_t stream);

struct RopeArgs {
    const bf16 *q, *k, *v, *qw, *kw, *cos, *sin;
    bf16 *K_cache, *V_cache, *q_out, *k_out;
    int B, NQ, NKV, D, S, position;
    const int* positions;
    float eps;
};
cudaError_t launch_qk_norm_rope(const RopeArgs& a, cudaStream_t stream);

// ------------------------------------------------------------- attention ---
struct AttnArgs {
    const bf16* Q = nullptr;  // query for (b, h) at Q + b*q_bstride + h*D
    long long q_bstride = 0;
    const bf16* K = nullptr;  // [B, NKV, S, D] contiguous
    const bf16* V = nullptr;
    bf16* Out = nullptr;  // output for (b, h) at Out + b*o_bstride + h*D
    long long o_bstride = 0;
    const int* seq_lens = nullptr;
    int B = 0, H = 0, NKV = 0, S = 0, D = 0;
    void* workspace = nullptr;
    // decode-layer mode: q/k/v of the new token come from the fused projection
    // output qkv[b] = [q heads | k heads | v heads]; q and k get a unit-weight
    // RMSNorm over D; k and v are written to cache slot S-1 before it is read.
    int fuse_new_token = 0;
    const bf16* qkv = nullptr;
    long long qkv_bstride = 0;
    bf16* K_cache_w = nullptr;
    bf16* V_cache_w = nullptr;
    float eps = 1e-6f;
    // decode-layer mode, optional: weights of the q / k head norms ([D], null = unit) and the
    // rows of the rotary tables for the token's position ([D] each, HF layout with the halves
    // repeated; null = no rotation).  Norm, weight and rotation stay in fp32 with one
    // rounding at the end, as in the stand-alone q/k-norm + RoPE operator.
    const bf16* q_norm_w = nullptr;
    const bf16* k_norm_w = nullptr;
    const bf16* rope_cos = nullptr;
    const bf16* rope_sin = nullptr;
    // with seq_lens in decode-layer mode the new token of row b sits in slot seq_lens[b]-1 and only
    // seq_lens[b] keys are attended; rope_by_len = 1 then makes rope_cos / rope_sin table bases
    // ([>= S, D]) indexed by that slot
    int rope_by_len = 0;
    // paged caches: K / V (and K_cache_w / V_cache_w) are page pools [pages, NKV, P, D], page_table is
    // [B, max_pages] int32 on the device, P = 1 << page_shift >= 64, S = max_pages * P
    const int* page_table = nullptr;
    int page_shift = 0;
    int max_pages = 0;
    int num_pages = 0;  // pages in each pool
    PrefetchList next = {};
};
size_t attn_workspace_bytes(int B, int H, int NKV, int S, int D);
size_t attn_counters_bytes(int B, int H, int NKV);  // leading part of the workspace that must be zero before a call
int attn_chunk_keys(int B, int NKV, int S, bool ragged, int D = 128);  // keys per KV split chosen for this shape
cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t stream);

// ------------------------------------------------- whole layer, batch 1 ---
// The decode layer at batch 1 as one persistent kernel (decode_mega.cu).  `qkv`, `attn_out`, `x2`, `h` are the
// activation rows of the layer workspace; `mega_workspace` (decode_mega_workspace_bytes(), zero before first use)
// holds the grid-barrier counters and the attention slices' records.
struct MegaArgs {
    const bf16* hidden = nullptr;
    bf16* out = nullptr;
    bf16* Kc = nullptr;  // [1, NKV, S, D] contiguous; slot S-1 receives the new token
    bf16* Vc = nullptr;
    const bf16 *Wqkv = nullptr, *Wo = nullptr, *Wgu = nullptr, *Wd = nullptr;
    const bf16 *input_norm_w = nullptr, *post_norm_w = nullptr, *q_norm_w = nullptr, *k_norm_w = nullptr;
    const bf16 *rope_cos = nullptr, *rope_sin = nullptr;  // rows of the rotary tables for the token's position
    bf16 *qkv = nullptr, *attn_out = nullptr, *x2 = nullptr, *h = nullptr;
    void* mega_workspace = nullptr;
    int S = 0, H = 0, I = 0, NH = 0, NKV = 0, D = 0;
    float eps = 1e-6f;
    // tensor parallel (world > 0): the pointers above are this rank's shards, NH / NKV / I the local sizes; the partial
    // sums of o_proj and down are exchanged inside the kernel through the communication buffers of the link
    TpLink link = {0, 0, {}, {}, 0, -1, -1, -1};
};
bool decode_mega_supported(const MegaArgs& a);  // shape inside what the kernel covers on the current device (and switched on)
size_t decode_mega_workspace_bytes(int NKV, int D);
cudaError_t launch_decode_mega(const MegaArgs& a, cudaStream_t stream);

// STREAM-style calibration kernels (hbm_stream.cu): op 0 read b, 1 write a, 2 copy b->a, 3 triad a = b + s*c.
cudaError_t launch_hbm_stream(int op, const void* b, const void* c, void* a, long long n_vec4, float s, int block,
                              int blocks_per_sm, float* sink, cudaStream_t stream);

// The reference's teaching operators (tutorial_ops.cu).
cudaError_t launch_vector_add_f32(const float* A, const float* B, float* C, long long n, cudaStream_t stream);
cudaError_t launch_softmax_f32(const float* X, float* Out, int rows, int dim, cudaStream_t stream);
// Two chained fp32 GEMMs y = x . W1, z = y . W2 (pdl_gemm.cu); use_pdl: the second may start while the first drains.
cudaError_t launch_pdl_gemm_f32(const float* x, const float* W1, const float* W2, float* y, float* z, int M, int K, int N, int P,
                                bool use_pdl, cudaStream_t stream);
size_t reduce_workspace_bytes();  // zero-filled once by the caller
cudaError_t launch_reduce_sum_f32(const float* A, float* Out, long long n, void* workspace, cudaStream_t stream);

}  // namespace ezb

