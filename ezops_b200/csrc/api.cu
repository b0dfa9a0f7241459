// The C ABI of the library (declared in include/ezb200.h): argument checks,
// workspace carving and the kernel chains of the fused operators.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "launchers.h"

namespace ezb {

__device__ unsigned int g_status_word = 0;

static thread_local char t_message[256] = "";

void set_last_message(const char* msg) {
    std::snprintf(t_message, sizeof(t_message), "%s", msg ? msg : "");
}
void set_last_cuda_error(cudaError_t e) {
    std::snprintf(t_message, sizeof(t_message), "CUDA error %d: %s", (int)e, cudaGetErrorString(e));
}

static constexpr int kMaxDevices = 64;

static int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    return dev;
}

int sm_count() {
    static std::atomic<int> cache[kMaxDevices];
    const int dev = current_device();
    int v = cache[dev].load();
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cache[dev].store(v);
    }
    return v;
}

int max_smem_optin() {
    static std::atomic<int> cache[kMaxDevices];
    const int dev = current_device();
    int v = cache[dev].load();
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess || v <= 0) v = 232448;
        cache[dev].store(v);
    }
    return v;
}

unsigned int* status_ptr() {
    static std::atomic<unsigned int*> cache[kMaxDevices];
    const int dev = current_device();
    unsigned int* p = cache[dev].load();
    if (!p) {
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_status_word) != cudaSuccess) return nullptr;
        p = static_cast<unsigned int*>(addr);
        cache[dev].store(p);
    }
    return p;
}

// Timeline tracing: buffers are supplied by the caller (ezb_trace_enable), one set per process.
static Trace g_trace = {nullptr, nullptr, 0};
Trace trace_handle() { return g_trace; }

static thread_local bool t_chain_first = false;
void chain_begin() { t_chain_first = true; }
bool chain_take_first() {
    const bool f = t_chain_first;
    t_chain_first = false;
    return f;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

static std::atomic<int> g_tuning[EZB_TUNE_COUNT];
static std::atomic<bool> g_tuning_ready{false};
static const int kTuningDefaults[EZB_TUNE_COUNT] = {
    1,    // EZB_TUNE_PDL
    220,  // EZB_TUNE_GEMV_SMEM_KB
    1,    // EZB_TUNE_GEMV_PREFETCH (one stage ahead of the dependency wait measured fastest in the chained layer)
    1,    // EZB_TUNE_GEMV_CTAS_PER_SM
    128,  // EZB_TUNE_ATTN_MIN_CHUNK
    8,    // EZB_TUNE_ATTN_WAVES
    0,    // EZB_TUNE_GEMV_KC (automatic)
    1,    // EZB_TUNE_GEMV_ROWS8
    0,    // EZB_TUNE_PDL_ACROSS_CALLS
    1,    // EZB_TUNE_L2_PREFETCH
    192,  // EZB_TUNE_L2_PREFETCH_KB
    0,    // EZB_TUNE_GEMV_WINDOW
    0,    // EZB_TUNE_L2_PREFETCH_ATTN_KB
    1,    // EZB_TUNE_TC
    0,    // EZB_TUNE_ATTN_WAVES_UNIFORM
    0,    // EZB_TUNE_TP_POLL_ALL
    0,    // EZB_TUNE_TP_PULL
    1,    // EZB_TUNE_MEGA
    0,    // EZB_TUNE_MEGA_L2_STAGES (pulling stages into L2 behind a full ring measured slower: 78.7 | 80.9 | 80.5 us at 0 | 4 | 6)
    1000, // EZB_TUNE_WAIT_LIMIT_MS
    0,    // EZB_TUNE_MEGA_STAGES
    2,    // EZB_TUNE_MEGA_INFLIGHT (two of the three stages of the ring outstanding: 77.7 us against 78.3 with all three)
    1,    // EZB_TUNE_MEGA_GATE
    5000, // EZB_TUNE_TP_WAIT_LIMIT_MS
    0,    // EZB_TUNE_TP_STRONG_STORES
    1,    // EZB_TUNE_STREAM_EVICT_FIRST
};
static const char* kTuningEnv[EZB_TUNE_COUNT] = {
    "EZB_TUNE_PDL",          "EZB_TUNE_GEMV_SMEM_KB",   "EZB_TUNE_GEMV_PREFETCH", "EZB_TUNE_GEMV_CTAS_PER_SM",
    "EZB_TUNE_ATTN_MIN_CHUNK", "EZB_TUNE_ATTN_WAVES", "EZB_TUNE_GEMV_KC", "EZB_TUNE_GEMV_ROWS8", "EZB_TUNE_PDL_ACROSS_CALLS", "EZB_TUNE_L2_PREFETCH", "EZB_TUNE_L2_PREFETCH_KB", "EZB_TUNE_GEMV_WINDOW", "EZB_TUNE_L2_PREFETCH_ATTN_KB", "EZB_TUNE_TC",
    "EZB_TUNE_ATTN_WAVES_UNIFORM", "EZB_TUNE_TP_POLL_ALL", "EZB_TUNE_TP_PULL", "EZB_TUNE_MEGA", "EZB_TUNE_MEGA_L2_STAGES",
    "EZB_TUNE_WAIT_LIMIT_MS", "EZB_TUNE_MEGA_STAGES", "EZB_TUNE_MEGA_INFLIGHT", "EZB_TUNE_MEGA_GATE",
    "EZB_TUNE_TP_WAIT_LIMIT_MS", "EZB_TUNE_TP_STRONG_STORES", "EZB_TUNE_STREAM_EVICT_FIRST",
};

static void tuning_init() {
    if (g_tuning_ready.load()) return;
    for (int i = 0; i < EZB_TUNE_COUNT; ++i) {
        int v = kTuningDefaults[i];
        if (const char* e = std::getenv(kTuningEnv[i])) v = std::atoi(e);
        g_tuning[i].store(v);
    }
    g_tuning_ready.store(true);
}

int tuning(int key) {
    tuning_init();
    return (key >= 0 && key < EZB_TUNE_COUNT) ? g_tuning[key].load() : 0;
}

long long wait_limit_cycles() {
    long long ms = tuning(EZB_TUNE_WAIT_LIMIT_MS);
    if (ms < 1) ms = 1;
    return ms * 2000000LL;
}

static size_t round256(size_t v) { return (v + 255) / 256 * 256; }

// Carves the layer workspace.  The attention part comes first because it holds
// the counters that must start at zero.
struct LayerWorkspace {
    void* attn;
    void* tc;  // tensor-core path: split counters (zero between calls) and partial tiles; null at batch 1
    bf16 *qkv, *attn_out, *x2, *h, *xn;
    void* mega;  // batch 1: barrier counters and slice records of the single-kernel layer (zero before first use)
    size_t total;
};

// Largest tensor-core workspace any projection of a layer with these sizes needs.
static size_t layer_tc_bytes(int B, int H, int I, int rows_qkv) {
    if (B < 2) return 0;
    size_t m = gemm_tc_workspace_bytes(B, rows_qkv, false);
    size_t v = gemm_tc_workspace_bytes(B, H, false);
    if (v > m) m = v;
    v = gemm_tc_workspace_bytes(B, I, true);
    if (v > m) m = v;
    return m;
}

static LayerWorkspace carve_layer_ws(void* base, int B, int S, int H, int I, int NH, int NKV, int D) {
    LayerWorkspace w;
    unsigned char* p = static_cast<unsigned char*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        unsigned char* r = p ? p + off : nullptr;
        off += round256(bytes);
        return r;
    };
    w.attn = take(attn_workspace_bytes(B, NH, NKV, S, D));
    const size_t tc_bytes = layer_tc_bytes(B, H, I, (NH + 2 * NKV) * D);
    w.tc = tc_bytes ? take(tc_bytes) : nullptr;
    w.qkv = reinterpret_cast<bf16*>(take((size_t)B * (NH + 2 * NKV) * D * 2));
    w.attn_out = reinterpret_cast<bf16*>(take((size_t)B * NH * D * 2));
    w.x2 = reinterpret_cast<bf16*>(take((size_t)B * H * 2));
    w.h = reinterpret_cast<bf16*>(take((size_t)B * I * 2));
    w.xn = reinterpret_cast<bf16*>(take((size_t)B * H * 2));
    w.mega = (B == 1) ? take(decode_mega_workspace_bytes(NKV, D)) : nullptr;
    w.total = off;
    return w;
}

struct FfnWorkspace {
    void* tc;
    bf16 *x2, *h, *xn;
    size_t total;
};

static FfnWorkspace carve_ffn_ws(void* base, int B, int H, int I) {
    FfnWorkspace w;
    unsigned char* p = static_cast<unsigned char*>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        unsigned char* r = p ? p + off : nullptr;
        off += round256(bytes);
        return r;
    };
    const size_t tc_bytes = layer_tc_bytes(B, H, I, H);
    w.tc = tc_bytes ? take(tc_bytes) : nullptr;
    w.x2 = reinterpret_cast<bf16*>(take((size_t)B * H * 2));
    w.h = reinterpret_cast<bf16*>(take((size_t)B * I * 2));
    w.xn = reinterpret_cast<bf16*>(take((size_t)B * H * 2));
    w.total = off;
    return w;
}

static int check_common_layer_dims(int B, int H, int I, int Q) {
    EZB_REQUIRE(B >= 1 && H >= 1 && I >= 1 && Q >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(B <= 64, "batch above 64 is not supported");
    EZB_REQUIRE_SHAPE(H % 16 == 0, "hidden_size must be divisible by 16");
    EZB_REQUIRE_SHAPE(I % 16 == 0, "intermediate_size must be divisible by 16");
    EZB_REQUIRE_SHAPE(Q % 16 == 0, "num_heads * head_dim must be divisible by 16");
    return EZB_OK;
}

static const PrefetchList kNoPrefetch = {};

// Rows [skip_kb, skip_kb + kb) (in KB per CTA) of a following GEMV's weight(s).
static PrefetchPlan next_rows(const bf16* W0, const bf16* W1, int N, int K, int kb, int skip_kb = 0) {
    const long long row_bytes = (long long)K * 2 * (W1 ? 2 : 1);
    long long cap = (long long)kb * 1024 / row_bytes;
    if (cap < 1) cap = 1;
    const long long skip = (long long)skip_kb * 1024 / row_bytes;
    return prefetch_plan_rows(W0, W1, N, K, (int)cap, (int)skip);
}
static PrefetchList one_plan(const PrefetchPlan& a) {
    PrefetchList l = {};
    l.plan[0] = a;
    return l;
}

// o_proj (+residual or fp32 partial), gate/up + SwiGLU, down (+residual or fp32 partial)
static cudaError_t launch_o_proj(const bf16* attn, const bf16* Wo, int B, int H, int Q, const bf16* residual, void* out,
                                 bool f32_partial, cudaStream_t stream, const PrefetchList& next = kNoPrefetch,
                                 void* tc = nullptr) {
    GemvArgs g;
    g.tc_workspace = tc;
    g.W0 = Wo, g.ldw = Q, g.N = H, g.K = Q, g.B = B;
    g.x = attn, g.ldx = Q;
    g.prologue = PRO_NONE;
    g.epilogue = f32_partial ? EPI_STORE_F32 : EPI_RESIDUAL;
    g.residual = residual, g.ldres = H;
    g.out = out, g.ldout = H;
    g.next = next;
    g.trace_id = 3;
    return launch_gemv(g, stream);
}

static cudaError_t launch_gate_up(const bf16* x, const float* x_add, bf16* x_sum_out, const bf16* norm_w, const bf16* Wg,
                                  const bf16* Wu, int B, int H, int I, float eps, bf16* h, bf16* xn_scratch,
                                  cudaStream_t stream, const PrefetchList& next = kNoPrefetch, void* tc = nullptr) {
    GemvArgs g;
    g.tc_workspace = tc;
    g.W0 = Wg, g.W1 = Wu, g.ldw = H, g.N = I, g.K = H, g.B = B;
    g.x = x, g.ldx = H;
    g.x_add = x_add, g.ldadd = H, g.x_sum_out = x_sum_out, g.ldsum = H;
    g.norm_w = norm_w, g.eps = eps;
    g.prologue = x_add ? PRO_ADD_RMSNORM : PRO_RMSNORM;
    g.epilogue = EPI_SWIGLU;
    g.out = h, g.ldout = I;
    g.xn_scratch = xn_scratch;
    g.next = next;
    g.trace_id = 4;
    return launch_gemv(g, stream);
}

static cudaError_t launch_down(const bf16* h, const bf16* Wd, int B, int H, int I, const bf16* residual, void* out,
                               bool f32_partial, cudaStream_t stream, const PrefetchList& next = kNoPrefetch,
                               void* tc = nullptr) {
    GemvArgs g;
    g.tc_workspace = tc;
    g.W0 = Wd, g.ldw = I, g.N = H, g.K = I, g.B = B;
    g.x = h, g.ldx = I;
    g.prologue = PRO_NONE;
    g.epilogue = f32_partial ? EPI_STORE_F32 : EPI_RESIDUAL;
    g.residual = residual, g.ldres = H;
    g.out = out, g.ldout = H;
    g.trace_id = 5;
    g.next = next;
    return launch_gemv(g, stream);
}

// What a layer of a decoder stack has beyond the reference's layer operator: norm weights
// (null = unit), the rotary table rows of the token's position (null = no rotation), and the
// weights the last kernel should start pulling into L2 for the layer that follows.
struct LayerExtras {
    const bf16* input_norm_w = nullptr;
    const bf16* post_norm_w = nullptr;
    const bf16* q_norm_w = nullptr;
    const bf16* k_norm_w = nullptr;
    const bf16* rope_cos = nullptr;
    const bf16* rope_sin = nullptr;
    const bf16* next_Wqkv = nullptr;
    const int* seq_lens = nullptr;  // per-row valid lengths (device); the new token goes to slot len-1
    int rope_by_len = 0;            // rope_cos / rope_sin are table bases indexed by that slot
    const int* page_table = nullptr;  // paged caches (see AttnArgs)
    int page_shift = 0, max_pages = 0, num_pages = 0;
};
static const LayerExtras kPlainLayer = {};

static cudaError_t launch_qkv_and_attention(const bf16* hidden, bf16* Kc, bf16* Vc, const bf16* Wqkv, const LayerWorkspace& w,
                                            int B, int S, int H, int NH, int NKV, int D, float eps, cudaStream_t stream,
                                            const bf16* Wo, const PrefetchPlan* after_wo = nullptr,
                                            const LayerExtras& ex = kPlainLayer) {
    const int rows = (NH + 2 * NKV) * D;
    GemvArgs g;
    g.W0 = Wqkv, g.ldw = H, g.N = rows, g.K = H, g.B = B;
    g.x = hidden, g.ldx = H;
    g.norm_w = ex.input_norm_w;
    g.eps = eps, g.prologue = PRO_RMSNORM, g.epilogue = EPI_STORE;
    g.out = w.qkv, g.ldout = rows;
    g.xn_scratch = w.xn;
    g.tc_workspace = w.tc;
    g.trace_id = 1;
    // while the projection drains, start pulling the KV cache (if it is small enough to sit in L2)
    const size_t kv_bytes = (size_t)B * NKV * S * D * 2;
    if (!ex.page_table && 2 * kv_bytes <= ((size_t)48 << 20)) g.next = one_plan(prefetch_plan_flat(Kc, Vc, kv_bytes));
    cudaError_t e = launch_gemv(g, stream);
    if (e != cudaSuccess) return e;

    AttnArgs a;
    a.K = Kc, a.V = Vc;
    a.Out = w.attn_out, a.o_bstride = (long long)NH * D;
    a.B = B, a.H = NH, a.NKV = NKV, a.S = S, a.D = D;
    a.workspace = w.attn;
    a.fuse_new_token = 1;
    a.qkv = w.qkv, a.qkv_bstride = rows;
    a.K_cache_w = Kc, a.V_cache_w = Vc;
    a.eps = eps;
    a.q_norm_w = ex.q_norm_w, a.k_norm_w = ex.k_norm_w, a.rope_cos = ex.rope_cos, a.rope_sin = ex.rope_sin;
    a.seq_lens = ex.seq_lens, a.rope_by_len = ex.rope_by_len;
    a.page_table = ex.page_table, a.page_shift = ex.page_shift, a.max_pages = ex.max_pages, a.num_pages = ex.num_pages;
    // attention is latency-bound at small batch: let HBM stream the output projection meanwhile
    if ((size_t)H * NH * D * 2 <= ((size_t)64 << 20)) {
        a.next = one_plan(next_rows(Wo, nullptr, H, NH * D, 1 << 20));
        if (after_wo) a.next.plan[1] = *after_wo;
    }
    return launch_attn_decode(a, stream);
}

static int check_layer_args(int B, int S, int H, int I, int NH, int NKV, int D) {
    EZB_REQUIRE(S >= 1 && NH >= 1 && NKV >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(D == 64 || D == 128, "head_dim must be 64 or 128");
    EZB_REQUIRE_SHAPE(NH % NKV == 0, "num_heads must be divisible by num_kv_heads");
    EZB_REQUIRE_SHAPE(NH / NKV <= 16, "more than 16 query heads per kv head is not supported in the fused layer");
    return check_common_layer_dims(B, H, I, NH * D);
}

}  // namespace ezb

using namespace ezb;

extern "C" {

int ezb_version(void) { return 100; }

const char* ezb_strerror(int code) {
    switch (code) {
        case EZB_OK: return "ok";
        case EZB_ERR_INVALID_ARGUMENT: return "invalid argument";
        case EZB_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
        case EZB_ERR_CUDA: return "CUDA runtime error";
        case EZB_ERR_WORKSPACE: return "workspace missing or too small";
        case EZB_ERR_DEVICE_FAULT: return "a kernel recorded a device-side fault";
        default: return "unknown error code";
    }
}

const char* ezb_last_error_message(void) { return t_message; }

int ezb_set_tuning(int key, int value) {
    tuning_init();
    EZB_REQUIRE(key >= 0 && key < EZB_TUNE_COUNT, "unknown tuning key");
    g_tuning[key].store(value);
    return EZB_OK;
}

int ezb_get_tuning(int key) { return tuning(key); }

int ezb_trace_enable(void* records, unsigned int* cursor, unsigned int capacity) {
    g_trace.buf = static_cast<unsigned long long*>(records);
    g_trace.cursor = cursor;
    g_trace.capacity = (records && cursor) ? capacity : 0;
    if (!g_trace.capacity) g_trace.buf = nullptr;
    return EZB_OK;
}

int ezb_device_status(unsigned int* status_out_host, int clear) {
    EZB_REQUIRE(status_out_host != nullptr, "status_out_host is null");
    EZB_CUDA_TRY(cudaDeviceSynchronize());
    EZB_CUDA_TRY(cudaMemcpyFromSymbol(status_out_host, g_status_word, sizeof(unsigned int)));
    if (clear && *status_out_host != 0) {
        const unsigned int zero = 0;
        EZB_CUDA_TRY(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(unsigned int)));
    }
    return *status_out_host == 0 ? EZB_OK : EZB_ERR_DEVICE_FAULT;
}

int ezb_gemv_bf16(const void* x, const void* W, void* y, int N, int K, ezb_stream_t stream) {
    EZB_REQUIRE(x && W && y, "null pointer");
    EZB_REQUIRE(N >= 1 && K >= 1, "N and K must be positive");
    EZB_REQUIRE_SHAPE(K % 16 == 0, "K must be divisible by 16");
    EZB_REQUIRE(aligned16(x) && aligned16(W) && (reinterpret_cast<uintptr_t>(y) & 1u) == 0, "x and W must be 16-byte aligned, y 2-byte aligned");
    GemvArgs g;
    g.W0 = static_cast<const bf16*>(W), g.ldw = K, g.N = N, g.K = K, g.B = 1;
    g.x = static_cast<const bf16*>(x), g.ldx = K;
    g.out = y, g.ldout = N;
    chain_begin();
    EZB_CUDA_TRY(launch_gemv(g, stream));
    return EZB_OK;
}

size_t ezb_gemv_workspace_bytes(int B, int N, int K) {
    (void)K;
    if (B < 2 || N < 1) return 256;
    return gemm_tc_workspace_bytes(B, N, false);  // split counters and partial tiles of the tensor-core path
}

int ezb_gemv_batched_bf16(const void* X, const void* W, void* Y, void* workspace, size_t workspace_bytes, int B, int N, int K,
                          ezb_stream_t stream) {
    EZB_REQUIRE(X && W && Y, "null pointer");
    EZB_REQUIRE(N >= 1 && K >= 1 && B >= 1, "B, N and K must be positive");
    if (B >= 2 && (!workspace || workspace_bytes < gemm_tc_workspace_bytes(B, N, false))) {
        set_last_message("workspace missing or smaller than ezb_gemv_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    EZB_REQUIRE_SHAPE(B <= 64, "batch above 64 is not supported");
    EZB_REQUIRE_SHAPE(K % 16 == 0, "K must be divisible by 16");
    EZB_REQUIRE(aligned16(X) && aligned16(W), "X and W must be 16-byte aligned");
    GemvArgs g;
    g.W0 = static_cast<const bf16*>(W), g.ldw = K, g.N = N, g.K = K, g.B = B;
    g.x = static_cast<const bf16*>(X), g.ldx = K;
    g.out = Y, g.ldout = N;
    g.tc_workspace = B >= 2 ? workspace : nullptr;
    chain_begin();
    EZB_CUDA_TRY(launch_gemv(g, stream));
    return EZB_OK;
}

int ezb_rmsnorm_f32(const float* X, float* Out, int rows, int dim, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(X && Out, "null pointer");
    EZB_REQUIRE(rows >= 1 && dim >= 1, "rows and dim must be positive");
    EZB_REQUIRE(aligned16(X) && aligned16(Out), "X and Out must be 16-byte aligned");
    chain_begin();
    EZB_CUDA_TRY(launch_rmsnorm_f32(X, Out, rows, dim, eps, stream));
    return EZB_OK;
}

int ezb_rmsnorm_bf16(const void* X, const void* w_or_null, void* Out, int rows, int dim, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(X && Out, "null pointer");
    EZB_REQUIRE(rows >= 1 && dim >= 1, "rows and dim must be positive");
    EZB_REQUIRE_SHAPE(dim % 8 == 0, "dim must be divisible by 8");
    EZB_REQUIRE(aligned16(X) && aligned16(Out) && aligned16(w_or_null), "pointers must be 16-byte aligned");
    RowPrepArgs a;
    a.x = static_cast<const bf16*>(X), a.ldx = dim;
    a.w = static_cast<const bf16*>(w_or_null);
    a.y = static_cast<bf16*>(Out), a.ldy = dim;
    a.rows = rows, a.dim = dim, a.eps = eps, a.normalize = 1;
    chain_begin();
    EZB_CUDA_TRY(launch_row_prep(a, stream));
    return EZB_OK;
}

int ezb_qk_norm_rope(const void* q, const void* k, const void* v, const void* qw, const void* kw, const void* cos,
                     const void* sin, void* K_cache, void* V_cache, void* q_out, void* k_out, int B, int NQ, int NKV,
                     int D, int S, int position, const int* positions_or_null, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(q && k && v && qw && kw && cos && sin && K_cache && V_cache && q_out && k_out, "null pointer");
    EZB_REQUIRE(B >= 1 && NQ >= 1 && NKV >= 1 && S >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(D >= 8 && D <= 512 && (D & (D - 1)) == 0, "head_dim must be a power of two in [8, 512]");
    EZB_REQUIRE_SHAPE(NQ % NKV == 0, "num_heads must be divisible by num_kv_heads");
    EZB_REQUIRE(positions_or_null || (position >= 0 && position < S), "position must be in [0, max_seq_len)");
    RopeArgs a;
    a.q = static_cast<const bf16*>(q), a.k = static_cast<const bf16*>(k), a.v = static_cast<const bf16*>(v);
    a.qw = static_cast<const bf16*>(qw), a.kw = static_cast<const bf16*>(kw);
    a.cos = static_cast<const bf16*>(cos), a.sin = static_cast<const bf16*>(sin);
    a.K_cache = static_cast<bf16*>(K_cache), a.V_cache = static_cast<bf16*>(V_cache);
    a.q_out = static_cast<bf16*>(q_out), a.k_out = static_cast<bf16*>(k_out);
    a.B = B, a.NQ = NQ, a.NKV = NKV, a.D = D, a.S = S, a.position = position;
    a.positions = positions_or_null, a.eps = eps;
    chain_begin();
    EZB_CUDA_TRY(launch_qk_norm_rope(a, stream));
    return EZB_OK;
}

size_t ezb_attn_decode_workspace_bytes(int B, int H, int NKV, int S, int D) {
    if (B < 1 || H < 1 || NKV < 1 || S < 1 || D < 1 || H % NKV) return 0;
    return attn_workspace_bytes(B, H, NKV, S, D);
}

int ezb_attn_decode(const void* Q, const void* K, const void* V, void* Out, void* workspace, size_t workspace_bytes, int B,
                    int H, int NKV, int S, int D, const int* seq_lens_or_null, ezb_stream_t stream) {
    EZB_REQUIRE(Q && K && V && Out, "null pointer");
    EZB_REQUIRE(B >= 1 && H >= 1 && NKV >= 1 && S >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(D == 64 || D == 128, "head_dim must be 64 or 128");
    EZB_REQUIRE_SHAPE(H % NKV == 0, "num_heads must be divisible by num_kv_heads");
    EZB_REQUIRE_SHAPE(B <= 65535 && NKV <= 65535, "batch and kv heads are limited to 65535");
    EZB_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(Out), "Q, K, V and Out must be 16-byte aligned");
    if (!workspace || workspace_bytes < attn_workspace_bytes(B, H, NKV, S, D)) {
        set_last_message("attention workspace missing or smaller than ezb_attn_decode_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    AttnArgs a;
    a.Q = static_cast<const bf16*>(Q), a.q_bstride = (long long)H * D;
    a.K = static_cast<const bf16*>(K), a.V = static_cast<const bf16*>(V);
    a.Out = static_cast<bf16*>(Out), a.o_bstride = (long long)H * D;
    a.seq_lens = seq_lens_or_null;
    a.B = B, a.H = H, a.NKV = NKV, a.S = S, a.D = D;
    a.workspace = workspace;
    chain_begin();
    EZB_CUDA_TRY(launch_attn_decode(a, stream));
    return EZB_OK;
}

static int page_shift_of(int page_size) {
    int sh = 0;
    while ((1 << sh) < page_size) ++sh;
    return ((1 << sh) == page_size && page_size >= 64) ? sh : -1;
}

int ezb_attn_decode_paged(const void* Q, const void* K_pool, const void* V_pool, const int* page_table, void* Out,
                          void* workspace, size_t workspace_bytes, int B, int H, int NKV, int max_pages, int page_size, int D,
                          int num_pages, const int* seq_lens, ezb_stream_t stream) {
    EZB_REQUIRE(Q && K_pool && V_pool && page_table && Out && seq_lens, "null pointer");
    EZB_REQUIRE(B >= 1 && H >= 1 && NKV >= 1 && max_pages >= 1 && num_pages >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(page_shift_of(page_size) >= 0, "page_size must be a power of two >= 64");
    EZB_REQUIRE_SHAPE(D == 64 || D == 128, "head_dim must be 64 or 128");
    EZB_REQUIRE_SHAPE(H % NKV == 0, "num_heads must be divisible by num_kv_heads");
    EZB_REQUIRE_SHAPE(B <= 65535 && NKV <= 65535, "batch and kv heads are limited to 65535");
    EZB_REQUIRE(aligned16(Q) && aligned16(K_pool) && aligned16(V_pool) && aligned16(Out), "Q, Out and the page pools must be 16-byte aligned");
    const int S = max_pages * page_size;
    if (!workspace || workspace_bytes < attn_workspace_bytes(B, H, NKV, S, D)) {
        set_last_message("attention workspace missing or smaller than ezb_attn_decode_workspace_bytes(B, H, NKV, max_pages * page_size, D)");
        return EZB_ERR_WORKSPACE;
    }
    AttnArgs a;
    a.Q = static_cast<const bf16*>(Q), a.q_bstride = (long long)H * D;
    a.K = static_cast<const bf16*>(K_pool), a.V = static_cast<const bf16*>(V_pool);
    a.Out = static_cast<bf16*>(Out), a.o_bstride = (long long)H * D;
    a.seq_lens = seq_lens;
    a.B = B, a.H = H, a.NKV = NKV, a.S = S, a.D = D;
    a.page_table = page_table, a.page_shift = page_shift_of(page_size), a.max_pages = max_pages, a.num_pages = num_pages;
    a.workspace = workspace;
    chain_begin();
    EZB_CUDA_TRY(launch_attn_decode(a, stream));
    return EZB_OK;
}

size_t ezb_o_proj_ffn_workspace_bytes(int B, int H, int I, int Q) {
    if (B < 1 || H < 1 || I < 1 || Q < 1) return 0;
    return carve_ffn_ws(nullptr, B, H, I).total;
}

int ezb_o_proj_ffn(const void* attn, const void* residual, const void* Wo, const void* post_norm_w, const void* Wg,
                   const void* Wu, const void* Wd, void* out, void* workspace, size_t workspace_bytes, int B, int H, int I,
                   int Q, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(attn && residual && Wo && post_norm_w && Wg && Wu && Wd && out, "null pointer");
    if (int rc = check_common_layer_dims(B, H, I, Q)) return rc;
    EZB_REQUIRE(aligned16(attn) && aligned16(residual) && aligned16(Wo) && aligned16(post_norm_w) && aligned16(Wg) &&
                    aligned16(Wu) && aligned16(Wd) && aligned16(out),
                "pointers must be 16-byte aligned");
    FfnWorkspace w = carve_ffn_ws(workspace, B, H, I);
    if (!workspace || workspace_bytes < w.total) {
        set_last_message("workspace missing or smaller than ezb_o_proj_ffn_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    chain_begin();
    const int pf_kb = tuning(EZB_TUNE_L2_PREFETCH_KB);
    EZB_CUDA_TRY(launch_o_proj(static_cast<const bf16*>(attn), static_cast<const bf16*>(Wo), B, H, Q,
                               static_cast<const bf16*>(residual), w.x2, false, stream,
                               one_plan(next_rows(static_cast<const bf16*>(Wg), static_cast<const bf16*>(Wu), I, H, pf_kb)), w.tc));
    EZB_CUDA_TRY(launch_gate_up(w.x2, nullptr, nullptr, static_cast<const bf16*>(post_norm_w), static_cast<const bf16*>(Wg),
                                static_cast<const bf16*>(Wu), B, H, I, eps, w.h, w.xn, stream,
                                one_plan(next_rows(static_cast<const bf16*>(Wd), nullptr, H, I, pf_kb)), w.tc));
    EZB_CUDA_TRY(launch_down(w.h, static_cast<const bf16*>(Wd), B, H, I, w.x2, out, false, stream, kNoPrefetch, w.tc));
    return EZB_OK;
}

size_t ezb_qwen3_decode_layer_workspace_bytes(int B, int S, int H, int I, int NH, int NKV, int D) {
    if (B < 1 || S < 1 || H < 1 || I < 1 || NH < 1 || NKV < 1 || D < 1 || NH % NKV) return 0;
    return carve_layer_ws(nullptr, B, S, H, I, NH, NKV, D).total;
}

static MegaArgs mega_args(const bf16* hid, bf16* Kc, bf16* Vc, const bf16* Wqkv, const bf16* Wo, const bf16* wgu, const bf16* Wd,
                          bf16* out, const LayerWorkspace& w, int S, int H, int I, int NH, int NKV, int D, float eps,
                          const LayerExtras& ex) {
    MegaArgs m;
    m.hidden = hid, m.out = out, m.Kc = Kc, m.Vc = Vc;
    m.Wqkv = Wqkv, m.Wo = Wo, m.Wgu = wgu, m.Wd = Wd;
    m.input_norm_w = ex.input_norm_w, m.post_norm_w = ex.post_norm_w, m.q_norm_w = ex.q_norm_w, m.k_norm_w = ex.k_norm_w;
    m.rope_cos = ex.rope_cos, m.rope_sin = ex.rope_sin;
    m.qkv = w.qkv, m.attn_out = w.attn_out, m.x2 = w.x2, m.h = w.h;
    m.mega_workspace = w.mega;
    m.S = S, m.H = H, m.I = I, m.NH = NH, m.NKV = NKV, m.D = D, m.eps = eps;
    return m;
}

// One layer's five (seven with the tensor-core path) launches.  The caller has opened the chain.
static int run_layer(const bf16* hid, bf16* Kc, bf16* Vc, const bf16* Wqkv, const bf16* Wo, const bf16* wgu, const bf16* Wd,
                     bf16* out, const LayerWorkspace& w, int B, int S, int H, int I, int NH, int NKV, int D, float eps,
                     const LayerExtras& ex, cudaStream_t stream) {
    if (B == 1 && !ex.seq_lens && !ex.page_table && w.mega) {
        // batch 1 on contiguous caches: the whole layer as one persistent kernel
        const MegaArgs m = mega_args(hid, Kc, Vc, Wqkv, Wo, wgu, Wd, out, w, S, H, I, NH, NKV, D, eps, ex);
        if (decode_mega_supported(m)) {
            EZB_CUDA_TRY(launch_decode_mega(m, stream));
            return EZB_OK;
        }
    }
    const int pf_kb = tuning(EZB_TUNE_L2_PREFETCH_KB);
    const int pf_attn_kb = tuning(EZB_TUNE_L2_PREFETCH_ATTN_KB);
    // attention is latency-bound: besides Wo it can pull the head of the gate/up rows; o_proj then pulls the rows after those
    const PrefetchPlan gu_head = next_rows(wgu, wgu + (size_t)I * H, I, H, pf_attn_kb);
    EZB_CUDA_TRY(launch_qkv_and_attention(hid, Kc, Vc, Wqkv, w, B, S, H, NH, NKV, D, eps, stream, Wo,
                                          pf_attn_kb > 0 ? &gu_head : nullptr, ex));
    EZB_CUDA_TRY(launch_o_proj(w.attn_out, Wo, B, H, NH * D, hid, w.x2, false, stream,
                               one_plan(next_rows(wgu, wgu + (size_t)I * H, I, H, pf_kb, pf_attn_kb > 0 ? pf_attn_kb : 0)), w.tc));
    EZB_CUDA_TRY(launch_gate_up(w.x2, nullptr, nullptr, ex.post_norm_w, wgu, wgu + (size_t)I * H, B, H, I, eps, w.h, w.xn, stream,
                                one_plan(next_rows(Wd, nullptr, H, I, pf_kb)), w.tc));
    const PrefetchList after = ex.next_Wqkv ? one_plan(next_rows(ex.next_Wqkv, nullptr, (NH + 2 * NKV) * D, H, pf_kb)) : kNoPrefetch;
    EZB_CUDA_TRY(launch_down(w.h, Wd, B, H, I, w.x2, out, false, stream, after, w.tc));
    return EZB_OK;
}

int ezb_qwen3_decode_layer(const void* hidden, void* K_cache, void* V_cache, const void* Wqkv, const void* Wo,
                           const void* Wgu, const void* Wd, void* out, void* workspace, size_t workspace_bytes, int B,
                           int S, int H, int I, int NH, int NKV, int D, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(hidden && K_cache && V_cache && Wqkv && Wo && Wgu && Wd && out, "null pointer");
    if (int rc = check_layer_args(B, S, H, I, NH, NKV, D)) return rc;
    EZB_REQUIRE(aligned16(hidden) && aligned16(K_cache) && aligned16(V_cache) && aligned16(Wqkv) && aligned16(Wo) &&
                    aligned16(Wgu) && aligned16(Wd) && aligned16(out),
                "pointers must be 16-byte aligned");
    LayerWorkspace w = carve_layer_ws(workspace, B, S, H, I, NH, NKV, D);
    if (!workspace || workspace_bytes < w.total) {
        set_last_message("workspace missing or smaller than ezb_qwen3_decode_layer_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    chain_begin();
    return run_layer(static_cast<const bf16*>(hidden), static_cast<bf16*>(K_cache), static_cast<bf16*>(V_cache),
                     static_cast<const bf16*>(Wqkv), static_cast<const bf16*>(Wo), static_cast<const bf16*>(Wgu),
                     static_cast<const bf16*>(Wd), static_cast<bf16*>(out), w, B, S, H, I, NH, NKV, D, eps, kPlainLayer,
                     static_cast<cudaStream_t>(stream));
}

size_t ezb_qwen3_decode_stack_workspace_bytes(int B, int S, int H, int I, int NH, int NKV, int D) {
    if (check_layer_args(B, S, H, I, NH, NKV, D)) return 0;
    return carve_layer_ws(nullptr, B, S, H, I, NH, NKV, D).total + 2 * round256((size_t)B * H * sizeof(bf16));
}

static int run_stack(const void* hidden, void* out, const ezb_layer_t* layers, int n_layers, const void* rope_cos,
                     const void* rope_sin, int rope_position, const int* seq_lens, const int* page_table, int page_shift,
                     int max_pages, int num_pages, void* workspace, size_t workspace_bytes, int B, int S, int H, int I, int NH, int NKV, int D,
                     float eps, ezb_stream_t stream) {
    EZB_REQUIRE(hidden && out && layers && n_layers >= 1, "null pointer or no layers");
    EZB_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr) && rope_position >= 0, "rotary tables come as a pair; position >= 0");
    if (int rc = check_layer_args(B, S, H, I, NH, NKV, D)) return rc;
    EZB_REQUIRE(aligned16(hidden) && aligned16(out) && aligned16(rope_cos) && aligned16(rope_sin), "pointers must be 16-byte aligned");
    for (int l = 0; l < n_layers; ++l) {
        const ezb_layer_t& L = layers[l];
        EZB_REQUIRE(L.K_cache && L.V_cache && L.Wqkv && L.Wo && L.Wgu && L.Wd, "null pointer in a layer");
        EZB_REQUIRE(aligned16(L.K_cache) && aligned16(L.V_cache) && aligned16(L.Wqkv) && aligned16(L.Wo) && aligned16(L.Wgu) &&
                        aligned16(L.Wd) && aligned16(L.input_norm_w) && aligned16(L.post_norm_w) && aligned16(L.q_norm_w) &&
                        aligned16(L.k_norm_w),
                    "layer pointers must be 16-byte aligned");
    }
    LayerWorkspace w = carve_layer_ws(workspace, B, S, H, I, NH, NKV, D);
    const size_t hbytes = round256((size_t)B * H * sizeof(bf16));
    if (!workspace || workspace_bytes < w.total + 2 * hbytes) {
        set_last_message("workspace missing or smaller than ezb_qwen3_decode_stack_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    bf16* pp[2] = {reinterpret_cast<bf16*>(static_cast<unsigned char*>(workspace) + w.total),
                   reinterpret_cast<bf16*>(static_cast<unsigned char*>(workspace) + w.total + hbytes)};
    // one position for all rows: hand the kernel that table row; per-row lengths: the table base, indexed by len-1
    const size_t row_off = seq_lens ? 0 : (size_t)rope_position * D;
    const bf16* cos_row = rope_cos ? static_cast<const bf16*>(rope_cos) + row_off : nullptr;
    const bf16* sin_row = rope_sin ? static_cast<const bf16*>(rope_sin) + row_off : nullptr;
    chain_begin();  // one dependency chain through all layers
    const bf16* x = static_cast<const bf16*>(hidden);
    for (int l = 0; l < n_layers; ++l) {
        const ezb_layer_t& L = layers[l];
        LayerExtras ex;
        ex.input_norm_w = static_cast<const bf16*>(L.input_norm_w), ex.post_norm_w = static_cast<const bf16*>(L.post_norm_w);
        ex.q_norm_w = static_cast<const bf16*>(L.q_norm_w), ex.k_norm_w = static_cast<const bf16*>(L.k_norm_w);
        ex.rope_cos = cos_row, ex.rope_sin = sin_row;
        ex.seq_lens = seq_lens, ex.rope_by_len = seq_lens ? 1 : 0;
        ex.page_table = page_table, ex.page_shift = page_shift, ex.max_pages = max_pages, ex.num_pages = num_pages;
        ex.next_Wqkv = (l + 1 < n_layers) ? static_cast<const bf16*>(layers[l + 1].Wqkv) : nullptr;
        bf16* y = (l + 1 == n_layers) ? static_cast<bf16*>(out) : pp[l & 1];
        if (int rc = run_layer(x, static_cast<bf16*>(L.K_cache), static_cast<bf16*>(L.V_cache), static_cast<const bf16*>(L.Wqkv),
                               static_cast<const bf16*>(L.Wo), static_cast<const bf16*>(L.Wgu), static_cast<const bf16*>(L.Wd), y,
                               w, B, S, H, I, NH, NKV, D, eps, ex, static_cast<cudaStream_t>(stream)))
            return rc;
        x = y;
    }
    return EZB_OK;
}

int ezb_qwen3_decode_layer_tp_attn(const void* hidden, void* K_cache, void* V_cache, const void* Wqkv_local,
                                   const void* Wo_local, float* partial_o, void* workspace, size_t workspace_bytes, int B,
                                   int S, int H, int NH_local, int NKV_local, int D, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(hidden && K_cache && V_cache && Wqkv_local && Wo_local && partial_o, "null pointer");
    if (int rc = check_layer_args(B, S, H, 16, NH_local, NKV_local, D)) return rc;
    EZB_REQUIRE(aligned16(hidden) && aligned16(K_cache) && aligned16(V_cache) && aligned16(Wqkv_local) &&
                    aligned16(Wo_local) && aligned16(partial_o),
                "pointers must be 16-byte aligned");
    // the caller sized the workspace for its own I; only the attention part and the
    // activation rows in front of h are used here, which do not depend on I
    LayerWorkspace w = carve_layer_ws(workspace, B, S, H, 16, NH_local, NKV_local, D);
    if (!workspace || workspace_bytes < w.total) {
        set_last_message("workspace missing or smaller than ezb_qwen3_decode_layer_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    chain_begin();
    EZB_CUDA_TRY(launch_qkv_and_attention(static_cast<const bf16*>(hidden), static_cast<bf16*>(K_cache),
                                          static_cast<bf16*>(V_cache), static_cast<const bf16*>(Wqkv_local), w, B, S, H,
                                          NH_local, NKV_local, D, eps, stream, static_cast<const bf16*>(Wo_local)));
    EZB_CUDA_TRY(launch_o_proj(w.attn_out, static_cast<const bf16*>(Wo_local), B, H, NH_local * D, nullptr, partial_o, true,
                               stream, kNoPrefetch, w.tc));
    return EZB_OK;
}

int ezb_qwen3_decode_layer_tp_ffn(const void* hidden, const float* summed_o, const void* Wgu_local, const void* Wd_local,
                                  void* x2, float* partial_d, void* workspace, size_t workspace_bytes, int B, int H,
                                  int I_local, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(hidden && summed_o && Wgu_local && Wd_local && x2 && partial_d, "null pointer");
    if (int rc = check_common_layer_dims(B, H, I_local, 16)) return rc;
    EZB_REQUIRE(aligned16(hidden) && aligned16(summed_o) && aligned16(Wgu_local) && aligned16(Wd_local) && aligned16(x2) &&
                    aligned16(partial_d),
                "pointers must be 16-byte aligned");
    FfnWorkspace w = carve_ffn_ws(workspace, B, H, I_local);
    if (!workspace || workspace_bytes < w.total) {
        set_last_message("workspace missing or smaller than ezb_o_proj_ffn_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    const bf16* wgu = static_cast<const bf16*>(Wgu_local);
    chain_begin();
    EZB_CUDA_TRY(launch_gate_up(static_cast<const bf16*>(hidden), summed_o, static_cast<bf16*>(x2), nullptr, wgu,
                                wgu + (size_t)I_local * H, B, H, I_local, eps, w.h, w.xn, stream,
                                one_plan(next_rows(static_cast<const bf16*>(Wd_local), nullptr, H, I_local, tuning(EZB_TUNE_L2_PREFETCH_KB))), w.tc));
    EZB_CUDA_TRY(launch_down(w.h, static_cast<const bf16*>(Wd_local), B, H, I_local, nullptr, partial_d, true, stream,
                             kNoPrefetch, w.tc));
    return EZB_OK;
}

// The address a kernel uses for `p`: device memory as it is, pinned (page-locked, mapped) host memory through its
// device alias; pageable host memory has none.
static int device_view(const void* p, void** out, bool* is_host) {
    cudaPointerAttributes at;
    EZB_CUDA_TRY(cudaPointerGetAttributes(&at, p));
    if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) {
        *out = const_cast<void*>(p), *is_host = false;
        return EZB_OK;
    }
    if (at.type == cudaMemoryTypeHost && at.devicePointer) {
        *out = at.devicePointer, *is_host = true;
        return EZB_OK;
    }
    set_last_message("host buffers must be pinned (page-locked) memory: pageable memory has no device address");
    return EZB_ERR_INVALID_ARGUMENT;
}

int ezb_copy_pinned(void* dst, const void* src, size_t bytes, ezb_stream_t stream) {
    EZB_REQUIRE(dst && src && bytes >= 16 && bytes % 16 == 0, "null pointer, or a size that is not a positive multiple of 16");
    EZB_REQUIRE(aligned16(dst) && aligned16(src), "pointers must be 16-byte aligned");
    void *d = nullptr, *s = nullptr;
    bool d_host = false, s_host = false;
    if (int rc = device_view(dst, &d, &d_host)) return rc;
    if (int rc = device_view(src, &s, &s_host)) return rc;
    chain_begin();
    EZB_CUDA_TRY(launch_pinned_copy(d, s, bytes, d_host, static_cast<cudaStream_t>(stream)));
    return EZB_OK;
}

int ezb_vector_add_f32(const float* A, const float* B, float* C, long long n, ezb_stream_t stream) {
    EZB_REQUIRE(A && B && C && n >= 1, "null pointer or empty vector");
    EZB_CUDA_TRY(launch_vector_add_f32(A, B, C, n, static_cast<cudaStream_t>(stream)));
    return EZB_OK;
}

int ezb_softmax_f32(const float* X, float* Out, int rows, int dim, ezb_stream_t stream) {
    EZB_REQUIRE(X && Out && rows >= 1 && dim >= 1, "null pointer or empty matrix");
    EZB_CUDA_TRY(launch_softmax_f32(X, Out, rows, dim, static_cast<cudaStream_t>(stream)));
    return EZB_OK;
}

size_t ezb_reduce_workspace_bytes(void) { return reduce_workspace_bytes(); }

int ezb_reduce_sum_f32(const float* A, float* Out, long long n, void* workspace, size_t workspace_bytes, ezb_stream_t stream) {
    EZB_REQUIRE(A && Out && n >= 1, "null pointer or empty vector");
    if (!workspace || workspace_bytes < reduce_workspace_bytes()) {
        set_last_message("workspace missing or smaller than ezb_reduce_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    EZB_CUDA_TRY(launch_reduce_sum_f32(A, Out, n, workspace, static_cast<cudaStream_t>(stream)));
    return EZB_OK;
}

int ezb_pdl_gemm_f32(const float* x, const float* W1, const float* W2, float* y, float* z, int M, int K, int N, int P, int use_pdl,
                     ezb_stream_t stream) {
    EZB_REQUIRE(x && W1 && W2 && y && z, "null pointer");
    EZB_REQUIRE(M >= 1 && K >= 1 && N >= 1 && P >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(K % 4 == 0 && N % 4 == 0 && P % 4 == 0, "K, N and P must be divisible by 4 (16-byte row segments)");
    EZB_REQUIRE(aligned16(x) && aligned16(W1) && aligned16(W2) && aligned16(y) && aligned16(z), "pointers must be 16-byte aligned");
    EZB_CUDA_TRY(launch_pdl_gemm_f32(x, W1, W2, y, z, M, K, N, P, use_pdl != 0, static_cast<cudaStream_t>(stream)));
    return EZB_OK;
}

unsigned long long ezb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int ezb_hbm_stream(int op, const void* b, const void* c, void* a, long long n_vec4, float scalar, int block_size,
                   int blocks_per_sm, ezb_stream_t stream) {
    EZB_REQUIRE(op >= 0 && op <= 3, "op must be 0 (read), 1 (write), 2 (copy) or 3 (triad)");
    EZB_REQUIRE(a && (op == 1 || b) && (op != 3 || c), "null pointer");
    EZB_REQUIRE(n_vec4 >= 1 && block_size >= 32 && block_size <= 1024 && block_size % 32 == 0 && blocks_per_sm >= 1 &&
                    blocks_per_sm <= 32,
                "bad size, block size or blocks per SM");
    EZB_REQUIRE(aligned16(a) && aligned16(b) && aligned16(c), "pointers must be 16-byte aligned");
    // a read-only pass parks its (never written) checksum in the first word of `a`
    EZB_CUDA_TRY(launch_hbm_stream(op, b, c, a, n_vec4, scalar, block_size, blocks_per_sm, static_cast<float*>(a),
                                   static_cast<cudaStream_t>(stream)));
    return EZB_OK;
}

size_t ezb_tp_comm_bytes(int B, int H) {
    if (B < 1 || H < 1) return 0;
    return (size_t)kTpCtrlBytes + (size_t)2 * kTpSlots * B * H * sizeof(unsigned long long);
}

int ezb_tp_comm_alloc(size_t bytes, void** out) {
    EZB_REQUIRE(out && bytes >= (size_t)kTpCtrlBytes, "bad arguments");
    void* p = nullptr;
    EZB_CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        set_last_cuda_error(e);
        return EZB_ERR_CUDA;
    }
    *out = p;
    return EZB_OK;
}

int ezb_tp_comm_free(void* p) {
    if (p) EZB_CUDA_TRY(cudaFree(p));
    return EZB_OK;
}

int ezb_ipc_export(void* ptr, void* handle64) {
    EZB_REQUIRE(ptr && handle64, "null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    EZB_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
    std::memcpy(handle64, &h, sizeof(h));
    return EZB_OK;
}

int ezb_ipc_open(const void* handle64, void** out) {
    EZB_REQUIRE(handle64 && out, "null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    EZB_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *out = p;
    return EZB_OK;
}

int ezb_ipc_close(void* ptr) {
    if (ptr) EZB_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
    return EZB_OK;
}

static int make_tp_link(TpLink& base, void* const* comm_bases_host, int world, int rank, int B, int H) {
    EZB_REQUIRE(comm_bases_host, "null pointer");
    EZB_REQUIRE(world >= 1 && world <= kTpSlots && rank >= 0 && rank < world, "world must be 1..8 and rank inside it");
    for (int w = 0; w < world; ++w) EZB_REQUIRE(comm_bases_host[w] && aligned16(comm_bases_host[w]), "bad comm buffer pointer");
    const int poll_mode = tuning(EZB_TUNE_TP_POLL_ALL);
    const int pull_mode = tuning(EZB_TUNE_TP_PULL);
    long long wait_ms = tuning(EZB_TUNE_TP_WAIT_LIMIT_MS);
    if (wait_ms < 1) wait_ms = 1;
    base = {world, rank, {}, {}, (long long)B * H, -1, -1, -1, poll_mode == 1 || (poll_mode == 0 && world > 2) ? 1 : 0,
            pull_mode == 1 ? 1 : 0, wait_ms * 2000000LL, tuning(EZB_TUNE_TP_STRONG_STORES) ? 1 : 0};
    for (int r = 0; r < world; ++r) {
        base.ctrl_peer[r] = static_cast<unsigned int*>(comm_bases_host[r]);
        base.inbox_peer[r] = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(comm_bases_host[r]) + kTpCtrlBytes);
    }
    return EZB_OK;
}

int ezb_tp_allreduce_f32(void* buf, void* const* comm_bases_host, int world, int rank, int which, int B, int H,
                         ezb_stream_t stream) {
    EZB_REQUIRE(buf && aligned16(buf), "null or misaligned buffer");
    EZB_REQUIRE(which == 0 || which == 1, "which must be 0 or 1");
    EZB_REQUIRE(B >= 1 && H >= 1 && ((long long)B * H) % 4 == 0, "B * H must be a positive multiple of 4");
    TpLink link;
    if (int rc = make_tp_link(link, comm_bases_host, world, rank, B, H)) return rc;
    chain_begin();
    EZB_CUDA_TRY(launch_tp_allreduce(static_cast<float*>(buf), link, which, (long long)B * H, static_cast<cudaStream_t>(stream)));
    return EZB_OK;
}

static int check_tp_fused_shape(int B, int H, int I_local, int NH_local, int NKV_local, int D) {
    // every projection must run a kernel that knows the exchange: the small-batch kernel, or (batch >= 2)
    // the tensor-core kernel with the row kernel in front
    auto covered = [&](int K, int N, bool pair) {
        return gemv_small_batch_eligible(B, K) || (tuning(EZB_TUNE_TC) != 0 && gemm_tc_supported(B, K) && gemm_tc_fits(N, pair));
    };
    EZB_REQUIRE_SHAPE(covered(H, (NH_local + 2 * NKV_local) * D, false) && covered(NH_local * D, H, false) &&
                          covered(H, I_local, true) && covered(I_local, H, false),
                      "no kernel with the fused exchange covers this batch and these sizes");
    return EZB_OK;
}

// One tensor-parallel layer with the sums over ranks inside the kernels (five launches).
//   x_prev / gather_prev: the layer input is x_prev + sum(inbox 1) when gather_prev is set (the
//   previous layer's down projection pushed there), and is written to layer_in by the QKV kernel;
//   otherwise the layer input is x_prev itself and layer_in is not used.
//   x2_out receives hidden + sum(inbox 0); the down projection pushes into inbox 1, so the caller
//   finishes with x2_out + sum(inbox 1) (the next layer's QKV prologue, or a final row kernel).
static int run_layer_tp_fused(const bf16* x_prev, bool gather_prev, bf16* layer_in, bf16* x2_out, bf16* Kc, bf16* Vc,
                              const bf16* Wqkv, const bf16* Wo, const bf16* wgu, const bf16* Wd, const LayerWorkspace& w,
                              const TpLink& base, int B, int S, int H, int I_local, int NH_local, int NKV_local, int D, float eps,
                              const LayerExtras& ex, cudaStream_t stream) {
    const int Q = NH_local * D, rows = (NH_local + 2 * NKV_local) * D;
    const int pf_kb = tuning(EZB_TUNE_L2_PREFETCH_KB);
    const bf16* hid = gather_prev ? layer_in : x_prev;
    {   // QKV projection (norm prologue; gathers the previous layer's second sum when there is one)
        GemvArgs g;
        g.tc_workspace = w.tc, g.xn_scratch = w.xn;
        g.W0 = Wqkv, g.ldw = H, g.N = rows, g.K = H, g.B = B;
        g.x = x_prev, g.ldx = H;
        g.norm_w = ex.input_norm_w;
        g.eps = eps, g.prologue = gather_prev ? PRO_ADD_RMSNORM : PRO_RMSNORM, g.epilogue = EPI_STORE;
        g.out = w.qkv, g.ldout = rows;
        g.trace_id = 1;
        if (gather_prev) {
            g.x_sum_out = layer_in, g.ldsum = H;
            g.link = base, g.link.gather_inbox = 1;
        }
        const size_t kv_bytes = (size_t)B * NKV_local * S * D * 2;
        if (2 * kv_bytes <= ((size_t)48 << 20)) g.next = one_plan(prefetch_plan_flat(Kc, Vc, kv_bytes));
        EZB_CUDA_TRY(launch_gemv(g, stream));
    }
    {
        AttnArgs a;
        a.K = Kc, a.V = Vc;
        a.Out = w.attn_out, a.o_bstride = Q;
        a.B = B, a.H = NH_local, a.NKV = NKV_local, a.S = S, a.D = D;
        a.workspace = w.attn;
        a.fuse_new_token = 1;
        a.qkv = w.qkv, a.qkv_bstride = rows;
        a.K_cache_w = Kc, a.V_cache_w = Vc;
        a.eps = eps;
        a.q_norm_w = ex.q_norm_w, a.k_norm_w = ex.k_norm_w, a.rope_cos = ex.rope_cos, a.rope_sin = ex.rope_sin;
        a.seq_lens = ex.seq_lens, a.rope_by_len = ex.rope_by_len;
        if ((size_t)H * Q * 2 <= ((size_t)64 << 20)) a.next = one_plan(next_rows(Wo, nullptr, H, Q, 1 << 20));
        EZB_CUDA_TRY(launch_attn_decode(a, stream));
    }
    {   // o_proj: partial -> inbox 0 of every rank; also opens the next epoch of inbox 1
        GemvArgs g;
        g.tc_workspace = w.tc, g.xn_scratch = w.xn;
        g.W0 = Wo, g.ldw = Q, g.N = H, g.K = Q, g.B = B;
        g.x = w.attn_out, g.ldx = Q;
        g.epilogue = EPI_PUSH_F32, g.ldout = H;
        g.link = base, g.link.push_inbox = 0, g.link.bump_inbox = 1;
        g.next = one_plan(next_rows(wgu, wgu + (size_t)I_local * H, I_local, H, pf_kb));
        g.trace_id = 3;
        EZB_CUDA_TRY(launch_gemv(g, stream));
    }
    {   // gate/up: x2 = layer input + sum(inbox 0), norm, SwiGLU
        GemvArgs g;
        g.tc_workspace = w.tc, g.xn_scratch = w.xn;
        g.W0 = wgu, g.W1 = wgu + (size_t)I_local * H, g.ldw = H, g.N = I_local, g.K = H, g.B = B;
        g.x = hid, g.ldx = H;
        g.x_sum_out = x2_out, g.ldsum = H;
        g.norm_w = ex.post_norm_w;
        g.eps = eps, g.prologue = PRO_ADD_RMSNORM, g.epilogue = EPI_SWIGLU;
        g.out = w.h, g.ldout = I_local;
        g.link = base, g.link.gather_inbox = 0;
        g.next = one_plan(next_rows(Wd, nullptr, H, I_local, pf_kb));
        g.trace_id = 4;
        EZB_CUDA_TRY(launch_gemv(g, stream));
    }
    {   // down: partial -> inbox 1 of every rank; opens the next epoch of inbox 0
        GemvArgs g;
        g.tc_workspace = w.tc, g.xn_scratch = w.xn;
        g.W0 = Wd, g.ldw = I_local, g.N = H, g.K = I_local, g.B = B;
        g.x = w.h, g.ldx = I_local;
        g.epilogue = EPI_PUSH_F32, g.ldout = H;
        g.link = base, g.link.push_inbox = 1, g.link.bump_inbox = 0;
        if (ex.next_Wqkv) g.next = one_plan(next_rows(ex.next_Wqkv, nullptr, rows, H, pf_kb));
        g.trace_id = 5;
        EZB_CUDA_TRY(launch_gemv(g, stream));
    }
    return EZB_OK;
}

// out = x2 + sum(inbox 1): closes the last layer of a fused tensor-parallel chain
static int finish_tp_fused(const bf16* x2, bf16* out, const TpLink& base, int B, int H, cudaStream_t stream) {
    RowPrepArgs a;
    a.x = x2, a.ldx = H;
    a.sum_out = out, a.ldsum = H;
    a.rows = B, a.dim = H, a.normalize = 0;
    a.link = base, a.link.gather_inbox = 1;
    EZB_CUDA_TRY(launch_row_prep(a, stream));
    return EZB_OK;
}

int ezb_qwen3_decode_layer_tp_fused(const void* hidden, void* K_cache, void* V_cache, const void* Wqkv_local,
                                    const void* Wo_local, const void* Wgu_local, const void* Wd_local, void* out,
                                    void* workspace, size_t workspace_bytes, void* const* comm_bases_host, int world,
                                    int rank, int B, int S, int H, int I_local, int NH_local, int NKV_local, int D, float eps,
                                    ezb_stream_t stream) {
    EZB_REQUIRE(hidden && K_cache && V_cache && Wqkv_local && Wo_local && Wgu_local && Wd_local && out, "null pointer");
    TpLink base;
    if (int rc = make_tp_link(base, comm_bases_host, world, rank, B, H)) return rc;
    if (int rc = check_layer_args(B, S, H, I_local, NH_local, NKV_local, D)) return rc;
    if (int rc = check_tp_fused_shape(B, H, I_local, NH_local, NKV_local, D)) return rc;
    EZB_REQUIRE(aligned16(hidden) && aligned16(K_cache) && aligned16(V_cache) && aligned16(Wqkv_local) &&
                    aligned16(Wo_local) && aligned16(Wgu_local) && aligned16(Wd_local) && aligned16(out),
                "pointers must be 16-byte aligned");
    LayerWorkspace w = carve_layer_ws(workspace, B, S, H, I_local, NH_local, NKV_local, D);
    if (!workspace || workspace_bytes < w.total) {
        set_last_message("workspace missing or smaller than ezb_qwen3_decode_layer_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    chain_begin();
    if (B == 1 && w.mega) {
        // batch 1: the whole rank-local layer and both exchanges in one persistent kernel
        MegaArgs m = mega_args(static_cast<const bf16*>(hidden), static_cast<bf16*>(K_cache), static_cast<bf16*>(V_cache),
                               static_cast<const bf16*>(Wqkv_local), static_cast<const bf16*>(Wo_local),
                               static_cast<const bf16*>(Wgu_local), static_cast<const bf16*>(Wd_local), static_cast<bf16*>(out), w,
                               S, H, I_local, NH_local, NKV_local, D, eps, kPlainLayer);
        m.link = base;
        if (decode_mega_supported(m)) {
            EZB_CUDA_TRY(launch_decode_mega(m, st));
            return EZB_OK;
        }
    }
    if (int rc = run_layer_tp_fused(static_cast<const bf16*>(hidden), false, nullptr, w.x2, static_cast<bf16*>(K_cache),
                                    static_cast<bf16*>(V_cache), static_cast<const bf16*>(Wqkv_local),
                                    static_cast<const bf16*>(Wo_local), static_cast<const bf16*>(Wgu_local),
                                    static_cast<const bf16*>(Wd_local), w, base, B, S, H, I_local, NH_local, NKV_local, D, eps,
                                    kPlainLayer, st))
        return rc;
    return finish_tp_fused(w.x2, static_cast<bf16*>(out), base, B, H, st);
}

int ezb_qwen3_decode_stack(const void* hidden, void* out, const ezb_layer_t* layers, int n_layers, const void* rope_cos,
                           const void* rope_sin, int rope_position, const int* seq_lens, void* workspace,
                           size_t workspace_bytes, int B, int S, int H, int I, int NH, int NKV, int D, float eps,
                           ezb_stream_t stream) {
    return run_stack(hidden, out, layers, n_layers, rope_cos, rope_sin, rope_position, seq_lens, nullptr, 0, 0, 0, workspace,
                     workspace_bytes, B, S, H, I, NH, NKV, D, eps, stream);
}

int ezb_qwen3_decode_stack_paged(const void* hidden, void* out, const ezb_layer_t* layers, int n_layers, const void* rope_cos,
                                 const void* rope_sin, const int* seq_lens, const int* page_table, int page_size,
                                 int max_pages, int num_pages, void* workspace, size_t workspace_bytes, int B, int H, int I,
                                 int NH, int NKV, int D, float eps, ezb_stream_t stream) {
    EZB_REQUIRE(seq_lens && page_table && max_pages >= 1 && num_pages >= 1, "paged caches need seq_lens, a page table and the pool size");
    EZB_REQUIRE_SHAPE(page_shift_of(page_size) >= 0, "page_size must be a power of two >= 64");
    return run_stack(hidden, out, layers, n_layers, rope_cos, rope_sin, 0, seq_lens, page_table, page_shift_of(page_size),
                     max_pages, num_pages, workspace, workspace_bytes, B, max_pages * page_size, H, I, NH, NKV, D, eps, stream);
}

size_t ezb_qwen3_decode_stack_tp_fused_workspace_bytes(int B, int S, int H, int I_local, int NH_local, int NKV_local, int D) {
    if (check_layer_args(B, S, H, I_local, NH_local, NKV_local, D)) return 0;
    return carve_layer_ws(nullptr, B, S, H, I_local, NH_local, NKV_local, D).total + 4 * round256((size_t)B * H * sizeof(bf16));
}

int ezb_qwen3_decode_stack_tp_fused(const void* hidden, void* out, const ezb_layer_t* layers_local, int n_layers,
                                    const void* rope_cos, const void* rope_sin, int rope_position, const int* seq_lens,
                                    void* workspace, size_t workspace_bytes, void* const* comm_bases_host, int world, int rank,
                                    int B, int S, int H, int I_local, int NH_local, int NKV_local, int D, float eps,
                                    ezb_stream_t stream) {
    EZB_REQUIRE(hidden && out && layers_local && n_layers >= 1, "null pointer or no layers");
    EZB_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr) && rope_position >= 0, "rotary tables come as a pair; position >= 0");
    TpLink base;
    if (int rc = make_tp_link(base, comm_bases_host, world, rank, B, H)) return rc;
    if (int rc = check_layer_args(B, S, H, I_local, NH_local, NKV_local, D)) return rc;
    if (int rc = check_tp_fused_shape(B, H, I_local, NH_local, NKV_local, D)) return rc;
    EZB_REQUIRE(aligned16(hidden) && aligned16(out) && aligned16(rope_cos) && aligned16(rope_sin), "pointers must be 16-byte aligned");
    for (int l = 0; l < n_layers; ++l) {
        const ezb_layer_t& L = layers_local[l];
        EZB_REQUIRE(L.K_cache && L.V_cache && L.Wqkv && L.Wo && L.Wgu && L.Wd, "null pointer in a layer");
        EZB_REQUIRE(aligned16(L.K_cache) && aligned16(L.V_cache) && aligned16(L.Wqkv) && aligned16(L.Wo) && aligned16(L.Wgu) &&
                        aligned16(L.Wd) && aligned16(L.input_norm_w) && aligned16(L.post_norm_w) && aligned16(L.q_norm_w) &&
                        aligned16(L.k_norm_w),
                    "layer pointers must be 16-byte aligned");
    }
    LayerWorkspace w = carve_layer_ws(workspace, B, S, H, I_local, NH_local, NKV_local, D);
    const size_t hbytes = round256((size_t)B * H * sizeof(bf16));
    if (!workspace || workspace_bytes < w.total + 4 * hbytes) {
        set_last_message("workspace missing or smaller than ezb_qwen3_decode_stack_tp_fused_workspace_bytes()");
        return EZB_ERR_WORKSPACE;
    }
    unsigned char* extra = static_cast<unsigned char*>(workspace) + w.total;
    bf16* layer_in[2] = {reinterpret_cast<bf16*>(extra), reinterpret_cast<bf16*>(extra + hbytes)};
    bf16* x2[2] = {reinterpret_cast<bf16*>(extra + 2 * hbytes), reinterpret_cast<bf16*>(extra + 3 * hbytes)};
    // one position for all rows: hand the kernel that table row; per-row lengths: the table base, indexed by len-1
    const size_t row_off = seq_lens ? 0 : (size_t)rope_position * D;
    const bf16* cos_row = rope_cos ? static_cast<const bf16*>(rope_cos) + row_off : nullptr;
    const bf16* sin_row = rope_sin ? static_cast<const bf16*>(rope_sin) + row_off : nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    chain_begin();
    bool single_kernel = B == 1 && !seq_lens && w.mega;
    for (int l = 0; l < n_layers; ++l) {
        const ezb_layer_t& L = layers_local[l];
        LayerExtras ex;
        ex.input_norm_w = static_cast<const bf16*>(L.input_norm_w), ex.post_norm_w = static_cast<const bf16*>(L.post_norm_w);
        ex.q_norm_w = static_cast<const bf16*>(L.q_norm_w), ex.k_norm_w = static_cast<const bf16*>(L.k_norm_w);
        ex.rope_cos = cos_row, ex.rope_sin = sin_row;
        ex.seq_lens = seq_lens, ex.rope_by_len = seq_lens ? 1 : 0;
        ex.next_Wqkv = (l + 1 < n_layers) ? static_cast<const bf16*>(layers_local[l + 1].Wqkv) : nullptr;
        if (single_kernel) {
            // batch 1: one persistent kernel per layer, complete output of layer l in layer_in[l & 1] (the last in out)
            const bf16* in = l == 0 ? static_cast<const bf16*>(hidden) : layer_in[(l - 1) & 1];
            bf16* dst = l + 1 == n_layers ? static_cast<bf16*>(out) : layer_in[l & 1];
            MegaArgs m = mega_args(in, static_cast<bf16*>(L.K_cache), static_cast<bf16*>(L.V_cache), static_cast<const bf16*>(L.Wqkv),
                                   static_cast<const bf16*>(L.Wo), static_cast<const bf16*>(L.Wgu), static_cast<const bf16*>(L.Wd), dst,
                                   w, S, H, I_local, NH_local, NKV_local, D, eps, ex);
            m.link = base;
            if (decode_mega_supported(m)) {  // same answer for every layer: the sizes do not change
                EZB_CUDA_TRY(launch_decode_mega(m, st));
                if (l + 1 == n_layers) return EZB_OK;
                continue;
            }
            single_kernel = false;
        }
        // layer l > 0 reads x2 of layer l-1 and folds that layer's second sum into its own QKV prologue
        const bf16* x_prev = l == 0 ? static_cast<const bf16*>(hidden) : x2[(l - 1) & 1];
        if (int rc = run_layer_tp_fused(x_prev, l > 0, layer_in[l & 1], x2[l & 1], static_cast<bf16*>(L.K_cache),
                                        static_cast<bf16*>(L.V_cache), static_cast<const bf16*>(L.Wqkv),
                                        static_cast<const bf16*>(L.Wo), static_cast<const bf16*>(L.Wgu),
                                        static_cast<const bf16*>(L.Wd), w, base, B, S, H, I_local, NH_local, NKV_local, D, eps, ex, st))
            return rc;
    }
    return finish_tp_fused(x2[(n_layers - 1) & 1], static_cast<bf16*>(out), base, B, H, st);
}

int ezb_residual_add_f32(const void* x2, const float* summed_d, void* out, int B, int H, ezb_stream_t stream) {
    EZB_REQUIRE(x2 && summed_d && out, "null pointer");
    EZB_REQUIRE(B >= 1 && H >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(H % 8 == 0, "hidden_size must be divisible by 8");
    EZB_REQUIRE(aligned16(x2) && aligned16(summed_d) && aligned16(out), "pointers must be 16-byte aligned");
    RowPrepArgs a;
    a.x = static_cast<const bf16*>(x2), a.ldx = H;
    a.add = summed_d, a.ldadd = H;
    a.sum_out = static_cast<bf16*>(out), a.ldsum = H;
    a.rows = B, a.dim = H, a.normalize = 0;
    chain_begin();
    EZB_CUDA_TRY(launch_row_prep(a, stream));
    return EZB_OK;
}

}  // extern "C"
