// ezb_attn_decode_static: decode attention for callers that cannot allocate
// device memory.
//
// The regular entry point, ezb_attn_decode, needs a caller-allocated workspace
// for the per-split partial results and the split counters.  Some callers have
// no way to provide one: a plugin that runs inside a host framework which owns
// the whole device heap and hands the plugin nothing but its input and output
// buffers, or a latency-critical serving loop in which a cudaMalloc (it
// synchronises the device) is not acceptable.  For them this file keeps the
// scratch in a fixed array that is part of the library image: every GPU that
// loads the library carries kStaticScratchBytes of it until the process exits,
// and nothing is ever allocated or freed here -- no cudaMalloc, no cudaFree, no
// allocating library call.
//
// What a caller has to know:
//   * Shapes whose scratch need (ezb_attn_decode_workspace_bytes) exceeds
//     kStaticScratchBytes are refused with EZB_ERR_WORKSPACE and a message
//     that names both numbers.
//   * The first call on each device looks the array's device address up
//     (cudaGetSymbolAddress with that device current) and keeps it; make that
//     first call outside of any stream capture.
//   * All calls on a device share the one array, and it still holds whatever
//     the previous call left there.  The part that must start at zero (the split
//     counters) is cleared on `stream` before each launch.  Two calls that can
//     overlap on the GPU (different streams, or one graph launched twice at
//     once) race on the array: serialise them.
#include <cstdio>
#include <mutex>

#include "launchers.h"

namespace ezb {

static constexpr size_t kStaticScratchBytes = EZB_ATTN_STATIC_SCRATCH_BYTES;

// In host code this name is only a handle for the runtime's symbol lookup; it
// is NOT the device address.  Device code may name it directly.
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

static std::mutex g_scratch_mutex;
static void* g_scratch_addr[64] = {};  // per device, filled on first use

// Device address of the array on the current device, or null (message set).
static void* static_scratch_for_current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        if (e != cudaSuccess) set_last_cuda_error(e);
        else set_last_message("device ordinal outside the supported range");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_attn_static_scratch);
        if (e != cudaSuccess || !ptr) {
            set_last_cuda_error(e);
            return nullptr;
        }
        g_scratch_addr[dev] = ptr;
    }
    return g_scratch_addr[dev];
}

}  // namespace ezb

using namespace ezb;

extern "C" int ezb_attn_decode_static(const void* Q, const void* K, const void* V, void* Out, int B, int H, int NKV, int S,
                                      int D, const int* seq_lens_or_null, ezb_stream_t stream) {
    EZB_REQUIRE(Q && K && V && Out, "null pointer");
    EZB_REQUIRE(B >= 1 && H >= 1 && NKV >= 1 && S >= 1, "sizes must be positive");
    EZB_REQUIRE_SHAPE(D == 64 || D == 128, "head_dim must be 64 or 128");
    EZB_REQUIRE_SHAPE(H % NKV == 0, "num_heads must be divisible by num_kv_heads");
    EZB_REQUIRE_SHAPE(B <= 65535 && NKV <= 65535, "batch and kv heads are limited to 65535");
    EZB_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(Out), "Q, K, V and Out must be 16-byte aligned");
    const size_t need = attn_workspace_bytes(B, H, NKV, S, D);
    if (need > kStaticScratchBytes) {
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "this shape needs %zu bytes of scratch, the built-in array holds %zu; use ezb_attn_decode with a workspace",
                 need, kStaticScratchBytes);
        set_last_message(msg);
        return EZB_ERR_WORKSPACE;
    }
    void* scratch = static_scratch_for_current_device();
    if (!scratch) return EZB_ERR_CUDA;
    // the array keeps the previous call's contents: the counters must start at zero
    EZB_CUDA_TRY(cudaMemsetAsync(scratch, 0, attn_counters_bytes(B, H, NKV), stream));
    AttnArgs a;
    a.Q = static_cast<const bf16*>(Q), a.q_bstride = (long long)H * D;
    a.K = static_cast<const bf16*>(K), a.V = static_cast<const bf16*>(V);
    a.Out = static_cast<bf16*>(Out), a.o_bstride = (long long)H * D;
    a.seq_lens = seq_lens_or_null;
    a.B = B, a.H = H, a.NKV = NKV, a.S = S, a.D = D;
    a.workspace = scratch;
    chain_begin();
    EZB_CUDA_TRY(launch_attn_decode(a, stream));
    return EZB_OK;
}
