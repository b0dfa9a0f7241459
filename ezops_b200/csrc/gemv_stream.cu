// Weight-streaming GEMV / skinny GEMM for decode:  Y[b, n] = epi( sum_k X[b, k] * W[n, k] ),
// 1 <= b <= 64, W bf16 row-major, fp32 accumulation.
//
// The kernel is bound by reading W from HBM exactly once, so it is built around
// keeping many bytes in flight per SM with few instructions:
//   * persistent grid, one CTA per SM; CTA c owns a contiguous range of output
//     rows balanced to +-1 row, walked in blocks of 16 rows;
//   * one producer warp streams [16 rows x kc] weight tiles into a ring of
//     shared-memory stages with 1-D bulk TMA copies (one copy per row segment,
//     rows padded by 16 bytes so that ldmatrix is bank-conflict free), completion
//     counted on an mbarrier per stage; consumers hand stages back through a
//     second mbarrier per stage;
//   * eight consumer warps split the k range of every stage between them and
//     feed mma.sync m16n8k16 (weights as the 16-row A operand, activations as
//     the 8-wide B operand, batch padded to a multiple of 8), then combine
//     their partial tiles through shared memory in a fixed order, which keeps
//     results bit-reproducible from call to call;
//   * the activation block stays resident in shared memory when it fits (and
//     can then be RMS-normalised in the prologue); otherwise its k-chunks ride
//     along in every stage;
//   * programmatic dependent launch: the first weight stage is requested
//     before griddepcontrol.wait, because weights never depend on the kernel in
//     front; only then are activations read; once its own requests are out the
//     producer asks L2 for the head of the next kernel's weights.
// Every mbarrier wait is bounded (see mbar_wait_bounded).
//
// Two kernels share this structure:
//   gemv_rows8_kernel   batch <= 8 with the activations resident: the weights are
//                       the 8-wide B operand, so a stage is 8 whole weight rows
//                       (up to 4096 elements = 8 KB per bulk copy, the size at
//                       which the TMA unit reaches its streaming rate) and the
//                       batch rows form the A operand; template flags compile in
//                       the tensor-parallel exchange (LINK) and fix the batch-1
//                       activation staging at compile time (SINGLE);
//   gemv_stream_kernel  every other case (batch up to 64, activations streamed
//                       or resident): weights are the 16-row A operand, stages
//                       are [16 rows x kc].
#include "launchers.h"

namespace ezb {

#ifndef EZB_CONSUMER_WARPS
#define EZB_CONSUMER_WARPS 8
#endif
static constexpr int kConsumerWarps = EZB_CONSUMER_WARPS;
static constexpr int kConsumerThreads = kConsumerWarps * 32;
static constexpr int kGemvThreads = 32 + kConsumerThreads;
static constexpr int kMaxStages = 8;
static constexpr int kRowBlock = 16;
static constexpr int kHeaderBytes = 256;  // barriers + abort flag

struct GemvParams {
    const bf16* W0;
    const bf16* W1;
    long long ldw;
    int N, K, B;
    const bf16* x;
    long long ldx;
    const float* x_add;
    long long ldadd;
    bf16* x_sum_out;
    long long ldsum;
    const bf16* norm_w;
    float eps;
    int prologue, epilogue;
    const bf16* residual;
    long long ldres;
    void* out;
    long long ldout;
    int kc;        // k elements per stage (multiple of 16)
    int nstages;   // ring depth
    int prefetch;  // stages requested before the dependency wait
    int window;    // at most this many stages requested but not yet landed (0 = no limit)
    int evict_first;  // 1: weight rows are read with the L2 evict-first policy
    unsigned int* status;
    PrefetchList next;
    Trace trace;
    int trace_id;
    TpLink link;
};

__host__ __device__ constexpr size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <int NT, bool PAIR>
__host__ __device__ constexpr size_t red_bytes() {
    return (size_t)kConsumerWarps * (PAIR ? 2 : 1) * NT * 128 * sizeof(float);
}

// Rows of one stage: 16 (or 32 for gate/up pairs) weight rows, plus NT*8
// activation rows when the activations are streamed.
template <int NT, bool XRES, bool PAIR>
__host__ __device__ constexpr int stage_rows() {
    return kRowBlock * (PAIR ? 2 : 1) + (XRES ? 0 : NT * 8);
}


// Brings the activation block into shared memory (row stride xs_stride
// elements), optionally adding an fp32 term first and RMS-normalising:
// statistics in fp32, (x * r [* w]) in fp32, one rounding to bf16.  Called by
// all consumer threads; `scratch` needs one float per consumer warp.
// With PERMUTE32 every group of 32 elements is stored as four 16-byte blocks,
// block t holding the element pairs (j*8 + 2t, j*8 + 2t + 1), j = 0..3: exactly
// the four words that lane t of a quad feeds to two consecutive k-steps as its
// A fragments, so the rows8 kernel fetches them with one 128-bit load.
template <bool PERMUTE32>
__device__ __forceinline__ void store_x8(bf16* srow, int i, const uint32_t (&w)[4]) {
    if (!PERMUTE32) {
        *reinterpret_cast<uint4*>(srow + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
        uint32_t* base = reinterpret_cast<uint32_t*>(srow + (i >> 2) * 32);  // start of the 32-element group
        const int j = i & 3;
#pragma unroll
        for (int t = 0; t < 4; ++t) base[t * 4 + j] = w[t];
    }
}
// Half of store_x8: the 4 elements (two pairs) of half vector h = 2*i + (0 | 1).
template <bool PERMUTE32>
__device__ __forceinline__ void store_x4(bf16* srow, int h, const uint32_t (&w)[2]) {
    if (!PERMUTE32) {
        *reinterpret_cast<uint2*>(srow + h * 4) = make_uint2(w[0], w[1]);
    } else {
        const int i = h >> 1, t0 = (h & 1) * 2;
        uint32_t* base = reinterpret_cast<uint32_t*>(srow + (i >> 2) * 32);
        const int j = i & 3;
        base[t0 * 4 + j] = w[0];
        base[(t0 + 1) * 4 + j] = w[1];
    }
}
template <bool PERMUTE32>
__device__ __forceinline__ void load_x8(const bf16* srow, int i, uint32_t (&w)[4]) {
    if (!PERMUTE32) {
        const uint4 raw = *reinterpret_cast<const uint4*>(srow + i * 8);
        w[0] = raw.x, w[1] = raw.y, w[2] = raw.z, w[3] = raw.w;
    } else {
        const uint32_t* base = reinterpret_cast<const uint32_t*>(srow + (i >> 2) * 32);
        const int j = i & 3;
#pragma unroll
        for (int t = 0; t < 4; ++t) w[t] = base[t * 4 + j];
    }
}

template <bool PERMUTE32, bool LINK, bool SINGLE>
__device__ __forceinline__ void stage_activations(const GemvParams& p, bf16* xs, int xs_stride, float* scratch, int ct,
                                                  int cw, int lane, volatile int* abort_flag) {
    // independent 16-byte loads in flight per thread (16 spilled registers in the multi-row instances and was slower)
    constexpr int U = 8;
    const int nvec = p.K / 8;
    // Rows are staged side by side: the consumer warps are split into groups of `wpr` warps, one
    // group per batch row, so a batch of 8 rows costs the same number of L2 round trips and
    // barriers as one row (batch 1: all warps on the one row).
    // SINGLE (batch 1) fixes the split at compile time: all warps on row 0.
    int wpr = kConsumerWarps;
    if (!SINGLE)
        while (wpr > 1 && kConsumerWarps / wpr < p.B) wpr >>= 1;
    const int rows_per_pass = kConsumerWarps / wpr;
    const int sub = SINGLE ? ct : (cw % wpr) * 32 + lane, nthr = wpr * 32;
    const bool gather = LINK && p.link.world > 0 && p.link.gather_inbox >= 0;
    const unsigned int epoch = gather ? tp_next_epoch(p.link, p.link.gather_inbox) : 0u;
    const long long t0 = gather ? clock64() : 0;

    const int nrows = SINGLE ? 1 : p.B;
    for (int b0 = 0; b0 < nrows; b0 += rows_per_pass) {
        const int b = SINGLE ? 0 : b0 + cw / wpr;
        const bool active = SINGLE || b < nrows;
        const bf16* xrow = p.x + (long long)(active ? b : 0) * p.ldx;
        bf16* srow = xs + (size_t)(active ? b : 0) * xs_stride;
        float ssq = 0.f;
        if (LINK && active && gather) {
            // Fused tensor-parallel sum: x <- bf16(x + bf16(sum over ranks of the inbox slots)), see TpLink.
            // Two ranks: 8 elements per thread and step.  More ranks: 4 elements per step with all ranks
            // polled together, so the number of dependent L2 round trips does not grow with the world.
            if (!p.link.poll_all) {
                for (int i = sub; i < nvec; i += nthr) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(xrow + i * 8);
                    float add[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    // a gather that gave up (or a chain already poisoned) aborts the CTA: nothing is stored or pushed
                    const bool ok = !*abort_flag && tp_gather<2, 8>(p.link, epoch, (long long)b * p.K + i * 8, add, p.status, t0);
                    if (!ok) *abort_flag = 1;
                    uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        w4[e] = pack_bf16(bf16_lo(w4[e]) + round_bf16(add[2 * e]), bf16_hi(w4[e]) + round_bf16(add[2 * e + 1]));
                    if (ok && blockIdx.x == 0 && p.x_sum_out)
                        *reinterpret_cast<uint4*>(p.x_sum_out + (long long)b * p.ldsum + i * 8) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float lo = bf16_lo(w4[e]), hi = bf16_hi(w4[e]);
                        ssq += lo * lo + hi * hi;
                    }
                    store_x8<PERMUTE32>(srow, i, w4);
                }
            } else {
                for (int h = sub; h < 2 * nvec; h += nthr) {  // h: half vector (4 elements)
                    const uint2 raw = *reinterpret_cast<const uint2*>(xrow + h * 4);
                    float add[4] = {0.f, 0.f, 0.f, 0.f};
                    const bool ok = !*abort_flag && tp_gather<8, 4>(p.link, epoch, (long long)b * p.K + h * 4, add, p.status, t0);
                    if (!ok) *abort_flag = 1;
                    uint32_t w2[2] = {raw.x, raw.y};
#pragma unroll
                    for (int e = 0; e < 2; ++e)
                        w2[e] = pack_bf16(bf16_lo(w2[e]) + round_bf16(add[2 * e]), bf16_hi(w2[e]) + round_bf16(add[2 * e + 1]));
                    if (ok && blockIdx.x == 0 && p.x_sum_out)
                        *reinterpret_cast<uint2*>(p.x_sum_out + (long long)b * p.ldsum + h * 4) = make_uint2(w2[0], w2[1]);
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float lo = bf16_lo(w2[e]), hi = bf16_hi(w2[e]);
                        ssq += lo * lo + hi * hi;
                    }
                    store_x4<PERMUTE32>(srow, h, w2);
                }
            }
        } else if (active && p.prologue == PRO_ADD_RMSNORM) {
            constexpr int UA = 8;  // the fp32 term triples the registers per vector
            for (int base = 0; base < nvec; base += UA * nthr) {
                uint4 raw[UA];
                float4 add0[UA], add1[UA];
#pragma unroll
                for (int u = 0; u < UA; ++u) {
                    const int i = base + u * nthr + sub;
                    if (i < nvec) {
                        raw[u] = *reinterpret_cast<const uint4*>(xrow + i * 8);
                        add0[u] = *reinterpret_cast<const float4*>(p.x_add + (long long)b * p.ldadd + i * 8);
                        add1[u] = *reinterpret_cast<const float4*>(p.x_add + (long long)b * p.ldadd + i * 8 + 4);
                    }
                }
#pragma unroll
                for (int u = 0; u < UA; ++u) {
                    const int i = base + u * nthr + sub;
                    if (i < nvec) {
                        uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                        const float add[8] = {add0[u].x, add0[u].y, add0[u].z, add0[u].w, add1[u].x, add1[u].y, add1[u].z, add1[u].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            w[e] = pack_bf16(bf16_lo(w[e]) + round_bf16(add[2 * e]), bf16_hi(w[e]) + round_bf16(add[2 * e + 1]));
                        if (blockIdx.x == 0 && p.x_sum_out)
                            *reinterpret_cast<uint4*>(p.x_sum_out + (long long)b * p.ldsum + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float lo = bf16_lo(w[e]), hi = bf16_hi(w[e]);
                            ssq += lo * lo + hi * hi;
                        }
                        store_x8<PERMUTE32>(srow, i, w);
                    }
                }
            }
        } else if (active) {
            for (int base = 0; base < nvec; base += U * nthr) {
                // all loads of the batch are issued before any of them is used, so the
                // L2 latency is paid once per batch and not once per vector
                uint4 raw[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = base + u * nthr + sub;
                    if (i < nvec) raw[u] = *reinterpret_cast<const uint4*>(xrow + i * 8);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = base + u * nthr + sub;
                    if (i < nvec) {
                        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float lo = bf16_lo(w[e]), hi = bf16_hi(w[e]);
                            ssq += lo * lo + hi * hi;
                        }
                        store_x8<PERMUTE32>(srow, i, w);
                    }
                }
            }
        }
        if (p.prologue != PRO_NONE) {
            ssq = warp_sum(ssq);
            if (lane == 0) scratch[cw] = ssq;
            named_bar_sync(1, kConsumerThreads);
            if (active) {
                float tot = 0.f;
                for (int w = 0; w < wpr; ++w) tot += scratch[(cw / wpr) * wpr + w];  // fixed order: reproducible
                const float r = 1.0f / sqrtf(tot / (float)p.K + p.eps);
                // every thread rescales exactly the vectors it stored itself: no barrier in between
                for (int i = sub; i < nvec; i += nthr) {
                    uint32_t w[4];
                    load_x8<PERMUTE32>(srow, i, w);
                    uint32_t nw[4] = {0u, 0u, 0u, 0u};
                    if (p.norm_w) {
                        const uint4 q = *reinterpret_cast<const uint4*>(p.norm_w + i * 8);
                        nw[0] = q.x, nw[1] = q.y, nw[2] = q.z, nw[3] = q.w;
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float lo = bf16_lo(w[e]) * r, hi = bf16_hi(w[e]) * r;
                        if (p.norm_w) lo *= bf16_lo(nw[e]), hi *= bf16_hi(nw[e]);
                        w[e] = pack_bf16(lo, hi);
                    }
                    store_x8<PERMUTE32>(srow, i, w);
                }
            }
            if (b0 + rows_per_pass < nrows) named_bar_sync(1, kConsumerThreads);  // scratch is reused by the next pass
        }
    }
    named_bar_sync(1, kConsumerThreads);
}

// One output element: rounding points follow the torch reference's bf16 staging.
__device__ __forceinline__ void store_output(const GemvParams& p, int b, int n, float v0, float v1) {
    const long long o = (long long)b * p.ldout + n;
    if (p.epilogue == EPI_STORE_F32) {
        reinterpret_cast<float*>(p.out)[o] = v0;
    } else if (p.epilogue == EPI_RESIDUAL) {
        const float res = __bfloat162float(p.residual[(long long)b * p.ldres + n]);
        reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(res + round_bf16(v0));
    } else if (p.epilogue == EPI_SWIGLU) {
        const float gate = round_bf16(v0), up = round_bf16(v1);
        reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(round_bf16(silu_f32(gate)) * up);
    } else {
        reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(v0);
    }
}

// Producer's exit path after an abort: wait (bounded) until nothing is still in
// flight towards this CTA's shared memory.
__device__ __forceinline__ void drain_after_abort(uint64_t* full_bar, int NS, int issued, unsigned int* status) {
    const int first = max(0, issued - NS);
    for (int it = first; it < issued; ++it) {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&full_bar[it % NS]), (uint32_t)((it / NS) & 1))) {
            if (clock64() - t0 > kWaitLimitCycles) {
                report_fault(status, FAULT_GEMV_DRAIN);
                break;
            }
        }
    }
}

template <int NT, bool XRES, bool PAIR>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_stream_kernel(const GemvParams p) {
    constexpr int M = PAIR ? 2 : 1;
    constexpr int WROWS = kRowBlock * M;
    extern __shared__ __align__(128) unsigned char smem[];

    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = full_bar + kMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
    float* red = reinterpret_cast<float*>(smem + kHeaderBytes);
    bf16* xs = reinterpret_cast<bf16*>(smem + kHeaderBytes + red_bytes<NT, PAIR>());
    const int xs_stride = p.K + 8;  // elements; (K+8)*2 bytes keeps rows 16-byte aligned and 4 banks apart
    const size_t xs_bytes = XRES ? align_up((size_t)p.B * xs_stride * sizeof(bf16), 128) : 0;
    unsigned char* stage_base = smem + kHeaderBytes + red_bytes<NT, PAIR>() + xs_bytes;
    const int ws_stride = p.kc + 8;  // elements
    const uint32_t stage_bytes = (uint32_t)align_up((size_t)stage_rows<NT, XRES, PAIR>() * ws_stride * sizeof(bf16), 128);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int NS = p.nstages;

    const int r0 = (int)((long long)p.N * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.N * (blockIdx.x + 1) / gridDim.x);
    const int nrb = (r1 - r0 + kRowBlock - 1) / kRowBlock;
    const int nkc = (p.K + p.kc - 1) / p.kc;
    const int total = nrb * nkc;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // Arms the stage's barrier with the byte count of everything that will
        // land in it, then requests the weight rows (lanes 0..WROWS-1, one row
        // segment each).
        const unsigned long long w_policy = p.evict_first ? l2_evict_first_policy() : 0ull;
        auto request_weights = [&](int it) {
            const int rb = it / nkc, kci = it - rb * nkc, s = it % NS;
            const int k0 = kci * p.kc;
            const int len = min(p.kc, p.K - k0);
            const int row0 = r0 + rb * kRowBlock;
            const int nr = min(kRowBlock, r1 - row0);
            const uint32_t bar = smem_u32(&full_bar[s]);
            const uint32_t bytes = (uint32_t)((nr * M + (XRES ? 0 : p.B)) * len * (int)sizeof(bf16));
            if (lane == 0) mbar_arrive_expect_tx(bar, bytes);
            __syncwarp();
            if (lane < WROWS) {
                const int m = lane / kRowBlock, r = lane % kRowBlock;
                if (r < nr) {
                    const bf16* src = (m ? p.W1 : p.W0) + (long long)(row0 + r) * p.ldw + k0;
                    const uint32_t dst = smem_u32(stage_base + (size_t)s * stage_bytes) +
                                         (uint32_t)((m * kRowBlock + r) * ws_stride * (int)sizeof(bf16));
                    bulk_g2s(dst, src, (uint32_t)(len * (int)sizeof(bf16)), bar, w_policy);
                }
            }
        };
        auto request_activations = [&](int it) {
            if (XRES) return;
            const int rb = it / nkc, kci = it - rb * nkc, s = it % NS;
            const int k0 = kci * p.kc;
            const int len = min(p.kc, p.K - k0);
            const uint32_t bar = smem_u32(&full_bar[s]);
            for (int b = lane; b < p.B; b += 32) {
                const bf16* src = p.x + (long long)b * p.ldx + k0;
                const uint32_t dst = smem_u32(stage_base + (size_t)s * stage_bytes) +
                                     (uint32_t)((WROWS + b) * ws_stride * (int)sizeof(bf16));
                bulk_g2s(dst, src, (uint32_t)(len * (int)sizeof(bf16)), bar);
            }
        };

        const int npre = min(min(p.prefetch, NS), total);
        for (int it = 0; it < npre; ++it) request_weights(it);
        pdl_wait();
        for (int it = 0; it < npre; ++it) request_activations(it);
        int issued = npre;
        for (int it = npre; it < total; ++it) {
            const int s = it % NS;
            const uint32_t parity = (uint32_t)(((it / NS) & 1) ^ 1);
            if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), parity, abort_flag, p.status, FAULT_GEMV_EMPTY_WAIT)) break;
            request_weights(it);
            request_activations(it);
            issued = it + 1;
        }
        // Leave only when nothing is still in flight towards this CTA's shared
        // memory.  On the normal path the consumers have already waited for
        // every stage, so these waits return at once.
        if (*abort_flag) drain_after_abort(full_bar, NS, issued, p.status);
        else prefetch_next_operands(p.next, lane, blockIdx.x, gridDim.x);
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int cw = warp - 1;
    const int ct = tid - 32;  // 0..127 among consumer threads
    pdl_wait();

    if (XRES) stage_activations<false, false, false>(p, xs, xs_stride, red, ct, cw, lane, abort_flag);

    const int g4 = lane >> 2, t4 = lane & 3;
    for (int rb = 0; rb < nrb; ++rb) {
        float acc[M][NT][4];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][j][e] = 0.f;

        for (int kci = 0; kci < nkc; ++kci) {
            const int it = rb * nkc + kci;
            const int s = it % NS;
            mbar_wait_bounded(smem_u32(&full_bar[s]), (uint32_t)((it / NS) & 1), abort_flag, p.status, FAULT_GEMV_FULL_WAIT);
            const int k0 = kci * p.kc;
            const int len = min(p.kc, p.K - k0);
            const int nks = len >> 4;
            const unsigned char* st = stage_base + (size_t)s * stage_bytes;
            const uint32_t a_base = smem_u32(st) + (uint32_t)(((lane & 15) * ws_stride + (lane >> 4) * 8) * (int)sizeof(bf16));
            for (int ks = cw; ks < nks; ks += kConsumerWarps) {
                uint32_t a[M][4];
#pragma unroll
                for (int m = 0; m < M; ++m)
                    ldsm_x4(a_base + (uint32_t)((m * kRowBlock * ws_stride + ks * 16) * (int)sizeof(bf16)), a[m][0], a[m][1],
                            a[m][2], a[m][3]);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int b = j * 8 + g4;
                    uint32_t b0 = 0u, b1 = 0u;
                    if (b < p.B) {
                        const bf16* xb = XRES ? (xs + (size_t)b * xs_stride + k0 + ks * 16 + t4 * 2)
                                              : (reinterpret_cast<const bf16*>(st) + (size_t)(WROWS + b) * ws_stride + ks * 16 + t4 * 2);
                        b0 = *reinterpret_cast<const uint32_t*>(xb);
                        b1 = *reinterpret_cast<const uint32_t*>(xb + 8);
                    }
#pragma unroll
                    for (int m = 0; m < M; ++m) mma_bf16_16816(acc[m][j], a[m][0], a[m][1], a[m][2], a[m][3], b0, b1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
        }

        // Combine the four warps' partial tiles (fixed order) and apply the epilogue.
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int j = 0; j < NT; ++j)
                *reinterpret_cast<float4*>(red + ((size_t)((cw * M + m) * NT + j) * 32 + lane) * 4) =
                    make_float4(acc[m][j][0], acc[m][j][1], acc[m][j][2], acc[m][j][3]);
        named_bar_sync(1, kConsumerThreads);
        if (ct < 128) {
            const int fl = ct >> 2, e = ct & 3;
            const int row = (fl >> 2) + ((e >= 2) ? 8 : 0);
            const int col = (fl & 3) * 2 + (e & 1);
            const int n = r0 + rb * kRowBlock + row;
            const bool live = (n < r1) && !(*abort_flag);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int b = j * 8 + col;
                float v[M];
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float sum = 0.f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; ++w) sum += red[(size_t)((w * M + m) * NT + j) * 128 + ct];
                    v[m] = sum;
                }
                if (live && b < p.B) store_output(p, b, n, v[0], v[M - 1]);
            }
        }
        named_bar_sync(1, kConsumerThreads);
    }
}


// ---------------------------------------------------------------------------
// Small-batch kernel (batch <= 8, activations resident).
//
// A stage holds 8 weight rows (4 gate + 4 up rows in PAIR mode) of up to 4096
// elements each, one bulk copy per row.  ldmatrix.x4 on 8 rows x 32 k gives the
// B fragments of two k-steps; the activations (batch rows 0..7 of the 16-row A
// tile, rows 8..15 are zero) come from shared memory as 32-bit loads.  The C
// tile is [batch x 8 weight rows]; two accumulator chains per warp.
// ---------------------------------------------------------------------------
static constexpr int kRows8 = 8;
static constexpr int kXsPad8 = 32;  // activation rows 64 bytes apart in bank space: 128-bit loads of a quarter warp never collide
static constexpr int kRed8Bytes = 2 * kConsumerWarps * 64 * (int)sizeof(float);  // double buffered
static constexpr int kResidualSlots = 1024;  // residual values (batch x rows of this CTA) kept in shared memory

// LINK: the instance used by the fused tensor-parallel layer (prologue gathers from the inbox,
// epilogue pushes to the peers).  The plain instance contains none of that code.
template <bool PAIR, bool LINK, bool SINGLE>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_rows8_kernel(const GemvParams p) {
    constexpr int UNITS = PAIR ? 4 : 8;  // outputs per row block
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = full_bar + kMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
    float* red = reinterpret_cast<float*>(smem + kHeaderBytes);
    float* res_s = reinterpret_cast<float*>(smem + kHeaderBytes + kRed8Bytes);
    bf16* xs = reinterpret_cast<bf16*>(smem + kHeaderBytes + kRed8Bytes + kResidualSlots * sizeof(float));
    const int xs_stride = p.K + kXsPad8;
    const size_t xs_bytes = align_up((size_t)p.B * xs_stride * sizeof(bf16), 128);
    unsigned char* stage_base = reinterpret_cast<unsigned char*>(xs) + xs_bytes;
    const int ws_stride = p.kc + 8;
    const uint32_t stage_bytes = (uint32_t)align_up((size_t)kRows8 * ws_stride * sizeof(bf16), 128);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int NS = p.nstages;
    const int r0 = (int)((long long)p.N * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.N * (blockIdx.x + 1) / gridDim.x);
    const int nrb = (r1 - r0 + UNITS - 1) / UNITS;
    const int nkc = (p.K + p.kc - 1) / p.kc;
    const int total = nrb * nkc;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    unsigned long long* trec = (tid == 32) ? trace_open(p.trace, (unsigned)p.trace_id, blockIdx.x) : nullptr;
    __syncthreads();
    pdl_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        const unsigned long long w_policy = p.evict_first ? l2_evict_first_policy() : 0ull;
        auto request = [&](int it) {
            const int rb = it / nkc, kci = it - rb * nkc, s = it % NS;
            const int k0 = kci * p.kc;
            const int len = min(p.kc, p.K - k0);
            const int unit0 = r0 + rb * UNITS;
            const int nu = min(UNITS, r1 - unit0);
            const uint32_t bar = smem_u32(&full_bar[s]);
            if (lane == 0) mbar_arrive_expect_tx(bar, (uint32_t)(nu * (PAIR ? 2 : 1) * len * (int)sizeof(bf16)));
            __syncwarp();
            if (lane < kRows8) {
                const int m = PAIR ? (lane >> 2) : 0;
                const int u = PAIR ? (lane & 3) : lane;
                if (u < nu) {
                    const bf16* src = (m ? p.W1 : p.W0) + (long long)(unit0 + u) * p.ldw + k0;
                    const uint32_t dst = smem_u32(stage_base + (size_t)s * stage_bytes) + (uint32_t)(lane * ws_stride * (int)sizeof(bf16));
                    bulk_g2s(dst, src, (uint32_t)(len * (int)sizeof(bf16)), bar, w_policy);
                }
            }
        };
        // `window` (0 = off) bounds how many stages may be requested but not yet
        // landed: requests that are outstanding together complete together.
        auto landed = [&](int it) {
            return mbar_wait_bounded(smem_u32(&full_bar[it % NS]), (uint32_t)((it / NS) & 1), abort_flag, p.status,
                                     FAULT_GEMV_FULL_WAIT);
        };
        const int W = p.window;
        // Weights never depend on the kernel in front: fill the ring first.
        const int npre = min(min(p.prefetch, NS), total);
        bool ok = true;
        for (int it = 0; it < npre && ok; ++it) {
            if (W > 0 && it >= W) ok = landed(it - W);
            if (ok) request(it);
        }
        pdl_wait();
        int issued = ok ? npre : 0;
        for (int it = npre; it < total && ok; ++it) {
            const int s = it % NS;
            const uint32_t parity = (uint32_t)(((it / NS) & 1) ^ 1);
            if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), parity, abort_flag, p.status, FAULT_GEMV_EMPTY_WAIT)) break;
            if (W > 0 && it >= W && !landed(it - W)) break;
            request(it);
            issued = it + 1;
        }
        if (*abort_flag) drain_after_abort(full_bar, NS, issued, p.status);
        else prefetch_next_operands(p.next, lane, blockIdx.x, gridDim.x);
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int cw = warp - 1;
    const int ct = tid - 32;
    pdl_wait();
    trace_mark(trec, 3);
    // The residual values this CTA will add are fetched now, together with the
    // activations, so that no epilogue waits on a global load.
    const int rows_here = r1 - r0;
    const bool res_in_smem = p.epilogue == EPI_RESIDUAL && p.B * rows_here <= kResidualSlots;
    if (res_in_smem)
        for (int i = ct; i < p.B * rows_here; i += kConsumerThreads) {
            const int b = i / rows_here, r = i - b * rows_here;
            res_s[i] = __bfloat162float(p.residual[(long long)b * p.ldres + r0 + r]);
        }
    const unsigned int push_epoch = (LINK && p.link.world > 0 && p.link.push_inbox >= 0) ? tp_next_epoch(p.link, p.link.push_inbox) : 0u;
    if (LINK && p.link.world > 0 && tp_poisoned(p.status)) *abort_flag = 1;  // see tp_poisoned
    stage_activations<true, LINK, SINGLE>(p, xs, xs_stride, red, ct, cw, lane, abort_flag);  // ends with a barrier among the consumers

    const int g4 = lane >> 2, t4 = lane & 3;
    const bool has_row = g4 < p.B;
    const bf16* xrow = xs + (size_t)(has_row ? g4 : 0) * xs_stride + t4 * 8;  // permuted layout, see store_x8
    const uint32_t lds_off = (uint32_t)(((lane & 7) * ws_stride + (lane >> 3) * 8) * (int)sizeof(bf16));

    for (int rb = 0; rb < nrb; ++rb) {
        // Eight independent accumulator chains per warp (four 32-element groups in flight, two k-steps each): a
        // dependent mma.sync issues only after its predecessor has completed, and with two chains the warps spent
        // most of a stage waiting on that latency, which capped the kernel just above the HBM rate.
        float acc[8][4];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
        for (int kci = 0; kci < nkc; ++kci) {
            const int it = rb * nkc + kci;
            const int s = it % NS;
            mbar_wait_bounded(smem_u32(&full_bar[s]), (uint32_t)((it / NS) & 1), abort_flag, p.status, FAULT_GEMV_FULL_WAIT);
            if (it == 0) trace_mark(trec, 4);
            const int k0 = kci * p.kc;
            const int len = min(p.kc, p.K - k0);
            const int nk32 = len >> 5;
            const uint32_t w_base = smem_u32(stage_base + (size_t)s * stage_bytes) + lds_off;
            const bf16* xk = xrow + k0;
            int k32 = cw;
            for (; k32 + 3 * kConsumerWarps < nk32; k32 += 4 * kConsumerWarps) {
                uint32_t w[4][4];
                uint4 a[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    ldsm_x4(w_base + (uint32_t)((k32 + u * kConsumerWarps) * 32 * (int)sizeof(bf16)), w[u][0], w[u][1], w[u][2], w[u][3]);
                    a[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (has_row) a[u] = *reinterpret_cast<const uint4*>(xk + (k32 + u * kConsumerWarps) * 32);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    mma_bf16_16816(acc[2 * u], a[u].x, 0u, a[u].y, 0u, w[u][0], w[u][1]);
                    mma_bf16_16816(acc[2 * u + 1], a[u].z, 0u, a[u].w, 0u, w[u][2], w[u][3]);
                }
            }
            for (; k32 < nk32; k32 += kConsumerWarps) {
                uint32_t w0, w1, w2, w3;
                ldsm_x4(w_base + (uint32_t)(k32 * 32 * (int)sizeof(bf16)), w0, w1, w2, w3);
                uint4 a = make_uint4(0u, 0u, 0u, 0u);
                if (has_row) a = *reinterpret_cast<const uint4*>(xk + k32 * 32);
                mma_bf16_16816(acc[0], a.x, 0u, a.y, 0u, w0, w1);
                mma_bf16_16816(acc[1], a.z, 0u, a.w, 0u, w2, w3);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));
        }
        // fixed summation order over the chains
        const float sum0 = ((acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0])) + ((acc[4][0] + acc[5][0]) + (acc[6][0] + acc[7][0]));
        const float sum1 = ((acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1])) + ((acc[4][1] + acc[5][1]) + (acc[6][1] + acc[7][1]));
        // rows 0..7 of the C tile are the batch; this thread holds (batch g4, weight rows 2*t4, 2*t4+1).
        // The reduction buffer alternates between row blocks, so one barrier per block is enough.
        float* redb = red + (rb & 1) * (kConsumerWarps * 64);
        *reinterpret_cast<float2*>(redb + cw * 64 + g4 * 8 + t4 * 2) = make_float2(sum0, sum1);
        named_bar_sync(1, kConsumerThreads);
        if (ct < 64) {
            const int b = ct >> 3, j = ct & 7;
            const int n = r0 + rb * UNITS + j;
            if (j < UNITS && n < r1 && b < p.B && !(*abort_flag)) {
                float v0 = 0.f, v1 = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {
                    v0 += redb[w * 64 + b * 8 + j];
                    if (PAIR) v1 += redb[w * 64 + b * 8 + j + 4];
                }
                if (res_in_smem) {
                    const float res = res_s[b * rows_here + (n - r0)];
                    reinterpret_cast<bf16*>(p.out)[(long long)b * p.ldout + n] = __float2bfloat16_rn(res + round_bf16(v0));
                } else if (LINK && p.epilogue == EPI_PUSH_F32) {
                    // this rank's partial goes into its slot of the inbox on every rank
                    tp_push(p.link, (long long)b * p.ldout + n, v0, push_epoch);
                } else {
                    store_output(p, b, n, v0, v1);
                }
            }
        }
    }
    if (LINK && p.link.world > 0 && p.link.bump_inbox >= 0 && blockIdx.x == 0 && ct == 0 && !*abort_flag) tp_bump(p.link);
    trace_mark(trec, 5);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
struct GemvPlan {
    int NT;
    bool xres;
    int kc, nstages, prefetch, grid;
    size_t smem;
};

static int pick_nt(int B) { return B <= 8 ? 1 : (B <= 16 ? 2 : (B <= 32 ? 4 : 8)); }

// Resident activations are worth it while they leave room for a useful ring.
static bool x_fits_resident(int B, int K) { return (size_t)B * (K + 8) * 2 <= 72 * 1024 && B <= 8; }

bool gemv_needs_scratch(int B, int K) { return !x_fits_resident(B, K); }


PrefetchPlan prefetch_plan_rows(const bf16* W0, const bf16* W1, int N, int K, int cap_rows, int skip_rows) {
    PrefetchPlan pf;
    pf.skip_units = skip_rows;
    pf.base[0] = W0, pf.base[1] = W1;
    pf.unit_bytes = (long long)K * 2;
    pf.units = N;
    pf.next_grid = sm_count() < N ? sm_count() : N;
    pf.cap_units = cap_rows;
    return pf;
}

PrefetchPlan prefetch_plan_flat(const void* a, const void* b, size_t bytes_each) {
    PrefetchPlan pf;
    pf.base[0] = a, pf.base[1] = b;
    pf.unit_bytes = 4096;
    pf.units = (int)(bytes_each / 4096);
    pf.next_grid = sm_count();
    pf.cap_units = 1 << 30;
    pf.skip_units = 0;
    return pf;
}

static GemvPlan plan_gemv(const GemvArgs& a, bool pair) {
    GemvPlan pl;
    pl.NT = pick_nt(a.B);
    pl.xres = x_fits_resident(a.B, a.K);
    const int M = pair ? 2 : 1;
    const int rows = kRowBlock * M + (pl.xres ? 0 : pl.NT * 8);
    int kc = tuning(EZB_TUNE_GEMV_KC);
    if (kc <= 0) {
        // about 32 KB per stage
        kc = (int)(32768 / (2 * rows)) - 8;
        kc = kc / 64 * 64;
        if (kc < 64) kc = 64;
        if (kc > 2048) kc = 2048;
    }
    kc = kc / 16 * 16;
    if (kc > a.K) kc = a.K;
    pl.kc = kc;
    const size_t stage = align_up((size_t)rows * (kc + 8) * 2, 128);
    const size_t red = (size_t)kConsumerWarps * M * pl.NT * 128 * 4;
    const size_t xs = pl.xres ? align_up((size_t)a.B * (a.K + 8) * 2, 128) : 0;
    const size_t fixed = kHeaderBytes + red + xs;
    size_t budget = (size_t)tuning(EZB_TUNE_GEMV_SMEM_KB) * 1024;
    const size_t cap = (size_t)max_smem_optin();
    if (budget > cap) budget = cap;
    int ns = budget > fixed ? (int)((budget - fixed) / stage) : 0;
    if (ns < 2) ns = 2;
    if (ns > kMaxStages) ns = kMaxStages;
    while (ns > 2 && fixed + (size_t)ns * stage > cap) --ns;
    pl.nstages = ns;
    int pf = tuning(EZB_TUNE_GEMV_PREFETCH);
    pl.prefetch = (pf <= 0 || pf > ns) ? ns : pf;
    pl.smem = fixed + (size_t)ns * stage;
    int grid = sm_count() * max(1, tuning(EZB_TUNE_GEMV_CTAS_PER_SM));
    if (grid > a.N) grid = a.N;
    pl.grid = grid;
    return pl;
}

template <int NT, bool XRES, bool PAIR>
static cudaError_t launch_instance(const GemvParams& p, const GemvPlan& pl, cudaStream_t stream) {
    auto kernel = gemv_stream_kernel<NT, XRES, PAIR>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin());
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(pl.grid), dim3(kGemvThreads), pl.smem, stream, p);
}

template <bool XRES, bool PAIR>
static cudaError_t dispatch_nt(const GemvParams& p, const GemvPlan& pl, cudaStream_t stream) {
    switch (pl.NT) {
        case 1: return launch_instance<1, XRES, PAIR>(p, pl, stream);
        case 2: return launch_instance<2, XRES, PAIR>(p, pl, stream);
        case 4: return launch_instance<4, XRES, PAIR>(p, pl, stream);
        default: return launch_instance<8, XRES, PAIR>(p, pl, stream);
    }
}


// Plan for the small-batch kernel; returns false when the shape is outside it.
static bool plan_rows8(const GemvArgs& a, GemvPlan& pl) {
    if (a.B > 8 || a.K % 32 != 0) return false;
    if ((size_t)a.B * (a.K + kXsPad8) * 2 > 72 * 1024) return false;  // keep room for a ring of whole rows
    const size_t cap = (size_t)max_smem_optin();
    const size_t xs = align_up((size_t)a.B * (a.K + kXsPad8) * 2, 128);
    const size_t fixed = kHeaderBytes + kRed8Bytes + kResidualSlots * sizeof(float) + xs;
    int best_kc = 0, best_ns = 0;
    int forced = tuning(EZB_TUNE_GEMV_KC);
    for (int kc = 4096; kc >= 256; kc >>= 1) {
        int k = kc > a.K ? a.K : kc;
        if (forced > 0) k = (forced > a.K ? a.K : forced) / 32 * 32;
        if (k < 32) k = 32;
        const size_t stage = align_up((size_t)kRows8 * (k + 8) * 2, 128);
        if (fixed + 2 * stage > cap) continue;
        int ns = (int)((cap - fixed) / stage);
        if (ns > kMaxStages) ns = kMaxStages;
        // the longest row piece that leaves a ring of two stages: at batch 8, where the activations take 66 KB, two
        // stages of 8 KB row pieces beat four stages of 4 KB pieces (layer 123.1 against 126.8 us) - the size of a
        // bulk copy matters more than the depth of the ring
        best_kc = k, best_ns = ns;
        break;
    }
    if (best_kc == 0) return false;
    pl.NT = 1, pl.xres = true, pl.kc = best_kc;
    const size_t stage = align_up((size_t)kRows8 * (best_kc + 8) * 2, 128);
    // no more stages than the longest CTA can use, and at most ~200 KB in flight
    int ns = best_ns;
    const int budget_ns = (int)(((size_t)tuning(EZB_TUNE_GEMV_SMEM_KB) * 1024 > fixed
                                     ? (size_t)tuning(EZB_TUNE_GEMV_SMEM_KB) * 1024 - fixed : 0) / stage);
    if (budget_ns >= 2 && budget_ns < ns) ns = budget_ns;
    pl.nstages = ns;
    int pf = tuning(EZB_TUNE_GEMV_PREFETCH);
    pl.prefetch = (pf <= 0 || pf > ns) ? ns : pf;
    pl.smem = fixed + (size_t)ns * stage;
    int grid = sm_count() * max(1, tuning(EZB_TUNE_GEMV_CTAS_PER_SM));
    const int units = a.N;
    if (grid > units) grid = units;
    pl.grid = grid;
    return true;
}

bool gemv_small_batch_eligible(int B, int K) {
    if (tuning(EZB_TUNE_GEMV_ROWS8) == 0) return false;
    GemvArgs a;
    a.B = B, a.K = K, a.N = 1 << 20;
    GemvPlan pl;
    return plan_rows8(a, pl);
}

template <bool PAIR, bool LINK, bool SINGLE>
static cudaError_t launch_rows8(const GemvParams& p, const GemvPlan& pl, cudaStream_t stream) {
    auto kernel = gemv_rows8_kernel<PAIR, LINK, SINGLE>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin());
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(pl.grid), dim3(kGemvThreads), pl.smem, stream, p);
}

cudaError_t launch_gemv(const GemvArgs& a, cudaStream_t stream) {
    const bool pair = a.epilogue == EPI_SWIGLU;
    GemvPlan pl;
    const bool rows8 = tuning(EZB_TUNE_GEMV_ROWS8) != 0 && plan_rows8(a, pl);
    if (!rows8) pl = plan_gemv(a, pair);

    GemvParams p;
    p.W0 = a.W0, p.W1 = a.W1, p.ldw = a.ldw;
    p.N = a.N, p.K = a.K, p.B = a.B;
    p.x = a.x, p.ldx = a.ldx;
    p.x_add = a.x_add, p.ldadd = a.ldadd;
    p.x_sum_out = a.x_sum_out, p.ldsum = a.ldsum;
    p.norm_w = a.norm_w, p.eps = a.eps;
    p.prologue = a.prologue, p.epilogue = a.epilogue;
    p.residual = a.residual, p.ldres = a.ldres;
    p.out = a.out, p.ldout = a.ldout;
    p.kc = pl.kc, p.nstages = pl.nstages, p.prefetch = pl.prefetch;
    p.window = tuning(EZB_TUNE_GEMV_WINDOW);
    p.evict_first = tuning(EZB_TUNE_STREAM_EVICT_FIRST) ? 1 : 0;
    p.status = status_ptr();
    if (!p.status) return cudaErrorUnknown;
    p.next = a.next;
    if (!tuning(EZB_TUNE_L2_PREFETCH)) p.next.plan[0].units = p.next.plan[1].units = 0;
    p.trace = trace_handle();
    p.trace_id = a.trace_id;
    p.link = a.link;

    const bool use_tc = !rows8 && a.tc_workspace && tuning(EZB_TUNE_TC) != 0 && gemm_tc_supported(a.B, a.K) && gemm_tc_fits(a.N, pair);
    // The fused tensor-parallel exchange lives in the small-batch kernel (gather and push) and, for larger
    // batches, in the row kernel (gather) and the tensor-core kernel (push); the general fallback has none.
    const bool linked = a.link.world > 0;
    const bool gathers = linked && a.link.gather_inbox >= 0;
    if (linked && !rows8 && !use_tc) return cudaErrorNotSupported;
    GemvArgs tc_args = a;
    if ((use_tc || !pl.xres) && a.prologue != PRO_NONE) {
        // The activation block is not resident in this path: run the prologue as
        // its own (tiny) kernel into the scratch rows, then stream those.
        RowPrepArgs rp;
        rp.x = a.x, rp.ldx = a.ldx;
        rp.add = (a.prologue == PRO_ADD_RMSNORM && !gathers) ? a.x_add : nullptr, rp.ldadd = a.ldadd;
        rp.sum_out = (a.prologue == PRO_ADD_RMSNORM) ? a.x_sum_out : nullptr, rp.ldsum = a.ldsum;
        if (gathers) {  // the term to add comes from the inbox; the projection itself then has nothing to gather
            rp.link = a.link, rp.link.push_inbox = -1, rp.link.bump_inbox = -1;
            tc_args.link.gather_inbox = -1;
            if (tc_args.link.push_inbox < 0 && tc_args.link.bump_inbox < 0) tc_args.link.world = 0;
        }
        rp.w = a.norm_w;
        rp.y = a.xn_scratch, rp.ldy = a.K;
        rp.rows = a.B, rp.dim = a.K, rp.eps = a.eps, rp.normalize = 1;
        cudaError_t e = launch_row_prep(rp, stream);
        if (e != cudaSuccess) return e;
        p.x = a.xn_scratch, p.ldx = a.K;
        p.prologue = PRO_NONE;
    }
    if (use_tc) return launch_gemm_tc(tc_args, p.x, p.ldx, a.tc_workspace, stream);

    if (rows8) {
        const int which = (pair ? 4 : 0) | (a.link.world > 0 ? 2 : 0) | (a.B == 1 ? 1 : 0);
        switch (which) {
            case 0: return launch_rows8<false, false, false>(p, pl, stream);
            case 1: return launch_rows8<false, false, true>(p, pl, stream);
            case 2: return launch_rows8<false, true, false>(p, pl, stream);
            case 3: return launch_rows8<false, true, true>(p, pl, stream);
            case 4: return launch_rows8<true, false, false>(p, pl, stream);
            case 5: return launch_rows8<true, false, true>(p, pl, stream);
            case 6: return launch_rows8<true, true, false>(p, pl, stream);
            default: return launch_rows8<true, true, true>(p, pl, stream);
        }
    }
    if (pl.xres) return pair ? dispatch_nt<true, true>(p, pl, stream) : dispatch_nt<true, false>(p, pl, stream);
    return pair ? dispatch_nt<false, true>(p, pl, stream) : dispatch_nt<false, false>(p, pl, stream);
}

}  // namespace ezb
