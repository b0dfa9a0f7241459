// Batched projections on the 5th-generation tensor cores:
//   Y[b, n] = epi( sum_k X[b, k] * W[n, k] ),   2 <= b <= 64,
// used once the batch turns the weight-streaming GEMV into a skinny GEMM.
//
// The weights are still read from HBM exactly once, so the kernel is built like
// the GEMV -- persistent CTAs, a deep TMA ring, programmatic dependent launch --
// but the arithmetic moves to tcgen05:
//   * "swap AB": a tile is 128 weight rows (the MMA's M) by the whole batch
//     (the MMA's N = 16, 32 or 64) and walks K in blocks of 64 elements;
//   * one elected thread issues cp.async.bulk.tensor (2-D tiled TMA, 128-byte
//     swizzle) for the W block [128 x 64] and the X block [N x 64] of a stage;
//     one elected thread issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32)
//     with the accumulator in tensor memory, and tcgen05.commit hands the stage
//     back to the producer when the MMAs that read it have retired;
//   * four epilogue warps read the accumulator with tcgen05.ld (thread = weight
//     row, registers = batch columns) and apply the same epilogues as the GEMV;
//     the accumulator is double buffered in tensor memory, so the epilogue of
//     one tile overlaps the MMAs of the next;
//   * work is split "stream-K": the (tile, k-block) units are dealt evenly to
//     the CTAs in order, whatever the matrix shape (a 4096-row matrix has only
//     32 tiles for 148 SMs).  A CTA that covers only part of a tile's K range
//     stores its fp32 partial tile in the workspace; the last contributor of the
//     tile (one atomic ticket, no waiting) adds the partials in CTA order, so
//     results are bit-reproducible.  A CTA works through its shared tiles first
//     and its whole tiles after them, so that fix-up overlaps their streaming.
//   * the LINK instance pushes its fp32 results into the tensor-parallel peers'
//     inboxes instead of storing them (see TpLink).
// Every mbarrier wait is bounded; on a time-out the CTA records a fault, stops
// issuing work, waits (bounded) for copies in flight, frees its tensor memory
// and returns.
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "launchers.h"

namespace ezb {

static constexpr int kTcRows = 128;     // weight rows per tile (MMA M)
static constexpr int kTcBlockK = 64;    // k elements per stage: 128 bytes, one swizzle row
static constexpr int kTcThreads = 192;  // TMA warp, MMA warp, four epilogue warps
static constexpr int kTcMaxStages = 10;
static constexpr int kTcMaxSegs = 32;  // tile segments per CTA: at most tiles / CTAs + 2
static constexpr int kTcABytes = kTcRows * kTcBlockK * 2;
// Projections of different shapes share one workspace, so the region of the
// ticket counters (which must stay zero between launches) has one fixed size
// and never overlaps the partial tiles of another projection.
static constexpr size_t kTcCounterBytes = 16384;
static constexpr int kTcMaxTiles = (int)(kTcCounterBytes / 4);

struct TcParams {
    int N, K, B;          // output units (rows, or gate/up pairs), reduction length, batch
    int tiles, kblocks;   // ceil(N / units per tile), ceil(K / 64)
    int nstages;
    int pair;             // 1: tile = 64 gate rows + 64 up rows, SwiGLU epilogue
    int epilogue;
    const bf16* residual;
    long long ldres;
    void* out;
    long long ldout;
    float* partial;          // [grid][2][NB][128] fp32 partial tiles
    unsigned int* counters;  // [tiles], zero between launches
    unsigned int* status;
    Trace trace;
    int trace_id;
    TpLink link;  // fused tensor-parallel exchange (world 0: none); only the push side lives in this kernel
};

// ---- tcgen05 / TMA wrappers -------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major bf16 tile whose rows are 128
// bytes (64 elements) with the 128-byte swizzle that the tiled TMA wrote:
// start address / 16, stride between 8-row groups 1024 bytes, descriptor
// version 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Instruction descriptor, kind::f16: fp32 accumulator, bf16 A and B, both
// K-major, N in units of 8 at bit 17, M in units of 16 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// First unit of CTA c when T units are dealt to G CTAs in order.
__device__ __forceinline__ long long tc_first_unit(long long T, int G, int c) { return T * c / G; }
// CTA that owns unit u.
__device__ __forceinline__ int tc_owner(long long T, int G, long long u) {
    int c = (int)(u * G / T);
    while (c + 1 < G && tc_first_unit(T, G, c + 1) <= u) ++c;
    while (c > 0 && tc_first_unit(T, G, c) > u) --c;
    return c;
}

// LINK: the instance whose epilogue pushes its fp32 results into the peers' inboxes (see TpLink).
template <int NB, bool LINK>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapW0, const __grid_constant__ CUtensorMap mapW1,
               const __grid_constant__ CUtensorMap mapX, const TcParams p) {
    constexpr int B_BYTES = NB * kTcBlockK * 2;
    constexpr int STAGE_BYTES = kTcABytes + B_BYTES;
    constexpr int TMEM_COLS = (2 * NB < 32) ? 32 : 2 * NB;  // two accumulators, power of two >= 32
    constexpr uint32_t IDESC = umma_idesc_bf16(kTcRows, NB);

    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    unsigned char* smem = smem_raw + (((raw + 1023u) & ~1023u) - raw);  // swizzled tiles need 1024-byte alignment
    unsigned char* stages = smem;
    unsigned char* tail = smem + (size_t)p.nstages * STAGE_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
    uint64_t* empty_bar = full_bar + kTcMaxStages;
    uint64_t* acc_full = empty_bar + kTcMaxStages;  // [2] accumulator ready for the epilogue
    uint64_t* acc_empty = acc_full + 2;             // [2] accumulator drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* ticket = reinterpret_cast<int*>(tmem_slot + 2);
    float* xch = reinterpret_cast<float*>(tail + 256);  // [64][NB + 1]: up values handed to the gate warps
    // Segment table of this CTA, in processing order: {tile, first k-block, end k-block, partial slot}.
    int* segs = reinterpret_cast<int*>(tail + 256 + 64 * (NB + 1) * sizeof(float));
    int* nseg_s = segs + 4 * kTcMaxSegs;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = p.nstages;
    const int G = gridDim.x, cta = blockIdx.x;
    const long long T = (long long)p.tiles * p.kblocks;
    const long long u0 = tc_first_unit(T, G, cta), u1 = tc_first_unit(T, G, cta + 1);
    const int KB = p.kblocks;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&acc_full[a]), 1);
            mbar_init(smem_u32(&acc_empty[a]), 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
        // The unit range [u0, u1) cut at tile boundaries.  Partial tiles (shared with a neighbour CTA) are
        // processed FIRST, whole tiles after them: the fix-up of a shared tile then runs in the epilogue
        // warps while the producer and the MMA warp are already streaming the whole tiles, instead of
        // at the very end of the kernel where nothing can hide it.
        int n = 0;
        for (int pass = 0; pass < 2; ++pass) {
            long long u = u0;
            int natural = 0;
            while (u < u1) {
                const int t = (int)(u / KB), k0 = (int)(u % KB);
                const long long left = u1 - u;
                const int k1 = (KB - k0 < left) ? KB : k0 + (int)left;
                const bool whole = (k0 == 0 && k1 == KB);
                if ((pass == 0) != whole) {
                    segs[4 * n] = t, segs[4 * n + 1] = k0, segs[4 * n + 2] = k1, segs[4 * n + 3] = natural == 0 ? 0 : 1;
                    ++n;
                }
                u += k1 - k0;
                ++natural;
            }
        }
        *nseg_s = n;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    unsigned long long* trec = (tid == 64) ? trace_open(p.trace, (unsigned)p.trace_id, blockIdx.x) : nullptr;
    pdl_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // One thread feeds the whole ring, so its per-unit cost matters: all counters
            // are 32-bit and advance incrementally (no divisions in the loop).
            const int n_units = (int)(u1 - u0);
            const int nseg = *nseg_s;
            // two cursors over the segment table: the next unit whose weights / activations are requested
            int wsi = 0, wkb = nseg ? segs[1] : 0, xsi = 0, xkb = wkb;
            auto advance = [&](int& si, int& kb) {
                if (++kb == segs[4 * si + 2]) {
                    ++si;
                    kb = si < nseg ? segs[4 * si + 1] : 0;
                }
            };
            int stage = 0;
            uint32_t empty_parity = 1;  // a fresh barrier passes a wait on parity 1
            auto request_w = [&](int st, int t, int k) {
                const uint32_t bar = smem_u32(&full_bar[st]);
                mbar_arrive_expect_tx(bar, STAGE_BYTES);
                const uint32_t a = smem_u32(stages + (size_t)st * STAGE_BYTES);
                if (p.pair) {
                    tma_load_2d(a, &mapW0, k * kTcBlockK, t * (kTcRows / 2), bar);
                    tma_load_2d(a + kTcABytes / 2, &mapW1, k * kTcBlockK, t * (kTcRows / 2), bar);
                } else {
                    tma_load_2d(a, &mapW0, k * kTcBlockK, t * kTcRows, bar);
                }
            };
            auto request_x = [&](int st, int k) {
                tma_load_2d(smem_u32(stages + (size_t)st * STAGE_BYTES) + kTcABytes, &mapX, k * kTcBlockK, 0,
                            smem_u32(&full_bar[st]));
            };
            // weights do not depend on the kernel in front: request them before the dependency wait
            const int npre = n_units < NS ? n_units : NS;
            for (int i = 0; i < npre; ++i) {
                request_w(i, segs[4 * wsi], wkb);
                advance(wsi, wkb);
            }
            pdl_wait();
            for (int i = 0; i < npre; ++i) {
                request_x(i, xkb);
                advance(xsi, xkb);
            }
            int issued = npre;
            stage = (npre == NS) ? 0 : npre;
            if (npre == NS) empty_parity = 0;
            for (int i = npre; i < n_units; ++i) {
                if (!mbar_wait_bounded(smem_u32(&empty_bar[stage]), empty_parity, abort_flag, p.status, FAULT_GEMV_EMPTY_WAIT)) break;
                request_w(stage, segs[4 * wsi], wkb);
                request_x(stage, wkb);
                advance(wsi, wkb);
                if (++stage == NS) stage = 0, empty_parity ^= 1;
                issued = i + 1;
            }
            if (*abort_flag) {  // nothing may still be landing in this CTA's shared memory when it exits
                const int first = issued > NS ? issued - NS : 0;
                for (int i = first; i < issued; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try_wait(smem_u32(&full_bar[i % NS]), (uint32_t)((i / NS) & 1)))
                        if (clock64() - t0 > kWaitLimitCycles) {
                            report_fault(p.status, FAULT_GEMV_DRAIN);
                            break;
                        }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const int nseg = *nseg_s;
            int stage = 0;
            uint32_t full_parity = 0;
            for (int seg = 0; seg < nseg && !(*abort_flag); ++seg) {
                const int kb0 = segs[4 * seg + 1], kb1 = segs[4 * seg + 2];
                const int acc = seg & 1;
                // wait until the epilogue has drained this accumulator (passes at once for its first use)
                if (!mbar_wait_bounded(smem_u32(&acc_empty[acc]), (uint32_t)(((seg >> 1) & 1) ^ 1), abort_flag, p.status,
                                       FAULT_TC_ACC_WAIT))
                    break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * NB);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(&full_bar[stage]), full_parity, abort_flag, p.status, FAULT_GEMV_FULL_WAIT))
                        break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stages + (size_t)stage * STAGE_BYTES);
                    const uint64_t adesc = umma_desc_sw128(a_addr);
                    const uint64_t bdesc = umma_desc_sw128(a_addr + kTcABytes);
#pragma unroll
                    for (int k = 0; k < kTcBlockK / 16; ++k)  // 32 bytes along K per MMA: +2 in the 16-byte address field
                        tc_mma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit(smem_u32(&empty_bar[stage]));  // stage reusable once these MMAs have read it
                    if (++stage == NS) stage = 0, full_parity ^= 1;
                }
                tc_commit(smem_u32(&acc_full[acc]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int q = warp & 3;          // tensor-memory lane quarter this warp may read
        const int row = q * 32 + lane;   // row of the tile held by this thread
        const int et = (warp - 2) * 32 + lane;
        pdl_wait();
        trace_mark(trec, 3);
        const unsigned int push_epoch = (LINK && p.link.world > 0 && p.link.push_inbox >= 0) ? tp_next_epoch(p.link, p.link.push_inbox) : 0u;
        const bool poisoned = LINK && p.link.world > 0 && tp_poisoned(p.status);  // see tp_poisoned: push nothing, advance nothing
        const int nseg = *nseg_s;
        for (int seg = 0; seg < nseg; ++seg) {
            const int tile = segs[4 * seg], kb0 = segs[4 * seg + 1], kb1 = segs[4 * seg + 2];
            const int acc = seg & 1;
            mbar_wait_bounded(smem_u32(&acc_full[acc]), (uint32_t)((seg >> 1) & 1), abort_flag, p.status, FAULT_TC_ACC_WAIT);
            if (seg == 0) trace_mark(trec, 4);
            tc_fence_after();
            float v[NB];
#pragma unroll
            for (int c = 0; c < NB; c += 16) {
                float t[16];
                tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * NB + c), t);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[c + i] = t[i];
            }
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));

            const bool whole = (kb0 == 0 && kb1 == KB);
            if (!whole) {
                bool finish;
                // partial tile: park it, take a ticket; the last contributor adds all parts in CTA order
                float* mine = p.partial + ((size_t)cta * 2 + segs[4 * seg + 3]) * (NB * kTcRows);
#pragma unroll
                for (int b = 0; b < NB; ++b) mine[b * kTcRows + row] = v[b];
                named_bar_sync(2, 128);
                const long long t_first = (long long)tile * KB, t_last = t_first + KB - 1;
                const int c_first = tc_owner(T, G, t_first), c_last = tc_owner(T, G, t_last);
                if (et == 0) {
                    unsigned int prev;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(p.counters + tile) : "memory");
                    *ticket = (prev == (unsigned int)(c_last - c_first)) ? 1 : 0;
                    if (*ticket) p.counters[tile] = 0u;
                }
                named_bar_sync(2, 128);
                finish = (*ticket != 0);
                named_bar_sync(2, 128);  // `ticket` may be rewritten by the next segment
                if (!finish || *abort_flag) continue;

                // Fix-up by the last contributor.  Every value now comes from the parked parts, so the
                // threads regroup for memory-level parallelism: a thread owns 4 consecutive rows
                // (one 16-byte load per part and batch row) of a quarter of the batch, and the parts
                // of two contributors are in flight together.  Parts are added in CTA order, which
                // fixes the bits whatever the arrival order was.
                constexpr int NBG = NB / 4;
                const int r4 = lane * 4, b0 = (et >> 5) * NBG;
                float4 acc[NBG];
#pragma unroll
                for (int j = 0; j < NBG; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
                for (int c = c_first; c <= c_last; ++c) {
                    const bool first_seg = (tc_first_unit(T, G, c) / KB) == tile;
                    const float* part = p.partial + ((size_t)c * 2 + (first_seg ? 0 : 1)) * (NB * kTcRows) + b0 * kTcRows + r4;
#pragma unroll
                    for (int j = 0; j < NBG; ++j) {
                        const float4 t = __ldcg(reinterpret_cast<const float4*>(part + j * kTcRows));
                        acc[j].x += t.x, acc[j].y += t.y, acc[j].z += t.z, acc[j].w += t.w;
                    }
                }
                if (LINK && !p.pair && p.epilogue == EPI_PUSH_F32) {
                    // A lane holds 4 consecutive rows; stored as they are, a warp's 64-bit peer stores would
                    // be 32 bytes apart (one NVLink transaction each: measured 30 us per tile).  Shuffle so
                    // that lane L owns rows 2L, 2L+1 (then 64+2L, 64+2L+1): 512 contiguous bytes per store.
                    const int src = lane >> 1;
                    const bool odd = lane & 1;
#pragma unroll
                    for (int j = 0; j < NBG; ++j) {
#pragma unroll
                        for (int half = 0; half < 2; ++half) {
                            const int s2 = src + half * 16;
                            const float ax = __shfl_sync(0xffffffffu, acc[j].x, s2), ay = __shfl_sync(0xffffffffu, acc[j].y, s2);
                            const float az = __shfl_sync(0xffffffffu, acc[j].z, s2), aw = __shfl_sync(0xffffffffu, acc[j].w, s2);
                            if (!poisoned && b0 + j < p.B && tile * kTcRows + half * 64 + 2 * lane < p.N)
                                tp_push2(p.link, (long long)(b0 + j) * p.ldout + tile * kTcRows + half * 64 + 2 * lane,
                                         odd ? az : ax, odd ? aw : ay, push_epoch);
                        }
                    }
                    continue;
                }
                if (!p.pair) {
                    const int n = tile * kTcRows + r4;
                    if (n < p.N) {
                        if (p.epilogue == EPI_RESIDUAL) {
                            uint2 res[NBG];
#pragma unroll
                            for (int j = 0; j < NBG; ++j)
                                res[j] = (b0 + j < p.B) ? *reinterpret_cast<const uint2*>(p.residual + (long long)(b0 + j) * p.ldres + n)
                                                        : make_uint2(0u, 0u);
#pragma unroll
                            for (int j = 0; j < NBG; ++j)
                                if (b0 + j < p.B)
                                    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + (long long)(b0 + j) * p.ldout + n) =
                                        make_uint2(pack_bf16(bf16_lo(res[j].x) + round_bf16(acc[j].x), bf16_hi(res[j].x) + round_bf16(acc[j].y)),
                                                   pack_bf16(bf16_lo(res[j].y) + round_bf16(acc[j].z), bf16_hi(res[j].y) + round_bf16(acc[j].w)));
                        } else if (p.epilogue == EPI_STORE_F32) {
#pragma unroll
                            for (int j = 0; j < NBG; ++j)
                                if (b0 + j < p.B) *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (long long)(b0 + j) * p.ldout + n) = acc[j];
                        } else {
#pragma unroll
                            for (int j = 0; j < NBG; ++j)
                                if (b0 + j < p.B)
                                    *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + (long long)(b0 + j) * p.ldout + n) =
                                        make_uint2(pack_bf16(acc[j].x, acc[j].y), pack_bf16(acc[j].z, acc[j].w));
                        }
                    }
                } else {
                    // lanes 0..15 hold gate rows 0..63, lanes 16..31 the matching up rows
                    const int n = tile * (kTcRows / 2) + r4;
#pragma unroll
                    for (int j = 0; j < NBG; ++j) {
                        float4 up;
                        up.x = __shfl_down_sync(0xffffffffu, acc[j].x, 16), up.y = __shfl_down_sync(0xffffffffu, acc[j].y, 16);
                        up.z = __shfl_down_sync(0xffffffffu, acc[j].z, 16), up.w = __shfl_down_sync(0xffffffffu, acc[j].w, 16);
                        if (lane < 16 && n < p.N && b0 + j < p.B) {
                            const float o0 = round_bf16(silu_f32(round_bf16(acc[j].x))) * round_bf16(up.x);
                            const float o1 = round_bf16(silu_f32(round_bf16(acc[j].y))) * round_bf16(up.y);
                            const float o2 = round_bf16(silu_f32(round_bf16(acc[j].z))) * round_bf16(up.z);
                            const float o3 = round_bf16(silu_f32(round_bf16(acc[j].w))) * round_bf16(up.w);
                            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + (long long)(b0 + j) * p.ldout + n) =
                                make_uint2(pack_bf16(o0, o1), pack_bf16(o2, o3));
                        }
                    }
                }
                continue;
            }
            if (*abort_flag) continue;

            if (!p.pair) {
                const int n = tile * kTcRows + row;
                if (n < p.N) {
                    if (p.epilogue == EPI_RESIDUAL) {
                        // all residual values are fetched before the first store: the stores may alias
                        // them as far as the compiler knows, which would serialise 64 L2 round trips
                        float res[NB];
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            res[b] = (b < p.B) ? __bfloat162float(p.residual[(long long)b * p.ldres + n]) : 0.f;
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (b < p.B)
                                reinterpret_cast<bf16*>(p.out)[(long long)b * p.ldout + n] =
                                    __float2bfloat16_rn(res[b] + round_bf16(v[b]));
                    } else if (LINK && p.epilogue == EPI_PUSH_F32) {
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (b < p.B && !poisoned) tp_push(p.link, (long long)b * p.ldout + n, v[b], push_epoch);
                    } else if (p.epilogue == EPI_STORE_F32) {
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (b < p.B) reinterpret_cast<float*>(p.out)[(long long)b * p.ldout + n] = v[b];
                    } else {
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (b < p.B) reinterpret_cast<bf16*>(p.out)[(long long)b * p.ldout + n] = __float2bfloat16_rn(v[b]);
                    }
                }
            } else {
                // rows 0..63 hold gate values of pairs 0..63, rows 64..127 the matching up values
                if (row >= 64) {
#pragma unroll
                    for (int b = 0; b < NB; ++b) xch[(row - 64) * (NB + 1) + b] = v[b];
                }
                named_bar_sync(2, 128);
                if (row < 64) {
                    const int n = tile * (kTcRows / 2) + row;
                    if (n < p.N) {
#pragma unroll
                        for (int b = 0; b < NB; ++b) {
                            if (b >= p.B) break;
                            const float gate = round_bf16(v[b]), up = round_bf16(xch[row * (NB + 1) + b]);
                            reinterpret_cast<bf16*>(p.out)[(long long)b * p.ldout + n] =
                                __float2bfloat16_rn(round_bf16(silu_f32(gate)) * up);
                        }
                    }
                }
                named_bar_sync(2, 128);
            }
        }
        trace_mark(trec, 5);
        if (LINK && p.link.world > 0 && p.link.bump_inbox >= 0 && blockIdx.x == 0 && et == 0 && !*abort_flag && !poisoned) tp_bump(p.link);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D bf16 row-major [rows, cols] with leading dimension ld; box = [64 cols, box_rows], 128-byte swizzle,
// out-of-range elements read as zero.
static bool encode_map(CUtensorMap* map, const bf16* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)kTcBlockK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<bf16*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A descriptor is a pure function of (address, shape, leading dimension, box): a decode loop asks for the same few
// dozen over and over (four weight matrices per layer and the activation buffers of the workspace), so they are
// encoded once and kept in a small table (round-robin replacement; a hit costs a short scan under a mutex instead
// of a driver call per operand and launch).
struct MapKey {
    const void* base;
    long long rows, cols, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
static constexpr int kMapCacheSize = 256;
static bool make_map(CUtensorMap* map, const bf16* base, long long rows, long long cols, long long ld, int box_rows) {
    struct Entry {
        MapKey key;
        alignas(64) CUtensorMap map;
    };
    static std::mutex mu;
    static Entry* table = new Entry[kMapCacheSize]();  // never freed: lives as long as the library
    static int used = 0, next = 0;
    const MapKey key = {base, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; ++i)
        if (table[i].key == key) {
            std::memcpy(map, &table[i].map, sizeof(CUtensorMap));
            return true;
        }
    if (!encode_map(map, base, rows, cols, ld, box_rows)) return false;
    const int slot = used < kMapCacheSize ? used++ : (next = (next + 1) % kMapCacheSize);
    table[slot].key = key;
    std::memcpy(&table[slot].map, map, sizeof(CUtensorMap));
    return true;
}

static int tc_batch_tile(int B) { return B <= 16 ? 16 : (B <= 32 ? 32 : 64); }

bool gemm_tc_supported(int B, int K) { return B >= 2 && B <= 64 && K % 8 == 0 && encode_fn() != nullptr; }
bool gemm_tc_fits(int N, bool pair) { return (N + (pair ? 63 : 127)) / (pair ? 64 : 128) <= kTcMaxTiles; }

size_t gemm_tc_workspace_bytes(int B, int N, bool pair) {
    (void)N, (void)pair;
    const int NB = tc_batch_tile(B);
    return kTcCounterBytes + (size_t)sm_count() * 2 * NB * kTcRows * sizeof(float);
}

template <int NB, bool LINK>
static cudaError_t launch_tc_instance(const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& mx, TcParams& p,
                                      int grid, cudaStream_t stream) {
    auto kernel = gemm_tc_kernel<NB, LINK>;
    constexpr size_t stage = kTcABytes + (size_t)NB * kTcBlockK * 2;
    const size_t tail = 256 + (size_t)64 * (NB + 1) * sizeof(float) + (4 * kTcMaxSegs + 4) * sizeof(int);
    const size_t cap = (size_t)max_smem_optin();
    int ns = (int)((cap - 1024 - tail) / stage);
    if (ns > kTcMaxStages) ns = kTcMaxStages;
    p.nstages = ns;
    const size_t smem = 1024 + (size_t)ns * stage + tail;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cap);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(grid), dim3(kTcThreads), smem, stream, m0, m1, mx, p);
}

// x must already hold what the MMA consumes (any norm prologue has been run by the caller).
cudaError_t launch_gemm_tc(const GemvArgs& a, const bf16* x, long long ldx, void* workspace, cudaStream_t stream) {
    const bool pair = a.epilogue == EPI_SWIGLU;
    const int NB = tc_batch_tile(a.B);
    TcParams p;
    p.N = a.N, p.K = a.K, p.B = a.B;
    p.tiles = (a.N + (pair ? 63 : 127)) / (pair ? 64 : 128);
    p.kblocks = (a.K + kTcBlockK - 1) / kTcBlockK;
    p.pair = pair ? 1 : 0;
    p.epilogue = a.epilogue;
    p.residual = a.residual, p.ldres = a.ldres;
    p.out = a.out, p.ldout = a.ldout;
    if (p.tiles > kTcMaxTiles) return cudaErrorInvalidValue;
    p.counters = reinterpret_cast<unsigned int*>(workspace);
    p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kTcCounterBytes);
    p.status = status_ptr();
    if (!p.status) return cudaErrorUnknown;
    p.trace = trace_handle();
    p.trace_id = a.trace_id;
    p.link = a.link;
    if (a.link.world > 0 && (a.link.gather_inbox >= 0 || pair)) return cudaErrorNotSupported;  // only the push side lives here

    alignas(64) CUtensorMap m0, m1, mx;
    const int box_rows = pair ? 64 : 128;
    if (!make_map(&m0, a.W0, a.N, a.K, a.ldw, box_rows)) return cudaErrorInvalidValue;
    if (!make_map(&m1, pair ? a.W1 : a.W0, a.N, a.K, a.ldw, box_rows)) return cudaErrorInvalidValue;
    if (!make_map(&mx, x, a.B, a.K, ldx, NB)) return cudaErrorInvalidValue;

    long long T = (long long)p.tiles * p.kblocks;
    int grid = sm_count();
    if (grid > T) grid = (int)T;
    if (a.link.world > 0) {
        switch (NB) {
            case 16: return launch_tc_instance<16, true>(m0, m1, mx, p, grid, stream);
            case 32: return launch_tc_instance<32, true>(m0, m1, mx, p, grid, stream);
            default: return launch_tc_instance<64, true>(m0, m1, mx, p, grid, stream);
        }
    }
    switch (NB) {
        case 16: return launch_tc_instance<16, false>(m0, m1, mx, p, grid, stream);
        case 32: return launch_tc_instance<32, false>(m0, m1, mx, p, grid, stream);
        default: return launch_tc_instance<64, false>(m0, m1, mx, p, grid, stream);
    }
}

}  // namespace ezb
