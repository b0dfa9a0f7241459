// The whole Qwen3 dense decode layer at batch 1 as ONE persistent kernel.
//
// At batch 1 the layer is 386 MB of weights and 17 MB of KV cache streamed once;
// everything else is latency.  A chain of five kernels pays that latency at every
// boundary (drain, launch, activation staging, ring fill) with HBM idle.  Here one
// CTA per SM lives through all five phases
//     QKV projection -> attention -> output projection -> gate/up + SwiGLU -> down projection
// and its producer warp never stops: it walks ONE sequence of shared-memory
// stages that covers every byte this CTA will ever need (its rows of Wqkv, its
// slice of the K and V cache, its rows of Wo, Wg|Wu, Wd), requesting them with
// 1-D bulk TMA copies into a ring as slots come free.  Weights are immutable, so
// nothing in that sequence waits for a dependency; while the eight consumer warps
// sit in a grid-wide barrier between two phases (or normalise the next activation
// vector), the ring fills with the next phase's weights, and when the ring is
// full the producer keeps HBM busy by asking L2 for the stages after it
// (cp.async.bulk.prefetch.L2, a bounded look-ahead).
//
// Phases are separated by grid barriers: a counter in global memory, one
// arrive (fence + atomic) and one bounded poll per CTA.  All CTAs of the grid
// must be resident together, so the grid never exceeds the number of SMs and
// the kernel needs one CTA per SM worth of shared memory; the host checks both.
// The barrier counters are returned to zero by the CTA that leaves last.
//
// Arithmetic follows the chained kernels: bf16 storage, fp32 accumulation,
// every projection result rounded to bf16 where the torch reference rounds it
// (ezops/ops/qwen3_dense_decode.py:142-176).  The projections run on mma.sync
// m16n8k16 fed by plain 128-bit shared-memory loads (see mega_gemv_phase), eight
// warps split k and are summed in a fixed order.  Attention at batch 1 is tiny (S keys x G query heads per
// kv head): every kv head is cut into `nsp` slices, one CTA each; scores run on
// mma.sync straight from the unpadded K rows (128-bit loads, the k index of the
// mma permuted so that a lane's 8 consecutive elements feed two k-steps), the
// soft-max is fp32 in the exp2 domain, P.V is plain fp32 FMA with a lane owning
// D/32 output dims.  Slice results (max, sum, O) go to the workspace; the CTA
// that finishes last for a kv head (one atomic ticket) folds them in slice order.
// Nothing here depends on the order in which CTAs arrive, so results are
// bit-reproducible.
//
// Every wait (ring barriers, grid barriers) is bounded by a cycle budget taken
// from the tuning table; a wait that runs out sets the CTA's abort flag and the
// device status word, after which all waits fall through, global stores are
// suppressed, the producer drains its copies in flight and the kernel ends.
#include "launchers.h"

namespace ezb {

static constexpr int kMegaConsumerWarps = 8;
static constexpr int kMegaConsumerThreads = kMegaConsumerWarps * 32;
static constexpr int kMegaThreads = 32 + kMegaConsumerThreads;
static constexpr int kMegaMaxStages = 8;
static constexpr int kMegaHeaderBytes = 512;   // barriers, abort flag, norm scratch, flags
static constexpr int kMegaRedGroup = 4;        // row blocks whose partial sums are combined across the warps in one go
static constexpr int kMegaRedBytes = 2 * kMegaRedGroup * kMegaConsumerWarps * 8 * (int)sizeof(float);
static constexpr int kMegaRowPad = 32;         // elements of padding behind a weight row in a stage (64 B: 128-bit loads of two rows never collide)
static constexpr int kMegaResSlots = 256;      // output rows of one CTA in the H-row phases
static constexpr int kMegaSubKeysMax = 256;    // keys of one attention sub-chunk (one K stage + one V stage)
static constexpr int kMegaMaxSplits = 32;      // slices per kv head (the fold at the end reads them in two round trips)
static constexpr int kCombineBatch = 10;       // slice records a combining thread fetches per round trip

enum MegaCtrl : int { MB_QKV = 0, MB_ATTN = 1, MB_OPROJ = 2, MB_GATEUP = 3, MB_EXIT = 4, MB_TICKET0 = 8 };

struct MegaParams {
    const bf16* hidden;
    bf16* out;
    bf16* Kc;
    bf16* Vc;
    const bf16 *Wqkv, *Wo, *Wg, *Wu, *Wd;
    const bf16 *in_norm_w, *post_norm_w, *q_norm_w, *k_norm_w, *rope_cos, *rope_sin;
    bf16 *qkv, *attn_out, *x2, *h;
    unsigned int* ctrl;
    float* part_ml;  // [NKV][nsp][8][2]
    float* part_o;   // [NKV][nsp][8][D]
    int S, H, I, NH, NKV, G, Q, R;
    float eps, scale_log2e;
    int kc_h, kc_q, kc_i;
    int nsp, sub_keys;
    int NS, l2_window;
    int inflight;  // stages that may be requested but not yet landed (0 = the whole ring)
    int gate;      // bit 0: nothing behind this CTA's K/V stages is requested or prefetched before the QKV barrier has been
                   // passed; bit 1: no gate/up stage before the barrier behind o_proj; bit 2: no down stage before the
                   // barrier behind gate/up
    unsigned int stage_bytes, act_bytes;
    long long wait_cycles;
    int evict_first;  // L2 evict-first policy on the streams: 1 = weights, 2 = weights and K/V
    unsigned int* status;
    Trace trace;
    TpLink link;  // tensor parallel: world > 0, this rank's shard in every weight and cache pointer above
};

// What one CTA does in every phase; computed identically by producer and consumers.
struct MegaSched {
    int q_r0, q_r1;  // rows of Wqkv
    int o_r0, o_r1;  // rows of Wo and Wd (outputs of width H)
    int g_r0, g_r1;  // (gate, up) row pairs
    int nkc_h, nkc_q, nkc_i;
    int att_kvh, att_split, att_c0, att_c1, att_nsub;  // att_nsub == 0: this CTA has no attention slice
    int e_qkv, e_att, e_o, e_gu, e_d;                  // cumulative stage counts
};

template <int D>
__device__ __forceinline__ MegaSched mega_sched(const MegaParams& p, int cta, int grid) {
    MegaSched s;
    s.q_r0 = (int)((long long)p.R * cta / grid), s.q_r1 = (int)((long long)p.R * (cta + 1) / grid);
    // cut on even rows: the tensor-parallel form fetches two neighbouring rows' cells with one 16-byte load
    s.o_r0 = 2 * (int)((long long)(p.H / 2) * cta / grid), s.o_r1 = 2 * (int)((long long)(p.H / 2) * (cta + 1) / grid);
    s.g_r0 = (int)((long long)p.I * cta / grid), s.g_r1 = (int)((long long)p.I * (cta + 1) / grid);
    s.nkc_h = (p.H + p.kc_h - 1) / p.kc_h;
    s.nkc_q = (p.Q + p.kc_q - 1) / p.kc_q;
    s.nkc_i = (p.I + p.kc_i - 1) / p.kc_i;
    s.att_nsub = 0, s.att_kvh = 0, s.att_split = 0, s.att_c0 = 0, s.att_c1 = 0;
    if (cta < p.NKV * p.nsp) {
        s.att_kvh = cta / p.nsp, s.att_split = cta - s.att_kvh * p.nsp;
        s.att_c0 = (int)((long long)p.S * s.att_split / p.nsp);
        s.att_c1 = (int)((long long)p.S * (s.att_split + 1) / p.nsp);
        s.att_nsub = (s.att_c1 - s.att_c0 + p.sub_keys - 1) / p.sub_keys;
    }
    s.e_qkv = ((s.q_r1 - s.q_r0 + 7) / 8) * s.nkc_h;
    s.e_att = s.e_qkv + 2 * s.att_nsub;
    s.e_o = s.e_att + ((s.o_r1 - s.o_r0 + 7) / 8) * s.nkc_q;
    s.e_gu = s.e_o + ((s.g_r1 - s.g_r0 + 3) / 4) * s.nkc_h;
    s.e_d = s.e_gu + ((s.o_r1 - s.o_r0 + 7) / 8) * s.nkc_i;
    return s;
}

// One stage of the producer's sequence.
struct MegaStage {
    int kind;  // 0: up to 8 weight rows; 1: up to 4 gate rows + the matching up rows; 2: keys of the K or V cache
    const bf16* src0;
    const bf16* src1;
    long long ld;
    int row0, nu;  // first row / number of units (rows, pairs or keys)
    int k0, len;   // k range of the stage (weights)
    int stride;    // shared-memory row stride in bytes (weights)
};

template <int D>
__device__ __forceinline__ MegaStage mega_locate(const MegaParams& p, const MegaSched& s, int it) {
    MegaStage d;
    d.src1 = nullptr;
    if (it < s.e_qkv) {
        const int rb = it / s.nkc_h, kci = it - rb * s.nkc_h;
        d.kind = 0, d.src0 = p.Wqkv, d.ld = p.H;
        d.row0 = s.q_r0 + rb * 8, d.nu = min(8, s.q_r1 - d.row0);
        d.k0 = kci * p.kc_h, d.len = min(p.kc_h, p.H - d.k0), d.stride = (p.kc_h + kMegaRowPad) * 2;
    } else if (it < s.e_att) {
        const int j = it - s.e_qkv, sub = j >> 1;
        const int key0 = s.att_c0 + sub * p.sub_keys;
        d.kind = 2, d.ld = 0;
        d.src0 = ((j & 1) ? p.Vc : p.Kc) + ((long long)s.att_kvh * p.S + key0) * D;
        d.row0 = key0, d.nu = min(p.sub_keys, s.att_c1 - key0);
        d.k0 = 0, d.len = 0, d.stride = 0;
    } else if (it < s.e_o) {
        const int j = it - s.e_att, rb = j / s.nkc_q, kci = j - rb * s.nkc_q;
        d.kind = 0, d.src0 = p.Wo, d.ld = p.Q;
        d.row0 = s.o_r0 + rb * 8, d.nu = min(8, s.o_r1 - d.row0);
        d.k0 = kci * p.kc_q, d.len = min(p.kc_q, p.Q - d.k0), d.stride = (p.kc_q + kMegaRowPad) * 2;
    } else if (it < s.e_gu) {
        const int j = it - s.e_o, rb = j / s.nkc_h, kci = j - rb * s.nkc_h;
        d.kind = 1, d.src0 = p.Wg, d.src1 = p.Wu, d.ld = p.H;
        d.row0 = s.g_r0 + rb * 4, d.nu = min(4, s.g_r1 - d.row0);
        d.k0 = kci * p.kc_h, d.len = min(p.kc_h, p.H - d.k0), d.stride = (p.kc_h + kMegaRowPad) * 2;
    } else {
        const int j = it - s.e_gu, rb = j / s.nkc_i, kci = j - rb * s.nkc_i;
        d.kind = 0, d.src0 = p.Wd, d.ld = p.I;
        d.row0 = s.o_r0 + rb * 8, d.nu = min(8, s.o_r1 - d.row0);
        d.k0 = kci * p.kc_i, d.len = min(p.kc_i, p.I - d.k0), d.stride = (p.kc_i + kMegaRowPad) * 2;
    }
    return d;
}

// Bounded mbarrier wait with the cycle budget of this launch (see mbar_wait_bounded).
__device__ __forceinline__ bool mega_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int* status,
                                               unsigned int code, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            *abort_flag = 1;
            report_fault(status, code);
            return false;
        }
    }
}

// The activation vector lives in shared memory in its natural order, eight elements (16 bytes) per index.
__device__ __forceinline__ void mega_store_x8(bf16* xs, int i, const uint32_t (&w)[4]) {
    *reinterpret_cast<uint4*>(xs + i * 8) = make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void mega_load_x8(const bf16* xs, int i, uint32_t (&w)[4]) {
    const uint4 v = *reinterpret_cast<const uint4*>(xs + i * 8);
    w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
}

// Brings x[K] (global, written by other CTAs of this grid or by an earlier kernel: read through L2) into
// shared memory, optionally RMS-normalised: statistics in fp32, (x * r [* w]) in fp32, one rounding.
// Called by all consumer threads; ends with a barrier among them.
template <bool NORM>
__device__ __forceinline__ void mega_stage_x(const bf16* x, int K, const bf16* norm_w, float eps, bf16* xs, float* scratch,
                                             int ct, int cw, int lane) {
    constexpr int U = 8;
    const int nvec = K / 8;
    float ssq = 0.f;
    for (int base = 0; base < nvec; base += U * kMegaConsumerThreads) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * kMegaConsumerThreads + ct;
            if (i < nvec) raw[u] = __ldcg(reinterpret_cast<const uint4*>(x) + i);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = base + u * kMegaConsumerThreads + ct;
            if (i < nvec) {
                const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                if (NORM) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float lo = bf16_lo(w[e]), hi = bf16_hi(w[e]);
                        ssq += lo * lo + hi * hi;
                    }
                }
                mega_store_x8(xs, i, w);
            }
        }
    }
    if (NORM) {
        ssq = warp_sum(ssq);
        if (lane == 0) scratch[cw] = ssq;
        named_bar_sync(1, kMegaConsumerThreads);
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kMegaConsumerWarps; ++w) tot += scratch[w];  // fixed order: reproducible
        const float r = 1.0f / sqrtf(tot / (float)K + eps);
        for (int i = ct; i < nvec; i += kMegaConsumerThreads) {  // every thread rescales the vectors it stored itself
            uint32_t w[4];
            mega_load_x8(xs, i, w);
            uint32_t nw[4] = {0u, 0u, 0u, 0u};
            if (norm_w) {
                const uint4 q = __ldg(reinterpret_cast<const uint4*>(norm_w) + i);
                nw[0] = q.x, nw[1] = q.y, nw[2] = q.z, nw[3] = q.w;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float lo = bf16_lo(w[e]) * r, hi = bf16_hi(w[e]) * r;
                if (norm_w) lo *= bf16_lo(nw[e]), hi *= bf16_hi(nw[e]);
                w[e] = pack_bf16(lo, hi);
            }
            mega_store_x8(xs, i, w);
        }
    }
    named_bar_sync(1, kMegaConsumerThreads);
}

// ---- tensor-parallel exchange inside the kernel (the cells and epochs of TpLink, common.cuh)
__device__ __forceinline__ void mega_tp_push(const TpLink& l, int inbox, long long elem, float v, unsigned int epoch) {
    const unsigned long long cell = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
    for (int w = 0; w < l.world; ++w)
        tp_store_cell(l.inbox_peer[w] + ((long long)inbox * kTpSlots + l.rank) * l.slot_elems + elem, cell, l.strong_stores);
}

// add[0..1] += sum over ranks (in rank order) of the cells of rows n, n + 1 (n even) in `inbox` of this rank: the
// poll that ends each of the two exchanges for the rows a CTA owns.
__device__ __forceinline__ bool mega_tp_gather2(const TpLink& l, int inbox, unsigned int epoch, int n, float (&add)[2],
                                                unsigned int* status, long long t0) {
    return tp_gather_from<8, 2>(l, inbox, false, epoch, n, add, status, t0);
}

// Head RMSNorm (+ optional weight, + optional rotate-half RoPE) of one head held by a warp: lane owns
// elements lane + 32*j, so the rotation partner (i +- D/2) is in the same lane.  fp32 throughout.
template <int D>
__device__ __forceinline__ void mega_head_norm_rope(float (&x)[D / 32], float eps, const bf16* w, const bf16* cosr,
                                                    const bf16* sinr, int lane) {
    constexpr int NJ = D / 32, HJ = NJ / 2;
    float ssq = 0.f;
#pragma unroll
    for (int j = 0; j < NJ; ++j) ssq += x[j] * x[j];
    ssq = warp_sum(ssq);
    const float r = 1.0f / sqrtf(ssq / (float)D + eps);
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        x[j] = __fmul_rn(x[j], r);
        if (w) x[j] = __fmul_rn(x[j], __bfloat162float(w[lane + j * 32]));
    }
    if (cosr) {
#pragma unroll
        for (int j = 0; j < HJ; ++j) {
            const int i = lane + j * 32, i2 = i + D / 2;
            const float n1 = x[j], n2 = x[j + HJ];
            x[j] = __fadd_rn(__fmul_rn(n1, __bfloat162float(cosr[i])), __fmul_rn(-n2, __bfloat162float(sinr[i])));
            x[j + HJ] = __fadd_rn(__fmul_rn(n2, __bfloat162float(cosr[i2])), __fmul_rn(n1, __bfloat162float(sinr[i2])));
        }
    }
}

__device__ __forceinline__ float mega_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float mega_ldcg_bf16(const bf16* ptr) {
    return bf16_bits_to_float((uint32_t)__ldcg(reinterpret_cast<const unsigned short*>(ptr)));
}

// ---- explicit shared-memory loads (a pointer that went through a struct loses its address space, and generic loads
// are what the compiler then emits)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds128f(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

// Everything a consumer thread carries through the phases.
struct MegaCtx {
    uint64_t* full_bar;
    uint64_t* empty_bar;
    volatile int* abort_flag;
    float* norm_scratch;
    int* flag;  // CTA-wide flag written by one thread between two barriers
    float* red;
    float* res_s;
    unsigned char* act;
    unsigned char* stage_base;
    int it;        // next stage of the sequence
    int red_flip;  // which half of the reduction buffer the next row block uses
    int ct, cw, lane;
};

// Grid-wide barrier among the consumer threads of all CTAs.  Arrive: barrier among the consumers, then one
// thread publishes the CTA's stores (fence) and adds to the counter.  Wait: that thread polls (bounded) with
// acquire loads, then the consumers meet again.
__device__ __forceinline__ void mega_grid_barrier(const MegaParams& p, MegaCtx& c, int which) {
    named_bar_sync(1, kMegaConsumerThreads);
    if (c.ct == 0) {
        __threadfence();
        unsigned int* ctr = p.ctrl + which;
        atomicAdd(ctr, 1u);
        const unsigned int target = gridDim.x;
        if (!*c.abort_flag) {
            const long long t0 = clock64();
            for (;;) {
                unsigned int v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
                if (v >= target) break;
                if (clock64() - t0 > p.wait_cycles) {
                    *c.abort_flag = 1;
                    report_fault(p.status, FAULT_MEGA_GRID_BARRIER + (unsigned int)which);
                    break;
                }
            }
        }
    }
    named_bar_sync(1, kMegaConsumerThreads);
}

// One projection phase: this CTA's rows [r0, r1) of y = W . xs (xs: the staged activation vector), weights
// taken from the ring in stage order.  PAIR: a row block is 4 gate rows + 4 up rows and `epi` gets both sums.
//
// Inner loop.  A stage holds 8 weight rows; the k range of the stage is cut into groups of 32 elements and group j
// is paired with group j + half.  One mma.sync m16n8k16 pair then covers 8 rows x 64 k: rows 0-7 of the A tile are
// the weight rows over group j, rows 8-15 the SAME weight rows over group j + half; column 0 of the B tile is x
// over group j, column 1 is x over group j + half.  C[r][0] and C[r+8][1] are the two halves of row r's dot
// product (the cross terms C[r][1], C[r+8][0] are ignored).  Fragments come from plain 128-bit shared-memory loads:
// a lane reads 8 consecutive elements of "its" row and k quarter, which feed the k slots of two mma steps (the k
// index inside an mma is a free permutation as long as A and B use the same one).  Measured on this GPU, per 64 KB
// stage and SM: ldmatrix + mma with the weights as the 8-wide B operand 1290 cycles (the two pipes do not overlap),
// this form 950.
//
// Across the eight warps (each takes every eighth pair) the partial sums are combined through shared memory in a
// fixed order, once per kMegaRedGroup row blocks: one barrier and one short epilogue per group instead of per block.
template <bool PAIR, class Epi>
__device__ __forceinline__ void mega_gemv_phase(const MegaParams& p, MegaCtx& c, int r0, int r1, int K, int kc, int nkc,
                                                Epi epi, unsigned long long* trec, unsigned int prof_id) {
    constexpr int UNITS = PAIR ? 4 : 8;
    // With tracing on, lane 0 of every warp adds up the cycles it spends waiting for stages, computing, and in the
    // cross-warp reduction, and leaves them in a trace record {prof_id, block*8 + warp, wait, compute, reduce, stages}.
    const bool prof = p.trace.buf != nullptr && (p.trace.capacity & 1u) && c.lane == 0;  // per-warp cycle accounting: odd capacities only
    long long cyc_wait = 0, cyc_comp = 0, cyc_red = 0, stages_done = 0;
    const int nrb = (r1 - r0 + UNITS - 1) / UNITS;
    const int row_bytes = (kc + kMegaRowPad) * 2;
    const int g4 = c.lane >> 2, t4 = c.lane & 3;
    const uint32_t xs_b = smem_u32(c.act) + t4 * 16;
    const uint32_t lane_off = (uint32_t)(g4 * row_bytes + t4 * 16);
    bool first = true;
    auto reduce_group = [&](int rb_first, int count, const float* redb) {
        // threads 0 .. count*UNITS-1: one output each
        if (c.ct < count * UNITS) {
            const int blk = c.ct / UNITS, j = c.ct - blk * UNITS;
            const int n = r0 + (rb_first + blk) * UNITS + j;
            if (n < r1 && !(*c.abort_flag)) {
                const float* src = redb + blk * (kMegaConsumerWarps * 8);
                float v0 = 0.f, v1 = 0.f;
#pragma unroll
                for (int w = 0; w < kMegaConsumerWarps; ++w) {
                    v0 += src[w * 8 + j];
                    if (PAIR) v1 += src[w * 8 + j + 4];
                }
                epi(n, v0, v1);
            }
        }
    };
    int group_first = 0;
    for (int rb = 0; rb < nrb; ++rb) {
        float acc[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
        for (int kci = 0; kci < nkc; ++kci) {
            const int s = c.it % p.NS;
            const long long tp0 = prof ? clock64() : 0;
            mega_mbar_wait(smem_u32(&c.full_bar[s]), (uint32_t)((c.it / p.NS) & 1), c.abort_flag, p.status, FAULT_GEMV_FULL_WAIT,
                           p.wait_cycles);
            const long long tp1 = prof ? clock64() : 0;
            cyc_wait += tp1 - tp0;
            if (first) trace_mark(trec, 4), first = false;
            const int k0 = kci * kc;
            const int len = min(kc, K - k0);
            const int nk32 = len >> 5, half = (nk32 + 1) >> 1;
            const uint32_t wl = smem_u32(c.stage_base) + (uint32_t)s * p.stage_bytes + lane_off;
            // x for column 0 (lanes g4 == 0: group j) and column 1 (lanes g4 == 1: group j + half)
            const uint32_t xl = xs_b + (uint32_t)k0 * 2 + (g4 == 1 ? half * 64 : 0);
            const bool has_x = g4 < 2;
            int pr = c.cw;
            for (; pr + kMegaConsumerWarps < half; pr += 2 * kMegaConsumerWarps) {  // two pairs in flight
                const int p1 = pr + kMegaConsumerWarps;
                const uint4 l0 = lds128(wl + pr * 64);
                const uint4 l1 = lds128(wl + p1 * 64);
                uint4 h0 = make_uint4(0u, 0u, 0u, 0u), h1 = h0, x0 = h0, x1 = h0;
                if (pr + half < nk32) h0 = lds128(wl + (pr + half) * 64);
                if (p1 + half < nk32) h1 = lds128(wl + (p1 + half) * 64);
                if (has_x && (g4 == 0 || pr + half < nk32)) x0 = lds128(xl + pr * 64);
                if (has_x && (g4 == 0 || p1 + half < nk32)) x1 = lds128(xl + p1 * 64);
                mma_bf16_16816(acc[0], l0.x, h0.x, l0.y, h0.y, x0.x, x0.y);
                mma_bf16_16816(acc[1], l0.z, h0.z, l0.w, h0.w, x0.z, x0.w);
                mma_bf16_16816(acc[2], l1.x, h1.x, l1.y, h1.y, x1.x, x1.y);
                mma_bf16_16816(acc[3], l1.z, h1.z, l1.w, h1.w, x1.z, x1.w);
            }
            for (; pr < half; pr += kMegaConsumerWarps) {
                const uint4 l0 = lds128(wl + pr * 64);
                uint4 h0 = make_uint4(0u, 0u, 0u, 0u), x0 = h0;
                if (pr + half < nk32) h0 = lds128(wl + (pr + half) * 64);
                if (has_x && (g4 == 0 || pr + half < nk32)) x0 = lds128(xl + pr * 64);
                mma_bf16_16816(acc[0], l0.x, h0.x, l0.y, h0.y, x0.x, x0.y);
                mma_bf16_16816(acc[1], l0.z, h0.z, l0.w, h0.w, x0.z, x0.w);
            }
            __syncwarp();
            if (c.lane == 0) mbar_arrive(smem_u32(&c.empty_bar[s]));
            ++c.it;
            if (prof) cyc_comp += clock64() - tp1, ++stages_done;
        }
        const long long tp2 = prof ? clock64() : 0;
        // lanes with t4 == 0 hold row g4: C[g4][0] (first half of k) + C[g4+8][1] (second half); fixed order
        const float part = ((acc[0][0] + acc[0][3]) + (acc[1][0] + acc[1][3])) + ((acc[2][0] + acc[2][3]) + (acc[3][0] + acc[3][3]));
        const int in_group = rb - group_first;
        float* redb = c.red + (c.red_flip & 1) * (kMegaRedGroup * kMegaConsumerWarps * 8);
        if (t4 == 0) redb[(in_group * kMegaConsumerWarps + c.cw) * 8 + g4] = part;
        if (in_group == kMegaRedGroup - 1 || rb == nrb - 1) {
            named_bar_sync(1, kMegaConsumerThreads);
            reduce_group(group_first, in_group + 1, redb);
            group_first = rb + 1;
            ++c.red_flip;
        }
        if (prof) cyc_red += clock64() - tp2;
    }
    if (prof) {
        const unsigned int slot = atomicAdd(p.trace.cursor, 1u);
        if (slot < p.trace.capacity) {
            unsigned long long* r = p.trace.buf + (size_t)slot * 6;
            r[0] = prof_id, r[1] = blockIdx.x * 8 + c.cw, r[2] = (unsigned long long)cyc_wait, r[3] = (unsigned long long)cyc_comp;
            r[4] = (unsigned long long)cyc_red, r[5] = (unsigned long long)stages_done;
        }
    }
}

// LINK: the tensor-parallel instance (partial sums of the two row-parallel projections exchanged through peer memory
// inside the kernel); the plain instance contains none of that code.
template <int D, bool LINK>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_layer_b1_kernel(const MegaParams p) {
    constexpr int DPL = D / 32;  // output dims per lane in P.V
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = full_bar + kMegaMaxStages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kMegaMaxStages * 8);
    int* cta_flag = reinterpret_cast<int*>(smem + 2 * kMegaMaxStages * 8 + 16);
    volatile int* gate_open = reinterpret_cast<volatile int*>(smem + 2 * kMegaMaxStages * 8 + 20);
    float* norm_scratch = reinterpret_cast<float*>(smem + 2 * kMegaMaxStages * 8 + 32);
    float* red = reinterpret_cast<float*>(smem + kMegaHeaderBytes);
    float* res_s = reinterpret_cast<float*>(smem + kMegaHeaderBytes + kMegaRedBytes);
    unsigned char* act = smem + kMegaHeaderBytes + kMegaRedBytes + kMegaResSlots * sizeof(float);
    unsigned char* stage_base = act + p.act_bytes;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int NS = p.NS;
    const MegaSched s = mega_sched<D>(p, blockIdx.x, gridDim.x);
    const int total = s.e_d;

    if (tid == 0) {
        for (int i = 0; i < NS; ++i) {
            mbar_init(smem_u32(&full_bar[i]), 1);
            mbar_init(smem_u32(&empty_bar[i]), kMegaConsumerWarps);
        }
        *abort_flag = 0;
        *cta_flag = 0;
        *gate_open = 0;  // barriers passed by the consumers so far
        mbar_fence_init();
    }
    __syncthreads();
    pdl_trigger();

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        bool waited = false;
        const unsigned long long policy = p.evict_first ? l2_evict_first_policy() : 0ull;
        auto issue = [&](int it, bool l2_only) {
            const MegaStage d = mega_locate<D>(p, s, it);
            // The KV cache is mutable state of earlier kernels in the stream: nothing of it is touched
            // before they have finished.  Weights never wait.
            if (d.kind == 2 && !waited) {
                pdl_wait();
                waited = true;
            }
            const uint32_t bar = smem_u32(&full_bar[it % NS]);
            const uint32_t dst0 = smem_u32(stage_base + (size_t)(it % NS) * p.stage_bytes);
            const bf16* src = nullptr;
            uint32_t bytes = 0, off = 0, expect = 0;
            if (d.kind == 2) {
                const int kp = (d.nu + 7) / 8, k_lo = lane * kp;
                const int cnt = max(0, min(kp, d.nu - k_lo));
                src = d.src0 + (long long)k_lo * D, bytes = (uint32_t)(cnt * D * 2), off = (uint32_t)(k_lo * D * 2);
                expect = (uint32_t)(d.nu * D * 2);
            } else {
                const int m = d.kind == 1 ? (lane >> 2) : 0;
                const int u = d.kind == 1 ? (lane & 3) : lane;
                if (u < d.nu) {
                    src = (m ? d.src1 : d.src0) + (long long)(d.row0 + u) * d.ld + d.k0;
                    bytes = (uint32_t)(d.len * 2), off = (uint32_t)(lane * d.stride);
                }
                expect = (uint32_t)(d.nu * (d.kind == 1 ? 2 : 1) * d.len * 2);
            }
            if (l2_only) {
                if (lane < 8 && bytes) prefetch_l2_bulk(src, bytes);
                return;
            }
            if (lane == 0) mbar_arrive_expect_tx(bar, expect);
            __syncwarp();
            if (lane < 8 && bytes) bulk_g2s(dst0 + off, src, bytes, bar, (d.kind == 2 ? p.evict_first > 1 : p.evict_first > 0) ? policy : 0ull);
        };
        // Policy.  (1) Requests queue in front of everything else this SM sends to memory, the barrier traffic
        // included, so only `inflight` stages may be outstanding at a time: enough to cover the latency-bandwidth
        // product, not the whole ring.  (2) Until the QKV barrier has been passed, traffic for later phases only
        // delays the CTAs that still wait for their QKV rows (and with them everybody): the producer stops behind
        // its K/V stages until its consumers open the gate.  (3) With the gate open and the ring full, it pulls the
        // stages behind the ring into L2 (a bounded look-ahead) while attention, the barriers and the activation
        // staging leave HBM idle.
        int issued = 0, pf = 0;
        bool ok = true;
        auto give_up = [&](unsigned int code) {
            *abort_flag = 1;
            report_fault(p.status, code);
            ok = false;
        };
        for (int it = 0; it < total && ok; ++it) {
            // barriers the consumers must have passed before stage `it` may be requested (0: none)
            const int need = ((p.gate & 4) && it >= s.e_gu) ? 4 : ((p.gate & 2) && it >= s.e_o) ? 3 : ((p.gate & 1) && it >= s.e_att) ? 1 : 0;
            if (*gate_open < need) {
                const long long t0 = clock64();
                while (*gate_open < need && ok) {
                    if (*abort_flag) ok = false;
                    else if (clock64() - t0 > p.wait_cycles) give_up(FAULT_GEMV_EMPTY_WAIT);
                }
                if (!ok) break;
            }
            if (p.inflight > 0 && it >= p.inflight) {
                const int j = it - p.inflight;
                if (!mega_mbar_wait(smem_u32(&full_bar[j % NS]), (uint32_t)((j / NS) & 1), abort_flag, p.status, FAULT_GEMV_FULL_WAIT,
                                    p.wait_cycles))
                    break;
            }
            if (it >= NS) {
                const uint32_t bar = smem_u32(&empty_bar[it % NS]);
                const uint32_t parity = (uint32_t)(((it / NS) & 1) ^ 1);
                if (!mbar_test_wait(bar, parity)) {
                    long long t0 = clock64();
                    for (;;) {
                        if (mbar_test_wait(bar, parity)) break;
                        if (*abort_flag) {
                            ok = false;
                            break;
                        }
                        // The ring is full: keep HBM busy by pulling the stages behind it into L2.
                        if (pf < it) pf = it;
                        if ((*gate_open || !(p.gate & 1)) && pf < total && pf < it + p.l2_window) {
                            issue(pf, true);
                            ++pf;
                            t0 = clock64();
                        } else if (clock64() - t0 > p.wait_cycles) {
                            give_up(FAULT_GEMV_EMPTY_WAIT);
                            break;
                        }
                    }
                    if (!ok) break;
                }
            }
            issue(it, false);
            issued = it + 1;
        }
        if (*abort_flag) {
            // leave only when nothing is still in flight towards this CTA's shared memory
            const int first = max(0, issued - NS);
            for (int it = first; it < issued; ++it) {
                const long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full_bar[it % NS]), (uint32_t)((it / NS) & 1))) {
                    if (clock64() - t0 > p.wait_cycles) {
                        report_fault(p.status, FAULT_GEMV_DRAIN);
                        break;
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    MegaCtx c;
    c.full_bar = full_bar, c.empty_bar = empty_bar, c.abort_flag = abort_flag, c.norm_scratch = norm_scratch, c.flag = cta_flag;
    c.red = red, c.res_s = res_s, c.act = act, c.stage_base = stage_base;
    c.it = 0, c.red_flip = 0;
    c.ct = tid - 32, c.cw = warp - 1, c.lane = lane;
    const int ct = c.ct, cw = c.cw;
    const int g4 = lane >> 2, t4 = lane & 3;
    bf16* xs = reinterpret_cast<bf16*>(act);
    const unsigned int cta_id = blockIdx.x;

    unsigned long long* trec = (ct == 0) ? trace_open(p.trace, 20u, cta_id) : nullptr;
    pdl_wait();  // hidden, the caches and the control words belong to earlier kernels of the stream
    trace_mark(trec, 3);
    // tensor parallel: the tags of this launch's two exchanges (inbox 0 after o_proj, inbox 1 after down); a fault
    // recorded earlier poisons the exchange (see tp_poisoned)
    unsigned int tp_e0 = 0u, tp_e1 = 0u;
    if (LINK) {
        // (inbox 1 one further: the chained kernels advance its epoch between their two exchanges, and a cell they
        // left behind must never carry the tag this launch waits for)
        tp_e0 = tp_next_epoch(p.link, 0), tp_e1 = tp_next_epoch(p.link, 1) + 1u;
        if (tp_poisoned(p.status)) *abort_flag = 1;
    }

    // ================================================================ phase 0: QKV projection
    // residual values of this CTA's H rows, fetched now so that no epilogue waits on a global load
    for (int i = ct; i < s.o_r1 - s.o_r0; i += kMegaConsumerThreads) res_s[i] = mega_ldcg_bf16(p.hidden + s.o_r0 + i);
    mega_stage_x<true>(p.hidden, p.H, p.in_norm_w, p.eps, xs, norm_scratch, ct, cw, lane);
    mega_gemv_phase<false>(p, c, s.q_r0, s.q_r1, p.H, p.kc_h, s.nkc_h,
                           [&](int n, float v0, float) { p.qkv[n] = __float2bfloat16_rn(v0); }, trec, 30u);
    trace_mark(trec, 5);
    mega_grid_barrier(p, c, MB_QKV);
    if (ct == 0) *gate_open = 1;  // every CTA has its QKV rows: the producer may run ahead again

    // ================================================================ phase 1: attention slice
    trec = (ct == 0) ? trace_open(p.trace, 21u, cta_id) : nullptr;
    if (s.att_nsub > 0) {
        const int G = p.G, kvh = s.att_kvh;
        // scratch (aliases the activation vector, which nobody needs during this phase)
        float* Pw = reinterpret_cast<float*>(act) + cw * 256;             // this warp's probabilities [32 keys][8 heads]
        float* alpha_s = reinterpret_cast<float*>(act + 8192) + cw * 8;   // this warp's rescale factor per head
        bf16* q_s = reinterpret_cast<bf16*>(act + 8192 + 256);            // [8][D], rows >= G are zero
        bf16* kvn_s = q_s + 8 * D;                                        // [2][D] the new token's k and v
        float* mrg_ml = reinterpret_cast<float*>(kvn_s + 2 * D);          // [8 warps][8 heads][max, sum]
        float* mrg_o = mrg_ml + 128;                                      // [8 warps][4 heads][D]
        const bool owner = s.att_split == p.nsp - 1;  // the slice that ends with the token being decoded (slot S-1)

        for (int i = ct; i < D; i += kMegaConsumerThreads) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0u, 0u, 0u, 0u);
        named_bar_sync(1, kMegaConsumerThreads);
        if (cw < G) {
            const bf16* qsrc = p.qkv + (long long)(kvh * G + cw) * D;
            float x[DPL];
#pragma unroll
            for (int j = 0; j < DPL; ++j) x[j] = mega_ldcg_bf16(qsrc + lane + j * 32);
            mega_head_norm_rope<D>(x, p.eps, p.q_norm_w, p.rope_cos, p.rope_sin, lane);
#pragma unroll
            for (int j = 0; j < DPL; ++j) q_s[cw * D + lane + j * 32] = __float2bfloat16_rn(x[j]);
        }
        if (owner) {
            const long long slot = ((long long)kvh * p.S + (p.S - 1)) * D;
            if (cw == 7) {
                const bf16* ksrc = p.qkv + p.NH * D + kvh * D;
                float x[DPL];
#pragma unroll
                for (int j = 0; j < DPL; ++j) x[j] = mega_ldcg_bf16(ksrc + lane + j * 32);
                mega_head_norm_rope<D>(x, p.eps, p.k_norm_w, p.rope_cos, p.rope_sin, lane);
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    const bf16 kn = __float2bfloat16_rn(x[j]);
                    kvn_s[lane + j * 32] = kn;
                    if (!*abort_flag) p.Kc[slot + lane + j * 32] = kn;
                }
            } else if (cw == 6) {
                const bf16* vsrc = p.qkv + (p.NH + p.NKV) * D + kvh * D;
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    const bf16 vn = __ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(vsrc + lane + j * 32)));
                    kvn_s[D + lane + j * 32] = vn;
                    if (!*abort_flag) p.Vc[slot + lane + j * 32] = vn;
                }
            }
        }
        named_bar_sync(1, kMegaConsumerThreads);

        unsigned long long* trec2 = (ct == 0) ? trace_open(p.trace, 25u, cta_id) : nullptr;  // detail: q ready | V stage landed | P.V done | record + ticket
        // A fragments of Q (rows = query heads of this kv head); element order matches the K loads below
        uint4 qf[DPL];
#pragma unroll
        for (int j = 0; j < DPL; ++j) qf[j] = *reinterpret_cast<const uint4*>(q_s + g4 * D + 32 * j + t4 * 8);
        // Every warp owns the key blocks (8 keys) cw, cw+8, cw+16, cw+24 of a sub-chunk and runs its own online
        // soft-max over them: no barrier among the warps until their results are merged at the end.
        float o[8][DPL];
#pragma unroll
        for (int h = 0; h < 8; ++h)
#pragma unroll
            for (int j = 0; j < DPL; ++j) o[h][j] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;  // statistics of head g4 (the same in the four lanes of a quad)

        for (int sub = 0; sub < s.att_nsub; ++sub) {
            const int key0 = s.att_c0 + sub * p.sub_keys;
            const int n = min(p.sub_keys, s.att_c1 - key0);
            const int nblk = (n + 7) / 8;
            const bool patch = owner && sub == s.att_nsub - 1;  // this sub-chunk ends with slot S-1
            // ---- K: scores of this warp's keys
            const int sk = c.it % NS;
            mega_mbar_wait(smem_u32(&full_bar[sk]), (uint32_t)((c.it / NS) & 1), abort_flag, p.status, FAULT_GEMV_FULL_WAIT,
                           p.wait_cycles);
            if (sub == 0) trace_mark(trec, 4);
            unsigned char* Kst = stage_base + (size_t)sk * p.stage_bytes;
            if (patch) {
                // the copy brought the stale contents of slot S-1: overwrite that row with the new token's k
                if (ct < D / 8) reinterpret_cast<uint4*>(Kst + (size_t)(n - 1) * D * 2)[ct] = reinterpret_cast<const uint4*>(kvn_s)[ct];
                named_bar_sync(1, kMegaConsumerThreads);
            }
            float sc[4][2];
            {
                float acc[4][4];  // four independent accumulator chains
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    uint4 kf[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int kb = cw + u * kMegaConsumerWarps;
                        kf[u] = make_uint4(0u, 0u, 0u, 0u);
                        if (kb < nblk) kf[u] = lds128(smem_u32(Kst) + (uint32_t)(((kb * 8 + g4) * D + t4 * 8) * 2 + 64 * j));
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) mma_bf16_16816(acc[u], qf[j].x, 0u, qf[j].y, 0u, kf[u].x, kf[u].y);
#pragma unroll
                    for (int u = 0; u < 4; ++u) mma_bf16_16816(acc[u], qf[j].z, 0u, qf[j].w, 0u, kf[u].z, kf[u].w);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int key = (cw + u * kMegaConsumerWarps) * 8 + t4 * 2;  // this lane: head g4, keys key and key + 1
                    sc[u][0] = (key < n) ? acc[u][0] * p.scale_log2e : -INFINITY;
                    sc[u][1] = (key + 1 < n) ? acc[u][1] * p.scale_log2e : -INFINITY;
                }
            }
            if (patch) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[sk]));
            ++c.it;
            // ---- online soft-max (exp2 domain) for head g4 over this warp's keys
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < 4; ++u) mx = fmaxf(mx, fmaxf(sc[u][0], sc[u][1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);
            const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float alpha = mega_exp2(m_run - m_safe);
            float psum = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float pr = mega_exp2(sc[u][e] - m_safe);
                    psum += pr;
                    Pw[(u * 8 + t4 * 2 + e) * 8 + g4] = pr;
                }
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            l_run = l_run * alpha + psum;
            m_run = m_new;
            if (t4 == 0) alpha_s[g4] = alpha;
            __syncwarp();
            // ---- V: o += P . V over this warp's keys; a lane owns DPL consecutive output dims of every head
            const int sv = c.it % NS;
            mega_mbar_wait(smem_u32(&full_bar[sv]), (uint32_t)((c.it / NS) & 1), abort_flag, p.status, FAULT_GEMV_FULL_WAIT,
                           p.wait_cycles);
            unsigned char* Vst = stage_base + (size_t)sv * p.stage_bytes;
            if (patch) {
                if (ct < D / 8) reinterpret_cast<uint4*>(Vst + (size_t)(n - 1) * D * 2)[ct] = reinterpret_cast<const uint4*>(kvn_s + D)[ct];
                named_bar_sync(1, kMegaConsumerThreads);
            }
            {
                const float4 a0 = *reinterpret_cast<const float4*>(alpha_s), a1 = *reinterpret_cast<const float4*>(alpha_s + 4);
                const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                for (int h = 0; h < 8; ++h)
#pragma unroll
                    for (int j = 0; j < DPL; ++j) o[h][j] *= al[h];
            }
            if (sub == 0) trace_mark(trec2, 3);
            {
                const uint32_t pw_a = smem_u32(Pw), v_a = smem_u32(Vst) + lane * (DPL * 2);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int kb = cw + u * kMegaConsumerWarps;
                    if (kb < nblk) {
                        // the eight keys of a block: all loads first.  Keys beyond n have probability 0 and read the
                        // row of key n-1 instead (finite values), so no branch per key is needed.
                        float4 pl[8], ph[8];
                        float v[8][DPL];
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const int key = min(kb * 8 + kk, n - 1);
                            pl[kk] = lds128f(pw_a + (uint32_t)((u * 8 + kk) * 32));
                            ph[kk] = (G > 4) ? lds128f(pw_a + (uint32_t)((u * 8 + kk) * 32 + 16)) : make_float4(0.f, 0.f, 0.f, 0.f);
                            if (DPL == 4) {
                                const uint2 raw = lds64(v_a + (uint32_t)(key * D * 2));
                                v[kk][0] = bf16_lo(raw.x), v[kk][1] = bf16_hi(raw.x), v[kk][DPL - 2] = bf16_lo(raw.y), v[kk][DPL - 1] = bf16_hi(raw.y);
                            } else {
                                const uint32_t raw = lds32(v_a + (uint32_t)(key * D * 2));
                                v[kk][0] = bf16_lo(raw), v[kk][1] = bf16_hi(raw);
                            }
                        }
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const float p4[4] = {pl[kk].x, pl[kk].y, pl[kk].z, pl[kk].w};
#pragma unroll
                            for (int h = 0; h < 4; ++h)
#pragma unroll
                                for (int j = 0; j < DPL; ++j) o[h][j] = fmaf(p4[h], v[kk][j], o[h][j]);
                        }
                        if (G > 4) {
#pragma unroll
                            for (int kk = 0; kk < 8; ++kk) {
                                const float p4[4] = {ph[kk].x, ph[kk].y, ph[kk].z, ph[kk].w};
#pragma unroll
                                for (int h = 0; h < 4; ++h)
#pragma unroll
                                    for (int j = 0; j < DPL; ++j) o[4 + h][j] = fmaf(p4[h], v[kk][j], o[4 + h][j]);
                            }
                        }
                    }
                }
            }
            if (patch) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();  // also: every lane is done with Pw before the next sub-chunk overwrites it
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[sv]));
            ++c.it;
        }
        trace_mark(trec2, 4);

        // ---- merge the eight warps (each has its own max / sum / O) and park the slice's record
        const long long item = (long long)kvh * p.nsp + s.att_split;
        if (t4 == 0) mrg_ml[(cw * 8 + g4) * 2] = m_run, mrg_ml[(cw * 8 + g4) * 2 + 1] = l_run;
        for (int hb = 0; hb < G; hb += 4) {
#pragma unroll
            for (int hh = 0; hh < 4; ++hh) {
                float* dst = mrg_o + ((cw * 4 + hh) * D + lane * DPL);
                if (hb == 0) {  // (static indexing of o[][]: hb is 0 or 4)
#pragma unroll
                    for (int j = 0; j < DPL; ++j) dst[j] = o[hh][j];
                } else {
#pragma unroll
                    for (int j = 0; j < DPL; ++j) dst[j] = o[4 + hh][j];
                }
            }
            named_bar_sync(1, kMegaConsumerThreads);
            for (int idx = ct; idx < 4 * D; idx += kMegaConsumerThreads) {
                const int hh = idx / D, d = idx - hh * D, h = hb + hh;
                if (h < G && !*abort_flag) {
                    float M = -INFINITY;
#pragma unroll
                    for (int w = 0; w < kMegaConsumerWarps; ++w) M = fmaxf(M, mrg_ml[(w * 8 + h) * 2]);
                    float O = 0.f, L = 0.f;
#pragma unroll
                    for (int w = 0; w < kMegaConsumerWarps; ++w) {
                        const float f = (M == -INFINITY) ? 0.f : mega_exp2(mrg_ml[(w * 8 + h) * 2] - M);
                        O += f * mrg_o[(w * 4 + hh) * D + d];
                        L += f * mrg_ml[(w * 8 + h) * 2 + 1];
                    }
                    p.part_o[(item * 8 + h) * D + d] = O;
                    if (d == 0) p.part_ml[(item * 8 + h) * 2] = M, p.part_ml[(item * 8 + h) * 2 + 1] = L;
                }
            }
            named_bar_sync(1, kMegaConsumerThreads);  // orders the records before the ticket; the buffer is free again
        }
        // ---- the CTA that finishes last for this kv head folds the slices together (in slice order)
        if (ct == 0) {
            unsigned int prev;
            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(p.ctrl + MB_TICKET0 + kvh) : "memory");
            *c.flag = (prev == (unsigned int)(p.nsp - 1));
        }
        named_bar_sync(1, kMegaConsumerThreads);
        trace_mark(trec2, 5);
        if (*c.flag) {
            // One output quad (head, 4 dims) is shared by `ways` neighbouring threads, each folding every ways-th
            // slice; their partial results are merged with shuffles in a fixed order.
            const int items = G * (D / 4);
            int ways = 1;
            while (ways < 8 && items * ways * 2 <= kMegaConsumerThreads) ways *= 2;
            const int it_i = ct / ways, way = ct - it_i * ways;
            const bool active = it_i < items;
            const int hq = active ? it_i / (D / 4) : 0, d = active ? (it_i - hq * (D / 4)) * 4 : 0;
            const float* pm = p.part_ml + ((long long)kvh * p.nsp * 8 + hq) * 2;
            const float* po = p.part_o + ((long long)kvh * p.nsp * 8 + hq) * D + d;
            float M = -INFINITY, L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c0 = way; c0 < p.nsp; c0 += kCombineBatch * ways) {
                float2 ml[kCombineBatch];
                float4 v[kCombineBatch];
#pragma unroll
                for (int u = 0; u < kCombineBatch; ++u) {
                    const int cc = c0 + u * ways;
                    const bool live = active && cc < p.nsp;
                    ml[u] = live ? __ldcg(reinterpret_cast<const float2*>(pm + (long long)cc * 16)) : make_float2(-INFINITY, 0.f);
                    v[u] = live ? __ldcg(reinterpret_cast<const float4*>(po + (long long)cc * 8 * D)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float Mc = M;
#pragma unroll
                for (int u = 0; u < kCombineBatch; ++u) Mc = fmaxf(Mc, ml[u].x);
                const float keep = (Mc == -INFINITY) ? 0.f : mega_exp2(M - Mc);  // M == -inf: nothing accumulated yet, exp2 gives 0
                L *= keep, acc.x *= keep, acc.y *= keep, acc.z *= keep, acc.w *= keep;
#pragma unroll
                for (int u = 0; u < kCombineBatch; ++u) {
                    const float f = (Mc == -INFINITY) ? 0.f : mega_exp2(ml[u].x - Mc);
                    L += f * ml[u].y;
                    acc.x += f * v[u].x, acc.y += f * v[u].y, acc.z += f * v[u].z, acc.w += f * v[u].w;
                }
                M = Mc;
            }
            for (int off = 1; off < ways; off <<= 1) {
                const float M2 = __shfl_xor_sync(0xffffffffu, M, off), L2 = __shfl_xor_sync(0xffffffffu, L, off);
                const float bx = __shfl_xor_sync(0xffffffffu, acc.x, off), by = __shfl_xor_sync(0xffffffffu, acc.y, off);
                const float bz = __shfl_xor_sync(0xffffffffu, acc.z, off), bw = __shfl_xor_sync(0xffffffffu, acc.w, off);
                const float Mn = fmaxf(M, M2);
                // the lower way's term first, in both partners: the sum is the same bits on both sides
                const bool low = (way & off) == 0;
                const float Ma = low ? M : M2, Mb = low ? M2 : M;
                const float fa = (Mn == -INFINITY) ? 0.f : mega_exp2(Ma - Mn), fb = (Mn == -INFINITY) ? 0.f : mega_exp2(Mb - Mn);
                L = (low ? L : L2) * fa + (low ? L2 : L) * fb;
                acc.x = (low ? acc.x : bx) * fa + (low ? bx : acc.x) * fb;
                acc.y = (low ? acc.y : by) * fa + (low ? by : acc.y) * fb;
                acc.z = (low ? acc.z : bz) * fa + (low ? bz : acc.z) * fb;
                acc.w = (low ? acc.w : bw) * fa + (low ? bw : acc.w) * fb;
                M = Mn;
            }
            const float inv = (L > 0.f) ? 1.0f / L : 0.f;
            if (active && way == 0 && !*abort_flag)
                *reinterpret_cast<uint2*>(p.attn_out + (long long)(kvh * G + hq) * D + d) =
                    make_uint2(pack_bf16(acc.x * inv, acc.y * inv), pack_bf16(acc.z * inv, acc.w * inv));
            if (ct == 0) p.ctrl[MB_TICKET0 + kvh] = 0u;  // ready for the next launch
        }
    }
    trace_mark(trec, 5);
    mega_grid_barrier(p, c, MB_ATTN);
    if (ct == 0) *gate_open = 2;

    // ================================================================ phase 2: output projection + residual
    trec = (ct == 0) ? trace_open(p.trace, 22u, cta_id) : nullptr;
    mega_stage_x<false>(p.attn_out, p.Q, nullptr, p.eps, xs, norm_scratch, ct, cw, lane);
    trace_mark(trec, 3);
    mega_gemv_phase<false>(p, c, s.o_r0, s.o_r1, p.Q, p.kc_q, s.nkc_q,
                           [&](int n, float v0, float) {
                               if (LINK) {  // this rank's partial goes into its slot of inbox 0 on every rank
                                   mega_tp_push(p.link, 0, n, v0, tp_e0);
                                   return;
                               }
                               const bf16 x2v = __float2bfloat16_rn(res_s[n - s.o_r0] + round_bf16(v0));
                               p.x2[n] = x2v;
                               res_s[n - s.o_r0] = __bfloat162float(x2v);  // the down projection adds onto this
                           },
                           trec, 32u);
    if (LINK) {
        // Two-level gather.  Every CTA needs all of x2, but polling H cells of every rank in 148 CTAs costs more L2
        // traffic than the exchange itself.  So a CTA sums the ranks' partials only for the rows it owns, stores
        // x2 = hidden + bf16(sum) for them (the same bits on every rank: rank order), and the grid barrier below then
        // publishes the complete vector to everybody, exactly as on one GPU.
        const int npair = (s.o_r1 - s.o_r0) / 2;
        const long long t0 = clock64();
        for (int pr = ct; pr < npair; pr += kMegaConsumerThreads) {
            const int n = s.o_r0 + 2 * pr;
            float add[2] = {0.f, 0.f};
            if (*abort_flag || !mega_tp_gather2(p.link, 0, tp_e0, n, add, p.status, t0)) {
                *abort_flag = 1;  // a peer never delivered: nothing of this CTA is stored or pushed from here on
                break;
            }
            const uint32_t x2w = pack_bf16(res_s[n - s.o_r0] + round_bf16(add[0]), res_s[n + 1 - s.o_r0] + round_bf16(add[1]));
            *reinterpret_cast<uint32_t*>(p.x2 + n) = x2w;
            res_s[n - s.o_r0] = bf16_lo(x2w), res_s[n + 1 - s.o_r0] = bf16_hi(x2w);  // the down projection adds onto this
        }
    }
    trace_mark(trec, 5);
    mega_grid_barrier(p, c, MB_OPROJ);
    if (ct == 0) *gate_open = 3;

    // ================================================================ phase 3: gate/up + SwiGLU
    trec = (ct == 0) ? trace_open(p.trace, 23u, cta_id) : nullptr;
    mega_stage_x<true>(p.x2, p.H, p.post_norm_w, p.eps, xs, norm_scratch, ct, cw, lane);
    trace_mark(trec, 3);
    mega_gemv_phase<true>(p, c, s.g_r0, s.g_r1, p.H, p.kc_h, s.nkc_h,
                          [&](int n, float v0, float v1) {
                              const float gate = round_bf16(v0), up = round_bf16(v1);
                              p.h[n] = __float2bfloat16_rn(round_bf16(silu_f32(gate)) * up);
                          },
                          trec, 33u);
    trace_mark(trec, 5);
    mega_grid_barrier(p, c, MB_GATEUP);
    if (ct == 0) *gate_open = 4;
    // No CTA touches a barrier counter after this point.  The CTA that gets here last returns them to zero for the
    // next launch (which reads them only after this grid has finished); doing it now keeps it off the kernel's tail.
    if (ct == 0) {
        const unsigned int prev = atomicAdd(p.ctrl + MB_EXIT, 1u);
        if (prev == gridDim.x - 1) {
            p.ctrl[MB_QKV] = 0u, p.ctrl[MB_ATTN] = 0u, p.ctrl[MB_OPROJ] = 0u, p.ctrl[MB_GATEUP] = 0u;
            p.ctrl[MB_EXIT] = 0u;
            // tensor parallel: every CTA has read both epochs long ago; the next launch tags its cells one higher
            // (not after a fault: a poisoned chain advances nothing)
            if (LINK && !*abort_flag) p.link.ctrl_peer[p.link.rank][kTpEpoch + 0] += 1u, p.link.ctrl_peer[p.link.rank][kTpEpoch + 1] += 1u;
        }
    }

    // ================================================================ phase 4: down projection + residual
    trec = (ct == 0) ? trace_open(p.trace, 24u, cta_id) : nullptr;
    mega_stage_x<false>(p.h, p.I, nullptr, p.eps, xs, norm_scratch, ct, cw, lane);
    trace_mark(trec, 3);
    mega_gemv_phase<false>(p, c, s.o_r0, s.o_r1, p.I, p.kc_i, s.nkc_i,
                           [&](int n, float v0, float) {
                               if (LINK) mega_tp_push(p.link, 1, n, v0, tp_e1);
                               else p.out[n] = __float2bfloat16_rn(res_s[n - s.o_r0] + round_bf16(v0));
                           },
                           trec, 34u);
    trace_mark(trec, 5);
    if (LINK) {
        // out = x2 + bf16(sum over ranks of the down partials) for this CTA's rows: one thread per pair of rows polls
        // the pair's cells of every rank in inbox 1 (same bits on every rank: the sum runs in rank order)
        trec = (ct == 0) ? trace_open(p.trace, 26u, cta_id) : nullptr;
        const int npair = (s.o_r1 - s.o_r0) / 2;
        const long long t0 = clock64();
        for (int pr = ct; pr < npair; pr += kMegaConsumerThreads) {
            const int n = s.o_r0 + 2 * pr;
            float add[2] = {0.f, 0.f};
            const bool ok = !*abort_flag && mega_tp_gather2(p.link, 1, tp_e1, n, add, p.status, t0);
            if (ok)
                *reinterpret_cast<uint32_t*>(p.out + n) =
                    pack_bf16(res_s[n - s.o_r0] + round_bf16(add[0]), res_s[n + 1 - s.o_r0] + round_bf16(add[1]));
        }
        trace_mark(trec, 5);
    }

}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static size_t mega_align(size_t v, size_t a) { return (v + a - 1) / a * a; }

static int mega_splits(int S, int NKV, int grid) {
    int nsp = grid / NKV;
    const int by_len = (S + 63) / 64;
    if (nsp > by_len) nsp = by_len;
    if (nsp > kMegaMaxSplits) nsp = kMegaMaxSplits;
    if (nsp < 1) nsp = 1;
    return nsp;
}

size_t decode_mega_ctrl_bytes(int NKV) { return mega_align((size_t)(MB_TICKET0 + NKV) * sizeof(unsigned int), 256); }

size_t decode_mega_workspace_bytes(int NKV, int D) {
    int nsp = sm_count() / (NKV > 0 ? NKV : 1);
    if (nsp > kMegaMaxSplits) nsp = kMegaMaxSplits;
    if (nsp < 1) nsp = 1;
    const size_t items = (size_t)NKV * nsp * 8;
    return decode_mega_ctrl_bytes(NKV) + mega_align(items * 2 * sizeof(float), 256) + mega_align(items * D * sizeof(float), 256);
}

struct MegaPlan {
    int grid, NS, kc_h, kc_q, kc_i, sub_keys, nsp;
    size_t stage_bytes, act_bytes, smem;
};

static bool mega_plan(const MegaArgs& a, MegaPlan& pl) {
    if (tuning(EZB_TUNE_MEGA) == 0) return false;
    if (a.D != 64 && a.D != 128) return false;
    if (a.NH % a.NKV) return false;
    const int G = a.NH / a.NKV, Q = a.NH * a.D;
    if (G > 8) return false;
    if (a.H % 32 || Q % 32 || a.I % 32) return false;
    const int grid = sm_count();
    if (a.NKV > grid) return false;
    if ((a.H + grid - 1) / grid + 1 > kMegaResSlots) return false;
    auto kc_of = [](int K) { return K < 4096 ? K : 4096; };
    pl.grid = grid;
    pl.kc_h = kc_of(a.H), pl.kc_q = kc_of(Q), pl.kc_i = kc_of(a.I);
    const int kc_max = pl.kc_h > pl.kc_q ? (pl.kc_h > pl.kc_i ? pl.kc_h : pl.kc_i) : (pl.kc_q > pl.kc_i ? pl.kc_q : pl.kc_i);
    pl.stage_bytes = mega_align((size_t)8 * (kc_max + kMegaRowPad) * 2, 128);
    int sub = (int)(pl.stage_bytes / ((size_t)a.D * 2)) / 8 * 8;
    if (sub > kMegaSubKeysMax) sub = kMegaSubKeysMax;
    if (sub < 8) return false;
    pl.sub_keys = sub;
    pl.nsp = mega_splits(a.S, a.NKV, grid);
    const int maxK = a.H > Q ? (a.H > a.I ? a.H : a.I) : (Q > a.I ? Q : a.I);
    const size_t xs_bytes = (size_t)maxK * 2 + 64;
    // attention scratch: probabilities 8 warps x 32 keys x 8 heads, rescale factors, q rows, new k/v, merge buffers
    const size_t attn_bytes = (size_t)8192 + 256 + (size_t)8 * a.D * 2 + (size_t)2 * a.D * 2 + 512 + (size_t)8 * 4 * a.D * 4;
    pl.act_bytes = mega_align(xs_bytes > attn_bytes ? xs_bytes : attn_bytes, 128);
    const size_t fixed = kMegaHeaderBytes + kMegaRedBytes + kMegaResSlots * sizeof(float) + pl.act_bytes;
    const size_t cap = (size_t)max_smem_optin();
    if (fixed + 2 * pl.stage_bytes > cap) return false;
    int ns = (int)((cap - fixed) / pl.stage_bytes);
    if (ns > kMegaMaxStages) ns = kMegaMaxStages;
    const int ns_cap = tuning(EZB_TUNE_MEGA_STAGES);
    if (ns_cap >= 2 && ns > ns_cap) ns = ns_cap;
    pl.NS = ns;
    pl.smem = fixed + (size_t)ns * pl.stage_bytes;
    return true;
}

bool decode_mega_supported(const MegaArgs& a) {
    MegaPlan pl;
    return mega_plan(a, pl);
}

template <int D, bool LINK>
static cudaError_t launch_mega_instance(const MegaParams& p, const MegaPlan& pl, cudaStream_t stream) {
    auto kernel = decode_layer_b1_kernel<D, LINK>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem_optin());
        if (e != cudaSuccess) return e;
        // all CTAs of the grid wait on one another: each must fit on an SM of its own
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kMegaThreads, pl.smem);
        if (e != cudaSuccess) return e;
        if (per_sm < 1) return cudaErrorLaunchOutOfResources;
        configured[dev] = true;
    }
    return launch_pdl(kernel, dim3(pl.grid), dim3(kMegaThreads), pl.smem, stream, p);
}

cudaError_t launch_decode_mega(const MegaArgs& a, cudaStream_t stream) {
    MegaPlan pl;
    if (!mega_plan(a, pl)) return cudaErrorNotSupported;
    MegaParams p;
    p.hidden = a.hidden, p.out = a.out, p.Kc = a.Kc, p.Vc = a.Vc;
    p.Wqkv = a.Wqkv, p.Wo = a.Wo, p.Wg = a.Wgu, p.Wu = a.Wgu + (size_t)a.I * a.H, p.Wd = a.Wd;
    p.in_norm_w = a.input_norm_w, p.post_norm_w = a.post_norm_w, p.q_norm_w = a.q_norm_w, p.k_norm_w = a.k_norm_w;
    p.rope_cos = a.rope_cos, p.rope_sin = a.rope_sin;
    p.qkv = a.qkv, p.attn_out = a.attn_out, p.x2 = a.x2, p.h = a.h;
    unsigned char* ws = static_cast<unsigned char*>(a.mega_workspace);
    int nsp_max = sm_count() / a.NKV;
    if (nsp_max > kMegaMaxSplits) nsp_max = kMegaMaxSplits;
    if (nsp_max < 1) nsp_max = 1;
    p.ctrl = reinterpret_cast<unsigned int*>(ws);
    p.part_ml = reinterpret_cast<float*>(ws + decode_mega_ctrl_bytes(a.NKV));
    p.part_o = reinterpret_cast<float*>(ws + decode_mega_ctrl_bytes(a.NKV) + mega_align((size_t)a.NKV * nsp_max * 8 * 2 * sizeof(float), 256));
    p.S = a.S, p.H = a.H, p.I = a.I, p.NH = a.NH, p.NKV = a.NKV, p.G = a.NH / a.NKV, p.Q = a.NH * a.D, p.R = (a.NH + 2 * a.NKV) * a.D;
    p.eps = a.eps, p.scale_log2e = 1.4426950408889634f / sqrtf((float)a.D);
    p.kc_h = pl.kc_h, p.kc_q = pl.kc_q, p.kc_i = pl.kc_i;
    p.nsp = pl.nsp, p.sub_keys = pl.sub_keys;
    p.NS = pl.NS;
    p.l2_window = tuning(EZB_TUNE_MEGA_L2_STAGES);
    if (p.l2_window < 0 || !tuning(EZB_TUNE_L2_PREFETCH)) p.l2_window = 0;
    p.evict_first = tuning(EZB_TUNE_STREAM_EVICT_FIRST);
    p.inflight = tuning(EZB_TUNE_MEGA_INFLIGHT);
    if (p.inflight < 0 || p.inflight >= p.NS) p.inflight = 0;
    p.gate = tuning(EZB_TUNE_MEGA_GATE) & 7;
    p.stage_bytes = (unsigned int)pl.stage_bytes, p.act_bytes = (unsigned int)pl.act_bytes;
    p.wait_cycles = wait_limit_cycles();
    p.status = status_ptr();
    if (!p.status) return cudaErrorUnknown;
    p.trace = trace_handle();
    p.link = a.link;
    if (a.link.world > 0) {
        if (a.D == 128) return launch_mega_instance<128, true>(p, pl, stream);
        return launch_mega_instance<64, true>(p, pl, stream);
    }
    if (a.D == 128) return launch_mega_instance<128, false>(p, pl, stream);
    return launch_mega_instance<64, false>(p, pl, stream);
}

}  // namespace ezb
