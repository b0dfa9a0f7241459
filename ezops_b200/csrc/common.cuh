// Shared device helpers for the sm_100a kernels of this library: PTX wrappers
// (mbarrier, 1-D bulk TMA copies, cp.async, ldmatrix, mma, programmatic
// dependent launch), bf16 packing, the bounded barrier wait and the device
// status word.  Everything here is header-only and internal to csrc/.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ezb200.h"

namespace ezb {

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------
// Device status word.  A kernel that gives up on a wait stores a non-zero code
// here (first writer wins) and finishes without touching its outputs further;
// the host reads it with ezb_device_status().  The word is defined once (in
// api.cu); kernels receive its device address in their parameter block.
// ---------------------------------------------------------------------------

enum DeviceFault : unsigned int {
    FAULT_NONE = 0,
    FAULT_GEMV_FULL_WAIT = 0x101,   // consumer never saw a weight stage arrive
    FAULT_GEMV_EMPTY_WAIT = 0x102,  // producer never got a stage back
    FAULT_GEMV_DRAIN = 0x103,       // copies still in flight at exit
    FAULT_TC_ACC_WAIT = 0x104,      // tensor-memory accumulator hand-over never happened
    FAULT_AR_FLAG_WAIT = 0x201,     // a peer's partial result never arrived in the inbox
    FAULT_PAGE_RANGE = 0x302,       // a page-table entry points outside the page pools
    FAULT_MEGA_GRID_BARRIER = 0x400,  // + barrier index: a grid-wide barrier of the single-kernel layer never filled
};

__device__ __forceinline__ void report_fault(unsigned int* status, unsigned int code) {
    atomicCAS(status, 0u, code);
}

// About one second at B200 clocks; no legitimate wait in this library comes
// within five orders of magnitude of it.
static constexpr long long kWaitLimitCycles = 2000000000LL;

// ---------------------------------------------------------------------------
// Tensor-parallel exchange over peer memory (one-shot all-reduce split between
// the kernel that produces a partial result and the kernel that consumes the
// sum).  Every rank owns one buffer, mapped by all ranks:
//   control words (u32): [0],[1] epoch of inbox 0 / 1;
//   then two inboxes of 8 slots x slot_elems 64-bit cells: slot r of an inbox
//   holds the partial [B, H] that rank r pushed, every cell = {fp32 value in
//   the low half, epoch in the high half}.
// A producer stores each fp32 output, tagged with epoch+1, into slot `rank` of
// the chosen inbox of EVERY rank: one plain 64-bit peer store per value over NVLink,
// single-copy atomic, no fence and no flag behind it.  A consumer polls the cells
// of its own inbox (bounded) until their tag shows epoch+1 and adds the values
// in rank order, so every rank computes the same bits; a value is usable the
// moment its own store lands.  Epochs live on the device and are advanced by a
// later kernel of the chain, so a captured CUDA graph can be replayed.
// Two directions.  Push (the default): the producer stores into slot `rank` on every rank and
// consumers poll their own memory, so a value crosses NVLink once per peer however many CTAs
// read it.  Pull (EZB_TUNE_TP_PULL): the producer writes slot `rank` of its OWN buffer only and
// consumers poll slot w of rank w's buffer with peer loads.  Measured on two GPUs (us per layer,
// Qwen3-8B batch 32 KV 4096 | Qwen3-32B batch 64 KV 8192): NCCL all-reduce between the parts 162 | 345,
// push 168 | 408, pull 200 | 433 - with the stream-K split only the 32-40 CTAs that finish a tile store,
// 32-64 KB each, which takes them 16-22 us; at batch <= 8 (every CTA stores a few values) push is the fast one.
// ---------------------------------------------------------------------------
struct TpLink {
    int world;  // 0: no fused exchange
    int rank;
    unsigned int* ctrl_peer[8];
    unsigned long long* inbox_peer[8];
    long long slot_elems;
    int push_inbox;    // -1 or the inbox this kernel's outputs are pushed into
    int gather_inbox;  // -1 or the inbox whose slots this kernel's prologue sums
    int bump_inbox;    // -1 or the inbox whose epoch this kernel advances
    int poll_all;      // 1: the gathering prologue polls all ranks together, 4 elements per thread and step
    int pull;          // 1: a producer writes only its own buffer and consumers read every rank's buffer over NVLink
    long long wait_cycles;  // budget of one wait for the peers' partials (from EZB_TUNE_TP_WAIT_LIMIT_MS)
    int strong_stores;      // 1: cells are published with st.relaxed.sys (see tp_push)
};
// A recorded fault poisons the exchange: kernels that take part in it read the status word when they start and,
// if it is set, neither gather, push nor advance an epoch, so that a rank that gave up on a wait never hands its
// peers numbers computed from a partial sum (the peers then run into their own wait limit and report it too).
__device__ __forceinline__ bool tp_poisoned(const unsigned int* status) {
    return *reinterpret_cast<const volatile unsigned int*>(status) != 0u;
}
static constexpr int kTpEpoch = 0;
static constexpr int kTpCtrlBytes = 256;  // epochs of the fused exchange [0..1], epochs and exit tickets of tp_allreduce.cu [2..5]
static constexpr int kTpSlots = 8;

__device__ __forceinline__ unsigned long long* tp_slot(const TpLink& l, int on_rank, int inbox, int slot) {
    return l.inbox_peer[on_rank] + ((long long)inbox * kTpSlots + slot) * l.slot_elems;
}
// The tag the next push into / poll of `inbox` uses.
__device__ __forceinline__ unsigned int tp_next_epoch(const TpLink& l, int inbox) {
    return l.ctrl_peer[l.rank][kTpEpoch + inbox] + 1u;
}
// Publishing a cell.  Default: a plain (weak) 64-bit store.  Value and tag travel in one naturally aligned word and the
// consumer polls with strong system-scope loads.  This is a HARDWARE ASSUMPTION, not a guarantee of the PTX memory
// model: a weak store racing with a strong load is formally a data race, and the model promises neither that the 8
// bytes land together nor when they become visible.  On the GPUs this library targets an aligned 8-byte store is
// performed as one transaction (what the tests on 2, 4 and 8 GPUs exercise), and a weak store is posted - a thread can
// have many in flight - whereas with st.relaxed.sys a thread's stores to a peer went out one NVLink round trip at a
// time (64 of them cost the tensor-core epilogue 30 us).  `strong_stores` (EZB_TUNE_TP_STRONG_STORES) selects the
// conforming form, st.relaxed.sys.u64 per cell, for platforms where the assumption is in doubt; both forms are tested.
// The 16-byte form below is two independent cells whose halves may land separately; the per-cell tag check of the
// consumer tolerates that by construction.
__device__ __forceinline__ void tp_store_cell(unsigned long long* dst, unsigned long long cell, int strong) {
    if (strong) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(cell) : "memory");
    else asm volatile("st.weak.global.u64 [%0], %1;" ::"l"(dst), "l"(cell) : "memory");
}
__device__ __forceinline__ void tp_push(const TpLink& l, long long elem, float v, unsigned int epoch) {
    const unsigned long long cell = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
    for (int w = 0; w < l.world; ++w)
        if (!l.pull || w == l.rank) tp_store_cell(tp_slot(l, w, l.push_inbox, l.rank) + elem, cell, l.strong_stores);
}
// Two neighbouring cells (elem even) in one 16-byte store; each 64-bit half is a cell of its own.
__device__ __forceinline__ void tp_push2(const TpLink& l, long long elem, float v0, float v1, unsigned int epoch) {
    const unsigned long long c0 = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v0);
    const unsigned long long c1 = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v1);
    for (int w = 0; w < l.world; ++w)
        if (!l.pull || w == l.rank) {
            unsigned long long* dst = tp_slot(l, w, l.push_inbox, l.rank) + elem;
            if (l.strong_stores) {
                tp_store_cell(dst, c0, 1);
                tp_store_cell(dst + 1, c1, 1);
            } else {
                asm volatile("st.weak.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(c0), "l"(c1) : "memory");
            }
        }
}
// Called by exactly one thread of the grid, anywhere in the kernel.
__device__ __forceinline__ void tp_bump(const TpLink& l) { l.ctrl_peer[l.rank][kTpEpoch + l.bump_inbox] += 1u; }

// add[0..E-1] += sum over ranks (in rank order) of the E consecutive cells starting at `elem` of this
// rank's inbox; polls until every cell carries `epoch`, G ranks at a time (G x E 64-bit registers).
// Returns false (and records the fault) if the wait limit ran out.
// tp_gather_from names the inbox and the direction itself (a kernel that gathers from more than one inbox).
template <int G, int E>
__device__ __forceinline__ bool tp_gather_from(const TpLink& l, int inbox, bool pull, unsigned int epoch, long long elem,
                                               float (&add)[E], unsigned int* status, long long t0) {
    static_assert(E % 2 == 0, "cells are fetched in pairs");
    for (int w0 = 0; w0 < l.world; w0 += G) {
        unsigned long long c[G][E];
        unsigned int pending = 0;
#pragma unroll
        for (int g = 0; g < G; ++g)
            if (w0 + g < l.world) pending |= 1u << g;
        while (true) {
#pragma unroll
            for (int g = 0; g < G; ++g)
                if (pending & (1u << g)) {
                    const unsigned long long* src = tp_slot(l, pull ? w0 + g : l.rank, inbox, w0 + g) + elem;
#pragma unroll
                    for (int q = 0; q < E / 2; ++q)
                        asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];"
                                     : "=l"(c[g][2 * q]), "=l"(c[g][2 * q + 1])
                                     : "l"(src + 2 * q)
                                     : "memory");
                }
#pragma unroll
            for (int g = 0; g < G; ++g)
                if (pending & (1u << g)) {
                    bool all = true;
#pragma unroll
                    for (int e = 0; e < E; ++e) all = all && ((unsigned int)(c[g][e] >> 32) == epoch);
                    if (all) pending &= ~(1u << g);
                }
            if (!pending) break;
            if (clock64() - t0 > l.wait_cycles) {
                report_fault(status, FAULT_AR_FLAG_WAIT);
                return false;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g)
            if (w0 + g < l.world) {
#pragma unroll
                for (int e = 0; e < E; ++e) add[e] += __uint_as_float((unsigned int)c[g][e]);
            }
    }
    return true;
}
template <int G, int E>
__device__ __forceinline__ bool tp_gather(const TpLink& l, unsigned int epoch, long long elem, float (&add)[E],
                                          unsigned int* status, long long t0) {
    return tp_gather_from<G, E>(l, l.gather_inbox, l.pull != 0, epoch, elem, add, status, t0);
}

// ---------------------------------------------------------------------------
// Optional timeline tracing (off unless ezb_trace_enable() was called): thread 0
// of every CTA records %globaltimer at entry, after the dependency wait, when
// its first data arrived and at exit.  One record = 6 x u64:
// {kernel id, block index, t_entry, t_dep, t_data, t_exit} in nanoseconds.
// ---------------------------------------------------------------------------
struct Trace {
    unsigned long long* buf;
    unsigned int* cursor;
    unsigned int capacity;
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned long long* trace_open(const Trace& tr, unsigned int kernel_id, unsigned int block) {
    if (!tr.buf) return nullptr;
    const unsigned int slot = atomicAdd(tr.cursor, 1u);
    if (slot >= tr.capacity) return nullptr;
    unsigned long long* r = tr.buf + (size_t)slot * 6;
    r[0] = kernel_id, r[1] = block, r[2] = global_ns(), r[3] = 0, r[4] = 0, r[5] = 0;
    return r;
}
__device__ __forceinline__ void trace_mark(unsigned long long* rec, int field) {
    if (rec) rec[field] = global_ns();
}

// ---------------------------------------------------------------------------
// Address helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking probe of the phase with the given parity (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for the phase with the given parity, for at most kWaitLimitCycles.
// `abort_flag` lives in shared memory: once any thread of the CTA has given
// up, every later wait in the CTA returns at once, so the control flow of all
// warps (and the named barriers they meet at) stays the same and the CTA runs
// to its end without hanging.  Returns false when it gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned int* status, unsigned int fault_code) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitLimitCycles) {
            *abort_flag = 1;
            report_fault(status, fault_code);
            return false;
        }
    }
}

// ---------------------------------------------------------------------------
// 1-D bulk copy global -> shared through the TMA unit, completion counted in
// bytes on an mbarrier.  Both addresses 16-byte aligned, size a multiple of 16.
// ---------------------------------------------------------------------------
// `policy` (0 = none) is an L2 cache policy from l2_evict_first_policy(): lines a kernel reads once are marked as the
// first to be replaced, so a long stream recycles its own lines instead of pushing everything else - dirty lines
// that would first have to be written back included - out of L2.
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar,
                                         unsigned long long policy = 0ull) {
    if (policy)
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst_smem),
            "l"(src), "r"(bytes), "r"(bar), "l"(policy)
            : "memory");
    else
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
            "l"(src), "r"(bytes), "r"(bar)
            : "memory");
}

// ---------------------------------------------------------------------------
// L2 prefetch of what the NEXT kernel of a chain will stream first.  A kernel
// whose own requests are all issued (or that is latency-bound anyway) asks the
// memory system to pull the successor's leading weight bytes into L2, so HBM
// keeps working across the kernel boundary and the successor's ring fills from
// L2.  `units` contiguous units of `unit_bytes` are split over `next_grid` CTAs
// the way the successor splits its rows; each share is capped at `cap_units`.
// ---------------------------------------------------------------------------
struct PrefetchPlan {
    const void* base[2];
    long long unit_bytes;
    int units;
    int next_grid;
    int cap_units;
    int skip_units;  // leading units of every share that an earlier kernel already pulled
};
struct PrefetchList {
    PrefetchPlan plan[2];
};

__device__ __forceinline__ void prefetch_l2_bulk(const void* ptr, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(bytes) : "memory");
}

// Called by one warp; CTA `cta` of `grid` takes the shares cta, cta+grid, ...
__device__ __forceinline__ void prefetch_next_operand(const PrefetchPlan& pf, int lane, int cta, int grid) {
    if (pf.units <= 0 || pf.next_grid <= 0) return;
    constexpr long long kPiece = 16384;
    for (int c = cta; c < pf.next_grid; c += grid) {
        const long long u0 = (long long)pf.units * c / pf.next_grid + pf.skip_units;
        const long long u1 = (long long)pf.units * (c + 1) / pf.next_grid;
        long long n = u1 - u0;
        if (n <= 0) continue;
        if (n > pf.cap_units) n = pf.cap_units;
        const long long bytes = n * pf.unit_bytes;
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            if (!pf.base[m]) continue;
            const char* b = static_cast<const char*>(pf.base[m]) + u0 * pf.unit_bytes;
            for (long long off = (long long)lane * kPiece; off < bytes; off += 32 * kPiece) {
                const long long left = bytes - off;
                prefetch_l2_bulk(b + off, (uint32_t)(left < kPiece ? left : kPiece));
            }
        }
    }
}

__device__ __forceinline__ void prefetch_next_operands(const PrefetchList& l, int lane, int cta, int grid) {
    prefetch_next_operand(l.plan[0], lane, cta, grid);
    prefetch_next_operand(l.plan[1], lane, cta, grid);
}

// ---------------------------------------------------------------------------
// cp.async (16-byte, L2 only) with zero fill when `valid` is false
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, bool valid) {
    const int src_bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  `pdl_wait` blocks until every kernel this
// launch depends on has finished and its writes are visible; `pdl_trigger`
// lets the next kernel in the stream begin its independent prologue.
// Both are no-ops when the launch carries no programmatic dependency.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------
// Named barrier among a subset of warps
// ---------------------------------------------------------------------------
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------
// ldmatrix / mma.sync m16n8k16 bf16 -> fp32
// ---------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------
// bf16 helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t packed) { return __uint_as_float(packed << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t packed) { return __uint_as_float(packed & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// silu in fp32 as torch computes it for a bf16 tensor: x / (1 + exp(-x))
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

}  // namespace ezb

// ---------------------------------------------------------------------------
// Host-side helpers
// ---------------------------------------------------------------------------
#define EZB_CUDA_TRY(expr)                         \
    do {                                           \
        cudaError_t _e = (expr);                   \
        if (_e != cudaSuccess) {                   \
            ezb::set_last_cuda_error(_e);          \
            return EZB_ERR_CUDA;                   \
        }                                          \
    } while (0)

#define EZB_REQUIRE(cond, msg)                     \
    do {                                           \
        if (!(cond)) {                             \
            ezb::set_last_message(msg);            \
            return EZB_ERR_INVALID_ARGUMENT;       \
        }                                          \
    } while (0)

#define EZB_REQUIRE_SHAPE(cond, msg)               \
    do {                                           \
        if (!(cond)) {                             \
            ezb::set_last_message(msg);            \
            return EZB_ERR_UNSUPPORTED_SHAPE;      \
        }                                          \
    } while (0)

namespace ezb {
void set_last_cuda_error(cudaError_t e);
void set_last_message(const char* msg);
int sm_count();               // SMs of the current device (cached per device)
int max_smem_optin();         // opt-in shared memory per block of the current device
int tuning(int key);          // value of a tuning knob (see EZB_TUNE_* in ezb200.h)
long long wait_limit_cycles();  // cycle budget of one device-side wait in the kernels that take it as a parameter
unsigned int* status_ptr();   // device address of the status word on the current device (null on error)
Trace trace_handle();         // tracing buffers of the current device (buf == null when disabled)
void chain_begin();           // marks the next launch_pdl() of this thread as the first kernel of a call
bool chain_take_first();      // true once after chain_begin()
void count_launch();          // one more kernel launch issued by the library (ezb_launch_count)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launch with the programmatic-stream-serialization attribute, so that the
// kernel may start while its predecessor in the stream drains; every kernel
// launched this way calls pdl_wait() before it reads or writes anything the
// predecessor touches.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    const bool first = chain_take_first();
    const bool early_start = tuning(EZB_TUNE_PDL) && (!first || tuning(EZB_TUNE_PDL_ACROSS_CALLS));
    attr[0].val.programmaticStreamSerializationAllowed = early_start ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    count_launch();
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace ezb
