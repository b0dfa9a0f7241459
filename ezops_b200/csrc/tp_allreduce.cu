// In-place sum of an fp32 [B, H] buffer over the ranks of one node, through peer memory: the exchange step of the
// tensor-parallel layer at batch sizes where the partials are megabytes (the reference is single-GPU and has no
// counterpart; the library call this replaces is NCCL's all-reduce between the three local parts of the layer).
//
// Two-shot, one kernel per rank, 64 CTAs, and no flag and no fence anywhere: values travel as the epoch-tagged 64-bit
// cells of the fused exchange (common.cuh: value and tag in one word, plain peer stores, consumers poll their own
// memory).  Rank r owns the slice [r, r+1) * n / world of the elements.  Inbox `which` of a rank's communication
// buffer has one [B, H] slot of cells per sender.
//   1. scatter: every rank stores each element of its partial, as a cell, into its slot on the element's owner
//      (its own slice into its own buffer);
//   2. reduce: a rank polls, for the elements it owns, the cells of all senders (all ranks in flight together), adds
//      them in rank order - every element is computed once, by its owner, so all ranks end with identical bits - and
//   3. gather: stores the sum, as a cell again, into its slot on every other rank, at the element's own index (a
//      sender's slot is used for the partials of the receiver's slice and for the sums of the sender's slice:
//      disjoint index ranges), and as a plain float into the local buffer;
//   4. for the elements it does not own, a rank polls the owner's cell and stores the value into the local buffer.
// When the kernel has finished, the local buffer holds the sum.  In place is safe: an element is overwritten only
// after the cells derived from it have been consumed.  The CTA that leaves last (a ticket in the control block)
// advances the exchange's epoch, so the kernel replays from a CUDA graph.  A first version used release/acquire
// flags around 16-byte peer loads and stores of plain floats: one system-scope fence per CTA made it 19.5 us per
// exchange on two GPUs (NCCL: 27 alone, but faster than that inside the layer), a fence per polling thread 43 us.
// A rank can overwrite a peer's cells only after the peer has consumed them: the other exchange of the layer, in
// which every rank needs every other rank's cells, lies in between (ranks make the same sequence of calls, which
// alternates `which`).  The epochs are this kernel's own words of the control block, so a communication buffer must
// not be shared with the fused exchange (a cell left by one could carry the tag the other waits for).  Every wait is bounded (EZB_TUNE_TP_WAIT_LIMIT_MS); one that runs out records
// FAULT_AR_FLAG_WAIT and the thread stops storing; a recorded fault makes later exchanges return at once.
#include "launchers.h"

namespace ezb {

static constexpr int kArCtas = 64;
static constexpr int kArThreads = 256;

// control block (unsigned int words), behind the two epoch words of the fused exchange
static constexpr int kArEpoch = 2;   // [2]: epoch of exchange 0 / 1
static constexpr int kArTicket = 4;  // [2]: exit tickets
static_assert((kArTicket + 2) * 4 <= kTpCtrlBytes, "control block too small");

struct ArParams {
    TpLink link;
    int which;
    float* buf;    // local fp32 [n]: partial in, sum out
    long long n4;  // 16-byte elements
    unsigned int* status;
};

__device__ __forceinline__ unsigned long long ar_cell(float v, unsigned int epoch) {
    return ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
}
// four neighbouring cells (32 bytes) at dst
__device__ __forceinline__ void ar_store4(unsigned long long* dst, const float4& v, unsigned int epoch, int strong) {
    const unsigned long long c0 = ar_cell(v.x, epoch), c1 = ar_cell(v.y, epoch), c2 = ar_cell(v.z, epoch), c3 = ar_cell(v.w, epoch);
    if (strong) {
        tp_store_cell(dst, c0, 1), tp_store_cell(dst + 1, c1, 1), tp_store_cell(dst + 2, c2, 1), tp_store_cell(dst + 3, c3, 1);
    } else {
        asm volatile("st.weak.global.v2.u64 [%0], {%1, %2};" ::"l"(dst), "l"(c0), "l"(c1) : "memory");
        asm volatile("st.weak.global.v2.u64 [%0], {%1, %2};" ::"l"(dst + 2), "l"(c2), "l"(c3) : "memory");
    }
}

__global__ void __launch_bounds__(kArThreads) tp_allreduce_kernel(const ArParams p) {
    __shared__ int live_s;
    pdl_wait();  // the projection in front has written the partial
    const TpLink& l = p.link;
    unsigned int* ctrl = l.ctrl_peer[l.rank];
    const int tid = threadIdx.x;
    const unsigned int epoch = ctrl[kArEpoch + p.which] + 1u;
    if (tid == 0) live_s = tp_poisoned(p.status) ? 0 : 1;  // one read per CTA: the branch below is uniform
    __syncthreads();
    if (!live_s) return;  // a fault recorded earlier: neither store, poll nor advance anything
    const int W = l.world, me = l.rank;
    const long long gtid = (long long)blockIdx.x * kArThreads + tid, nthr = (long long)kArCtas * kArThreads;
    const long long s0 = p.n4 * me / W, s1 = p.n4 * (me + 1) / W;
    const long long slot_me = ((long long)p.which * kTpSlots + me) * l.slot_elems;
    const float4* in4 = reinterpret_cast<const float4*>(p.buf);
    float4* out4 = reinterpret_cast<float4*>(p.buf);

    // 1. scatter
    {
        int q = 0;
        long long q_end = p.n4 / W;  // = n4 * 1 / W
        for (long long i = gtid; i < p.n4; i += nthr) {
            while (i >= q_end) ++q, q_end = p.n4 * (q + 1) / W;
            ar_store4(l.inbox_peer[q] + slot_me + 4 * i, __ldcg(in4 + i), epoch, l.strong_stores);
        }
    }
    // 2. + 3. reduce the slice this rank owns and hand the sums out
    const long long t0 = clock64();
    bool ok = true;
    for (long long i = s0 + gtid; i < s1 && ok; i += nthr) {
        float add[4] = {0.f, 0.f, 0.f, 0.f};
        ok = tp_gather_from<8, 4>(l, p.which, false, epoch, 4 * i, add, p.status, t0);
        if (!ok) break;
        const float4 sum = make_float4(add[0], add[1], add[2], add[3]);
        out4[i] = sum;
        for (int w = 0; w < W; ++w)
            if (w != me) ar_store4(l.inbox_peer[w] + slot_me + 4 * i, sum, epoch, l.strong_stores);
    }
    // Every rank has arrived once this CTA's share of the slice is summed: from here on the kernel behind may
    // start (its own bounded waits must not run while this one still waits for a rank that is seconds late).
    pdl_trigger();
    // 4. the other ranks' slices
    {
        int q = 0;
        long long q_end = p.n4 / W;
        const unsigned long long* mine = l.inbox_peer[me] + (long long)p.which * kTpSlots * l.slot_elems;
        for (long long i = gtid; i < p.n4 && ok; i += nthr) {
            while (i >= q_end) ++q, q_end = p.n4 * (q + 1) / W;
            if (q == me) {  // jump over the own slice, keeping the thread's stride
                const long long skip = (s1 - i + nthr - 1) / nthr;
                i += (skip - 1) * nthr;
                continue;
            }
            const unsigned long long* src = mine + (long long)q * l.slot_elems + 4 * i;
            unsigned long long c0, c1, c2, c3;
            for (;;) {
                asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(c0), "=l"(c1) : "l"(src) : "memory");
                asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(c2), "=l"(c3) : "l"(src + 2) : "memory");
                if ((unsigned int)(c0 >> 32) == epoch && (unsigned int)(c1 >> 32) == epoch && (unsigned int)(c2 >> 32) == epoch &&
                    (unsigned int)(c3 >> 32) == epoch)
                    break;
                if (clock64() - t0 > l.wait_cycles) {
                    report_fault(p.status, FAULT_AR_FLAG_WAIT);
                    ok = false;
                    break;
                }
            }
            if (ok)
                out4[i] = make_float4(__uint_as_float((unsigned int)c0), __uint_as_float((unsigned int)c1),
                                      __uint_as_float((unsigned int)c2), __uint_as_float((unsigned int)c3));
        }
    }
    if (!ok) live_s = 0;
    __syncthreads();
    // exit ticket: every CTA has read the epoch before it gets here, so the last one may advance it
    if (tid == 0) {
        const unsigned int prev = atomicAdd(ctrl + kArTicket + p.which, 1u);
        if (prev == (unsigned int)(kArCtas - 1)) {
            ctrl[kArTicket + p.which] = 0u;
            if (!tp_poisoned(p.status)) ctrl[kArEpoch + p.which] = epoch;
        }
    }
}

cudaError_t launch_tp_allreduce(float* buf, const TpLink& link, int which, long long n, cudaStream_t stream) {
    ArParams p;
    p.link = link;
    p.which = which;
    p.buf = buf;
    p.n4 = n / 4;
    p.status = status_ptr();
    if (!p.status) return cudaErrorUnknown;
    return launch_pdl(tp_allreduce_kernel, dim3(kArCtas), dim3(kArThreads), 0, stream, p);
}

}  // namespace ezb
