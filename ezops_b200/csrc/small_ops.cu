// The latency-bound row operators of the decode path: fp32 RMSNorm, bf16 row
// preparation (optional fp32 add, optional RMSNorm with weight) and the fused
// per-head QK-norm + RoPE + KV-cache write.  They touch well under a megabyte
// at decode sizes, so the design goal is one launch, vector loads and no second
// trip to HBM; all of them take part in programmatic dependent launch.
#include "launchers.h"

namespace ezb {

static constexpr int kRowThreads = 256;

// Sum over the block, same order on every call (warp shuffles, then a fixed
// loop over the per-warp partials).
__device__ __forceinline__ float block_sum_256(float v, float* scratch8) {
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // scratch may still be read from a previous use
    if (lane == 0) scratch8[warp] = v;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; ++w) tot += scratch8[w];
    return tot;
}

// ---------------------------------------------------------------- fp32 ----
// One CTA per row.  The row is staged in shared memory when it fits, so HBM is
// read once; longer rows are re-read (they come back from L2).
__global__ void __launch_bounds__(kRowThreads) rmsnorm_f32_kernel(const float* __restrict__ X, float* __restrict__ Out,
                                                                  int dim, float eps, int staged) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float scratch[8];
    pdl_trigger();
    pdl_wait();
    const float* x = X + (long long)blockIdx.x * dim;
    float* o = Out + (long long)blockIdx.x * dim;
    const bool vec = (dim & 3) == 0;
    float ssq = 0.f;
    if (vec) {
        for (int i = threadIdx.x; i < dim / 4; i += kRowThreads) {
            const float4 v = reinterpret_cast<const float4*>(x)[i];
            if (staged) reinterpret_cast<float4*>(row_s)[i] = v;
            ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += kRowThreads) {
            const float v = x[i];
            if (staged) row_s[i] = v;
            ssq += v * v;
        }
    }
    const float tot = block_sum_256(ssq, scratch);
    const float r = 1.0f / sqrtf(tot / (float)dim + eps);
    const float* src = staged ? row_s : x;
    if (vec) {
        for (int i = threadIdx.x; i < dim / 4; i += kRowThreads) {
            float4 v = reinterpret_cast<const float4*>(src)[i];
            v.x *= r, v.y *= r, v.z *= r, v.w *= r;
            reinterpret_cast<float4*>(o)[i] = v;
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += kRowThreads) o[i] = src[i] * r;
    }
}

cudaError_t launch_rmsnorm_f32(const float* X, float* Out, int rows, int dim, float eps, cudaStream_t stream) {
    const size_t bytes = (size_t)dim * sizeof(float);
    const int staged = bytes <= 40 * 1024;
    return launch_pdl(rmsnorm_f32_kernel, dim3(rows), dim3(kRowThreads), staged ? bytes : 0, stream, X, Out, dim, eps, staged);
}

// ---------------------------------------------------------------- bf16 ----
struct RowPrepParams {
    const bf16* x;
    long long ldx;
    const float* add;
    long long ldadd;
    bf16* sum_out;
    long long ldsum;
    const bf16* w;
    bf16* y;
    long long ldy;
    int dim;
    float eps;
    int normalize;
    TpLink link;
    unsigned int* status;
};

// `ok` turns false (and stays false) when the wait for the peers' partials ran out: the caller then stores nothing.
__device__ __forceinline__ uint4 load_row8(const RowPrepParams& p, long long row, int i, unsigned int epoch, long long t0, bool& ok) {
    uint4 raw = *reinterpret_cast<const uint4*>(p.x + row * p.ldx + i * 8);
    if (p.link.world > 0 && p.link.gather_inbox >= 0) {
        // the term to add is the sum, in rank order, of the partials in this rank's inbox
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        ok = ok && tp_gather<8, 8>(p.link, epoch, row * p.dim + i * 8, a, p.status, t0);
        raw.x = pack_bf16(bf16_lo(raw.x) + round_bf16(a[0]), bf16_hi(raw.x) + round_bf16(a[1]));
        raw.y = pack_bf16(bf16_lo(raw.y) + round_bf16(a[2]), bf16_hi(raw.y) + round_bf16(a[3]));
        raw.z = pack_bf16(bf16_lo(raw.z) + round_bf16(a[4]), bf16_hi(raw.z) + round_bf16(a[5]));
        raw.w = pack_bf16(bf16_lo(raw.w) + round_bf16(a[6]), bf16_hi(raw.w) + round_bf16(a[7]));
    } else if (p.add) {
        const float4 a0 = *reinterpret_cast<const float4*>(p.add + row * p.ldadd + i * 8);
        const float4 a1 = *reinterpret_cast<const float4*>(p.add + row * p.ldadd + i * 8 + 4);
        raw.x = pack_bf16(bf16_lo(raw.x) + round_bf16(a0.x), bf16_hi(raw.x) + round_bf16(a0.y));
        raw.y = pack_bf16(bf16_lo(raw.y) + round_bf16(a0.z), bf16_hi(raw.y) + round_bf16(a0.w));
        raw.z = pack_bf16(bf16_lo(raw.z) + round_bf16(a1.x), bf16_hi(raw.z) + round_bf16(a1.y));
        raw.w = pack_bf16(bf16_lo(raw.w) + round_bf16(a1.z), bf16_hi(raw.w) + round_bf16(a1.w));
    }
    return raw;
}

// Step input / output between pinned host memory and device memory, moved by a few CTAs instead of a copy engine:
// as a kernel the copy is an ordinary link of a programmatic-dependent-launch chain (the layer behind a copy-in
// starts streaming its weights while the input crosses PCIe; the copy-out is resident before the layer ends), and
// a graph of {copy in, layer, copy out} needs no hand-over between the copy engines and the SMs.
__global__ void __launch_bounds__(256) pinned_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16,
                                                          int to_host) {
    pdl_trigger();
    pdl_wait();  // src may be what the kernel in front wrote; dst may be what it still reads
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) dst[i] = src[i];
    if (to_host) __threadfence_system();
}

cudaError_t launch_pinned_copy(void* dst, const void* src, size_t bytes, bool to_host, cudaStream_t stream) {
    const long long n16 = (long long)(bytes / 16);
    int grid = (int)((n16 + 255) / 256);
    if (grid > 16) grid = 16;  // a step's activations are a few KB to a few hundred KB; PCIe is the limit, not SMs
    if (grid < 1) grid = 1;
    return launch_pdl(pinned_copy_kernel, dim3(grid), dim3(256), 0, stream, static_cast<const uint4*>(src), static_cast<uint4*>(dst),
                      n16, to_host ? 1 : 0);
}

__global__ void __launch_bounds__(kRowThreads) row_prep_kernel(const RowPrepParams p) {
    __shared__ float scratch[8];
    pdl_trigger();
    pdl_wait();
    const bool gather = p.link.world > 0 && p.link.gather_inbox >= 0;
    if (gather && tp_poisoned(p.status)) return;  // see tp_poisoned: the chain already gave up a wait
    const unsigned int epoch = gather ? tp_next_epoch(p.link, p.link.gather_inbox) : 0u;
    const long long t0 = clock64();
    const long long row = blockIdx.x;
    const int nvec = p.dim / 8;
    float ssq = 0.f;
    bool ok = true;
    for (int i = threadIdx.x; i < nvec; i += kRowThreads) {
        const uint4 s = load_row8(p, row, i, epoch, t0, ok);
        if (ok && p.sum_out) *reinterpret_cast<uint4*>(p.sum_out + row * p.ldsum + i * 8) = s;
        const uint32_t w[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) ssq += bf16_lo(w[e]) * bf16_lo(w[e]) + bf16_hi(w[e]) * bf16_hi(w[e]);
    }
    if (!p.y) return;
    float r = 1.f;
    if (p.normalize) {
        const float tot = block_sum_256(ssq, scratch);
        r = 1.0f / sqrtf(tot / (float)p.dim + p.eps);
    }
    for (int i = threadIdx.x; i < nvec; i += kRowThreads) {
        const uint4 s = load_row8(p, row, i, epoch, t0, ok);
        if (!ok) continue;
        uint32_t v[4] = {s.x, s.y, s.z, s.w};
        if (p.normalize) {
            uint32_t nw[4] = {0, 0, 0, 0};
            if (p.w) {
                const uint4 q = *reinterpret_cast<const uint4*>(p.w + i * 8);
                nw[0] = q.x, nw[1] = q.y, nw[2] = q.z, nw[3] = q.w;
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float lo = bf16_lo(v[e]) * r, hi = bf16_hi(v[e]) * r;
                if (p.w) lo *= bf16_lo(nw[e]), hi *= bf16_hi(nw[e]);
                v[e] = pack_bf16(lo, hi);
            }
        }
        *reinterpret_cast<uint4*>(p.y + row * p.ldy + i * 8) = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

cudaError_t launch_row_prep(const RowPrepArgs& a, cudaStream_t stream) {
    RowPrepParams p;
    p.x = a.x, p.ldx = a.ldx, p.add = a.add, p.ldadd = a.ldadd;
    p.sum_out = a.sum_out, p.ldsum = a.ldsum, p.w = a.w, p.y = a.y, p.ldy = a.ldy;
    p.dim = a.dim, p.eps = a.eps, p.normalize = a.normalize;
    p.link = a.link;
    p.status = status_ptr();
    if (!p.status) return cudaErrorUnknown;
    return launch_pdl(row_prep_kernel, dim3(a.rows), dim3(kRowThreads), 0, stream, p);
}

// ------------------------------------------------- QK-norm + RoPE + cache ---
// One warp per (batch row, head).  Lane l holds the element pairs (i, i + D/2),
// i = l, l + 32, ..., which are exactly the pairs that rotate_half mixes, so the
// rotation needs no exchange between lanes; only the sum of squares does.
// Multiplications and additions are issued one by one in the order of the torch
// reference (no fused multiply-add), so that k_out usually matches it bit for bit.
struct RopeParams {
    const bf16 *q, *k, *v, *qw, *kw, *cos, *sin;
    bf16 *K_cache, *V_cache, *q_out, *k_out;
    int B, NQ, NKV, D, S, position;
    const int* positions;
    float eps;
    unsigned int* status;
};

static constexpr int kRopeMaxPairsPerLane = 8;  // D <= 512

__global__ void __launch_bounds__(128) qk_norm_rope_kernel(const RopeParams p) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int heads = p.NQ + p.NKV;
    if (unit >= p.B * heads) return;
    const int b = unit / heads, hh = unit - b * heads;
    const bool is_q = hh < p.NQ;
    const int h = is_q ? hh : hh - p.NQ;
    const int half = p.D / 2;
    const bf16* in = is_q ? p.q + ((long long)b * p.NQ + h) * p.D : p.k + ((long long)b * p.NKV + h) * p.D;
    const bf16* w = is_q ? p.qw : p.kw;
    const bf16* vin = is_q ? nullptr : p.v + ((long long)b * p.NKV + h) * p.D;

    // The kernel is a chain of memory latencies, not bytes.  Everything that does not depend on the token's position
    // (the head, its norm weights, the v row) is requested together with the position itself; only the rotary
    // table rows wait for it: two dependent round trips instead of three.
    const int pos = p.positions ? __ldg(p.positions + b) : p.position;
    float x1[kRopeMaxPairsPerLane], x2[kRopeMaxPairsPerLane], w1[kRopeMaxPairsPerLane], w2[kRopeMaxPairsPerLane];
    bf16 v1[kRopeMaxPairsPerLane], v2[kRopeMaxPairsPerLane];
#pragma unroll
    for (int j = 0; j < kRopeMaxPairsPerLane; ++j) {
        const int i = lane + j * 32;
        x1[j] = x2[j] = w1[j] = w2[j] = 0.f;
        v1[j] = v2[j] = __float2bfloat16_rn(0.f);
        if (i < half) {
            x1[j] = __bfloat162float(in[i]);
            x2[j] = __bfloat162float(in[i + half]);
            w1[j] = __bfloat162float(__ldg(w + i));
            w2[j] = __bfloat162float(__ldg(w + i + half));
            if (!is_q) v1[j] = vin[i], v2[j] = vin[i + half];
        }
    }
    if (pos < 0 || pos >= p.S) {
        if (lane == 0) report_fault(p.status, 0x301u);
        return;
    }
    const bf16* c = p.cos + (long long)pos * p.D;
    const bf16* s = p.sin + (long long)pos * p.D;
    float c1[kRopeMaxPairsPerLane], c2[kRopeMaxPairsPerLane], s1[kRopeMaxPairsPerLane], s2[kRopeMaxPairsPerLane];
#pragma unroll
    for (int j = 0; j < kRopeMaxPairsPerLane; ++j) {
        const int i = lane + j * 32;
        c1[j] = c2[j] = s1[j] = s2[j] = 0.f;
        if (i < half) {
            c1[j] = __bfloat162float(__ldg(c + i)), c2[j] = __bfloat162float(__ldg(c + i + half));
            s1[j] = __bfloat162float(__ldg(s + i)), s2[j] = __bfloat162float(__ldg(s + i + half));
        }
    }
    float ssq = 0.f;
#pragma unroll
    for (int j = 0; j < kRopeMaxPairsPerLane; ++j)
        if (lane + j * 32 < half) ssq = __fadd_rn(ssq, __fadd_rn(__fmul_rn(x1[j], x1[j]), __fmul_rn(x2[j], x2[j])));
    ssq = warp_sum(ssq);
    const float r = 1.0f / sqrtf(__fadd_rn(ssq / (float)p.D, p.eps));

    bf16* out = is_q ? p.q_out + ((long long)b * p.NQ + h) * p.D : p.k_out + ((long long)b * p.NKV + h) * p.D;
    bf16* kslot = is_q ? nullptr : p.K_cache + (((long long)b * p.NKV + h) * p.S + pos) * p.D;
    bf16* vslot = is_q ? nullptr : p.V_cache + (((long long)b * p.NKV + h) * p.S + pos) * p.D;
#pragma unroll
    for (int j = 0; j < kRopeMaxPairsPerLane; ++j) {
        const int i = lane + j * 32;
        if (i < half) {
            const float n1 = __fmul_rn(__fmul_rn(x1[j], r), w1[j]);
            const float n2 = __fmul_rn(__fmul_rn(x2[j], r), w2[j]);
            const float o1 = __fadd_rn(__fmul_rn(n1, c1[j]), __fmul_rn(-n2, s1[j]));
            const float o2 = __fadd_rn(__fmul_rn(n2, c2[j]), __fmul_rn(n1, s2[j]));
            const bf16 r1 = __float2bfloat16_rn(o1), r2 = __float2bfloat16_rn(o2);
            out[i] = r1;
            out[i + half] = r2;
            if (!is_q) {
                kslot[i] = r1;
                kslot[i + half] = r2;
                vslot[i] = v1[j];
                vslot[i + half] = v2[j];
            }
        }
    }
}

cudaError_t launch_qk_norm_rope(const RopeArgs& a, cudaStream_t stream) {
    RopeParams p;
    p.q = a.q, p.k = a.k, p.v = a.v, p.qw = a.qw, p.kw = a.kw, p.cos = a.cos, p.sin = a.sin;
    p.K_cache = a.K_cache, p.V_cache = a.V_cache, p.q_out = a.q_out, p.k_out = a.k_out;
    p.B = a.B, p.NQ = a.NQ, p.NKV = a.NKV, p.D = a.D, p.S = a.S, p.position = a.position;
    p.positions = a.positions, p.eps = a.eps;
    p.status = status_ptr();
    if (!p.status) return cudaErrorUnknown;
    const int units = a.B * (a.NQ + a.NKV);
    return launch_pdl(qk_norm_rope_kernel, dim3((units + 3) / 4), dim3(128), 0, stream, p);
}

}  // namespace ezb
