// The reference's three small teaching operators as sm_100a kernels, for API
// completeness: vector_add (ezops/ops/vector_add.py:7-30), softmax over the last
// dimension of an fp32 matrix (ezops/ops/softmax.py:7-36) and the sum of an fp32
// vector (ezops/ops/reduce.py:7-33).  All three are memory- or latency-bound.
#include <cuda_runtime.h>

#include "common.cuh"
#include "launchers.h"

namespace ezb {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum / max over the 256 threads of a CTA in a fixed order (bit-reproducible).
__device__ __forceinline__ float block_reduce(float v, float* scratch8, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads();  // scratch may still be read from a previous call
    if ((threadIdx.x & 31) == 0) scratch8[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = scratch8[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; ++w) r = is_max ? fmaxf(r, scratch8[w]) : r + scratch8[w];
    return r;
}

// ------------------------------------------------------------- vector add ---
__global__ void __launch_bounds__(kThreads) vector_add_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                              float* __restrict__ C, long long n, int vec) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const long long n4 = n / 4;
        for (long long j = i; j < n4; j += stride) {
            const float4 a = reinterpret_cast<const float4*>(A)[j], b = reinterpret_cast<const float4*>(B)[j];
            reinterpret_cast<float4*>(C)[j] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        }
        for (long long j = n4 * 4 + i; j < n; j += stride) C[j] = A[j] + B[j];
    } else {
        for (; i < n; i += stride) C[i] = A[i] + B[i];
    }
}

// ---------------------------------------------------------------- softmax ---
// One CTA per row; the row is staged in shared memory when it fits, so HBM is read once.
// expf (not the approximate exp2) keeps the result within 1e-6 of torch's.
__global__ void __launch_bounds__(kThreads) softmax_f32_kernel(const float* __restrict__ X, float* __restrict__ Out, int dim,
                                                               int staged) {
    extern __shared__ __align__(16) float row_s[];
    __shared__ float scratch[8];
    const float* x = X + (long long)blockIdx.x * dim;
    float* o = Out + (long long)blockIdx.x * dim;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < dim; i += kThreads) {
        const float v = x[i];
        if (staged) row_s[i] = v;
        m = fmaxf(m, v);
    }
    m = block_reduce(m, scratch, true);
    const float* src = staged ? row_s : x;
    float s = 0.f;
    for (int i = threadIdx.x; i < dim; i += kThreads) {
        const float e = expf(src[i] - m);
        if (staged) row_s[i] = e;
        s += e;
    }
    s = block_reduce(s, scratch, false);
    const float inv = 1.0f / s;
    for (int i = threadIdx.x; i < dim; i += kThreads) o[i] = (staged ? row_s[i] : expf(x[i] - m)) * inv;
}

// ----------------------------------------------------------------- reduce ---
// Every CTA sums a grid-strided share; the last CTA to finish (one ticket) adds the
// per-CTA partials in index order, so the result does not depend on arrival order.
__global__ void __launch_bounds__(kThreads) reduce_sum_f32_kernel(const float* __restrict__ A, float* __restrict__ Out,
                                                                  long long n, int vec, float* __restrict__ partials,
                                                                  unsigned int* __restrict__ ticket) {
    __shared__ float scratch[8];
    __shared__ int last;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    float s = 0.f;
    if (vec) {
        const long long n4 = n / 4;
        for (long long j = i0; j < n4; j += stride) {
            const float4 a = reinterpret_cast<const float4*>(A)[j];
            s += (a.x + a.y) + (a.z + a.w);
        }
        for (long long j = n4 * 4 + i0; j < n; j += stride) s += A[j];
    } else {
        for (long long j = i0; j < n; j += stride) s += A[j];
    }
    s = block_reduce(s, scratch, false);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = s;
        unsigned int prev;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(ticket) : "memory");
        last = (prev == gridDim.x - 1) ? 1 : 0;
        if (last) *ticket = 0u;  // ready for the next launch
    }
    __syncthreads();
    if (!last) return;
    float t = 0.f;
    for (int c = threadIdx.x; c < (int)gridDim.x; c += kThreads) t += __ldcg(partials + c);
    t = block_reduce(t, scratch, false);
    if (threadIdx.x == 0) Out[0] = t;
}

}  // namespace

cudaError_t launch_vector_add_f32(const float* A, const float* B, float* C, long long n, cudaStream_t stream) {
    const int vec = aligned16(A) && aligned16(B) && aligned16(C);
    long long blocks = (n / 4 + kThreads - 1) / kThreads;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    count_launch();
    vector_add_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(A, B, C, n, vec);
    return cudaGetLastError();
}

cudaError_t launch_softmax_f32(const float* X, float* Out, int rows, int dim, cudaStream_t stream) {
    const size_t bytes = (size_t)dim * sizeof(float);
    // The 48 KB a launch may use without an opt-in attribute cover static + dynamic shared memory, and the kernel
    // holds a few static words (the reduction scratch): leave 1 KB for them.
    const int staged = bytes <= 47 * 1024;
    count_launch();
    softmax_f32_kernel<<<rows, kThreads, staged ? bytes : 0, stream>>>(X, Out, dim, staged);
    return cudaGetLastError();
}

size_t reduce_workspace_bytes() { return 4096; }  // up to 1000 partials + the ticket

cudaError_t launch_reduce_sum_f32(const float* A, float* Out, long long n, void* workspace, cudaStream_t stream) {
    const int vec = aligned16(A);
    long long blocks = (n / 4 + kThreads - 1) / kThreads;
    long long cap = (long long)sm_count() * 4;
    if (cap > 1000) cap = 1000;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    float* partials = static_cast<float*>(workspace);
    unsigned int* ticket = reinterpret_cast<unsigned int*>(static_cast<unsigned char*>(workspace) + 4000);
    count_launch();
    reduce_sum_f32_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(A, Out, n, vec, partials, ticket);
    return cudaGetLastError();
}

}  // namespace ezb
