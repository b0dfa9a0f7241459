// STREAM-style bandwidth kernels used to calibrate the HBM roofline of a GPU
// profile: read, write, copy and triad (a = b + s*c) over 128-bit elements.
// Same four measurements as the reference's calibrator
// (benchmarks/hardware/memory/hbm_saturation.cu:49-93), written for a
// persistent grid: `blocks_per_sm` x SM-count blocks walk the array with a
// grid stride, four independent 128-bit accesses per thread and step.
#include <cuda_runtime.h>

#include "common.cuh"
#include "launchers.h"

namespace ezb {
namespace {

constexpr int kUnroll = 4;

template <int OP>  // 0 read, 1 write, 2 copy, 3 triad
__global__ void hbm_stream_kernel(const float4* __restrict__ b, const float4* __restrict__ c, float4* __restrict__ a,
                                  long long n, float s, float* __restrict__ sink) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    float keep = 0.f;
    for (; i + (kUnroll - 1) * stride < n; i += kUnroll * stride) {
        float4 vb[kUnroll], vc[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (OP == 0 || OP == 2 || OP == 3) vb[u] = b[i + u * stride];
            if (OP == 3) vc[u] = c[i + u * stride];
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (OP == 0) keep += vb[u].x + vb[u].y + vb[u].z + vb[u].w;
            if (OP == 1) a[i + u * stride] = make_float4(s, s, s, s);
            if (OP == 2) a[i + u * stride] = vb[u];
            if (OP == 3)
                a[i + u * stride] = make_float4(vb[u].x + s * vc[u].x, vb[u].y + s * vc[u].y, vb[u].z + s * vc[u].z, vb[u].w + s * vc[u].w);
        }
    }
    for (; i < n; i += stride) {
        if (OP == 0) {
            const float4 v = b[i];
            keep += v.x + v.y + v.z + v.w;
        }
        if (OP == 1) a[i] = make_float4(s, s, s, s);
        if (OP == 2) a[i] = b[i];
        if (OP == 3) {
            const float4 vb = b[i], vc = c[i];
            a[i] = make_float4(vb.x + s * vc.x, vb.y + s * vc.y, vb.z + s * vc.z, vb.w + s * vc.w);
        }
    }
    if (OP == 0 && keep == 123456.789f) *sink = keep;  // keeps the loads alive; practically never true
}

}  // namespace

cudaError_t launch_hbm_stream(int op, const void* b, const void* c, void* a, long long n_vec4, float s, int block,
                              int blocks_per_sm, float* sink, cudaStream_t stream) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    const dim3 grid((unsigned)(sms * blocks_per_sm)), blk((unsigned)block);
    const float4 *pb = static_cast<const float4*>(b), *pc = static_cast<const float4*>(c);
    float4* pa = static_cast<float4*>(a);
    count_launch();
    switch (op) {
        case 0: hbm_stream_kernel<0><<<grid, blk, 0, stream>>>(pb, pc, pa, n_vec4, s, sink); break;
        case 1: hbm_stream_kernel<1><<<grid, blk, 0, stream>>>(pb, pc, pa, n_vec4, s, sink); break;
        case 2: hbm_stream_kernel<2><<<grid, blk, 0, stream>>>(pb, pc, pa, n_vec4, s, sink); break;
        default: hbm_stream_kernel<3><<<grid, blk, 0, stream>>>(pb, pc, pa, n_vec4, s, sink); break;
    }
    return cudaGetLastError();
}

}  // namespace ezb
