// Probe kernels and the class-agnostic fused GEMV built on decode_generic.
// One thread decodes one block; nothing here is tuned. These kernels define the
// semantics; the fused kernels (gemv_pipe.cuh, gemm_tab.cuh) must agree with them.
#pragma once
#include <cuda_fp16.h>

#include "decode_generic.cuh"

namespace llvq {

struct MatrixView {
    const unsigned char* codes;  // d_out * nb * 6 bytes, archive order
    const float2* cent;          // per row: the two gain centroids of the row's segment
    const float* rscale;         // per row
    const void* tail;            // d_out * tail_w, f32 or f16
    int d_out, d_in, nb, tail_w, tail_f16;
};

__global__ void decode_blocks_kernel(DevTables T, const unsigned char* __restrict__ codes, size_t n,
                                     signed char* __restrict__ points, unsigned char* __restrict__ shell,
                                     unsigned char* __restrict__ gain, unsigned long long limit) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n) return;
    const unsigned long long v = load_code48(codes, b);
    signed char* out = points + b * kDim;
    float scale;
    const int m = decode_generic(T, v >> 1, limit, [&](int pos, int val) { out[pos] = (signed char)val; }, &scale);
    shell[b] = (unsigned char)m;
    if (gain) gain[b] = (unsigned char)(v & 1ull);
}

__global__ void decode_indices_kernel(DevTables T, const unsigned long long* __restrict__ idx, size_t n,
                                      signed char* __restrict__ points, unsigned char* __restrict__ shell,
                                      unsigned long long limit) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n) return;
    signed char* out = points + b * kDim;
    float scale;
    const int m = decode_generic(T, idx[b], limit, [&](int pos, int val) { out[pos] = (signed char)val; }, &scale);
    shell[b] = (unsigned char)m;
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ void store_y(T* y, int r, float v);
template <>
__device__ __forceinline__ void store_y<float>(float* y, int r, float v) { y[r] = v; }
template <>
__device__ __forceinline__ void store_y<__half>(__half* y, int r, float v) { y[r] = __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Tail columns of row r against the staged activation: sum_t tail[r,t] * x[24 nb + t].
__device__ __forceinline__ float tail_dot(const MatrixView& mv, int r, const float* xs_tail, int lane) {
    float t = 0.0f;
    if (lane < mv.tail_w) {
        const float w = mv.tail_f16 ? __half2float(((const __half*)mv.tail)[(size_t)r * mv.tail_w + lane])
                                    : ((const float*)mv.tail)[(size_t)r * mv.tail_w + lane];
        t = w * xs_tail[lane];
    }
    return warp_sum(t);
}

constexpr int kGenRows = 8;       // rows per CTA
constexpr int kGenThreads = 256;  // one warp reduces one row

// Dynamic shared memory: 24 * nb floats of x transposed to [pos][block] (so that
// consecutive lanes, which hold consecutive blocks, read consecutive words),
// tail_w floats of x, then kGenRows * nb block partials.
template <typename XT, typename YT>
__global__ void __launch_bounds__(kGenThreads)
gemv_generic_kernel(DevTables T, MatrixView mv, const XT* __restrict__ x, YT* __restrict__ y,
                    unsigned long long limit, int* __restrict__ err_flag) {
    extern __shared__ float smem[];
    const int nb = mv.nb;
    float* xs = smem;
    float* xs_tail = xs + (size_t)kDim * nb;
    float* part = xs_tail + 32;
    for (int i = threadIdx.x; i < nb * kDim; i += kGenThreads) {
        const int b = i / kDim, pos = i - b * kDim;
        xs[pos * nb + b] = to_f32<XT>(x[i]);
    }
    if (threadIdx.x < 32) xs_tail[threadIdx.x] = threadIdx.x < mv.tail_w ? to_f32<XT>(x[nb * kDim + threadIdx.x]) : 0.0f;
    __syncthreads();

    const int row0 = blockIdx.x * kGenRows;
    const int rows = min(kGenRows, mv.d_out - row0);
    const unsigned char* codes = mv.codes + (size_t)row0 * nb * 6;
    for (int f = threadIdx.x; f < rows * nb; f += kGenThreads) {
        const int lr = f / nb, b = f - lr * nb;
        const unsigned long long v = load_code48(codes, (size_t)f);
        float acc = 0.0f, scale;
        const float* xb = xs + b;
        const int m = decode_generic(T, v >> 1, limit,
                                     [&](int pos, int val) { acc = fmaf((float)val, xb[pos * nb], acc); }, &scale);
        if (m == 255) atomicOr(err_flag, 1);
        const float2 cg = mv.cent[row0 + lr];
        part[f] = acc * (scale * ((v & 1ull) ? cg.y : cg.x));
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp < rows) {
        float s = 0.0f;
        for (int b = lane; b < nb; b += 32) s += part[warp * nb + b];
        s = warp_sum(s);
        const int r = row0 + warp;
        const float t = tail_dot(mv, r, xs_tail, lane);
        if (lane == 0) store_y<YT>(y, r, fmaf(s, mv.rscale[r], t));
    }
}

}  // namespace llvq
