// x' = Q x: one f16 activation rotated into the basis the sealed weights live in, f32 out
// (the reference's rot_apply, llvq-cuda/kernels/rotate.cu:38-67 with llvq_rot.cuh:114-235).
//
// The whole vector sits in shared memory of one CTA (up to 48 K coordinates on this part; the
// reference's default 48 KB stop at 12 K): 1024 threads, and the Walsh-Hadamard stages are taken
// three at a time in registers, so a group of m = 512 coordinates needs three barriers instead
// of nine. Each radix-8 pass applies the stages len = s, 2 s, 4 s to eight coordinates s apart in
// that order, which are exactly the butterflies of the stage-by-stage transform: the f32 result is
// the same expression tree as the reference kernel's, bit for bit. The 1 / sqrt(m) scale and the
// k x k odd mix come last, one output per thread and step: out[g m + j] = sum_t Q_odd[g][t] *
// (s[t m + j] * inv), t ascending, fused multiply-adds (llvq_rot.cuh:213-235).
#pragma once
#include <cuda_fp16.h>

namespace llvq {

constexpr int kRotThreads = 1024;

template <int R>
__device__ __forceinline__ void wht_radix(float* s, int base, int stride) {
    float v[R];
#pragma unroll
    for (int j = 0; j < R; ++j) v[j] = s[base + j * stride];
#pragma unroll
    for (int len = 1; len < R; len <<= 1) {
#pragma unroll
        for (int j = 0; j < R; ++j) {
            if ((j & len) == 0) {
                const float a = v[j], b = v[j + len];
                v[j] = a + b;
                v[j + len] = a - b;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < R; ++j) s[base + j * stride] = v[j];
}

// grid = rows of the batch (one CTA rotates one activation). Dynamic shared memory: n floats of the
// vector, then k * k floats of Q_odd.
__global__ void __launch_bounds__(kRotThreads)
rot_apply_kernel(const __half* __restrict__ x, const unsigned int* __restrict__ signbits, const float* __restrict__ small,
                 float* __restrict__ out, int n, int m, int k, float inv) {
    extern __shared__ float rot_s[];
    float* s = rot_s;
    float* q = rot_s + n;
    const int tid = threadIdx.x;
    x += (size_t)blockIdx.x * n;
    out += (size_t)blockIdx.x * n;
    for (int i = tid; i < n; i += kRotThreads) {
        const float v = __half2float(x[i]);
        s[i] = ((signbits[i >> 5] >> (i & 31)) & 1u) ? -v : v;
    }
    for (int i = tid; i < k * k; i += kRotThreads) q[i] = small[i];
    __syncthreads();

    for (int stride = 1; stride < m;) {
        const int r = min(8, m / stride);  // 8, or what is left of m: 4 or 2
        const int groups = n / r;
        for (int gi = tid; gi < groups; gi += kRotThreads) {
            const int lo = gi % stride, hi = gi / stride;
            const int base = hi * stride * r + lo;
            if (r == 8) wht_radix<8>(s, base, stride);
            else if (r == 4) wht_radix<4>(s, base, stride);
            else wht_radix<2>(s, base, stride);
        }
        __syncthreads();
        stride *= r;
    }

    if (k == 1) {
        for (int i = tid; i < n; i += kRotThreads) out[i] = s[i] * inv;
        return;
    }
    for (int i = tid; i < n; i += kRotThreads) {
        const int g = i / m, j = i - g * m;
        float acc = 0.0f;
        for (int t = 0; t < k; ++t) acc = __fmaf_rn(q[g * k + t], s[t * m + j] * inv, acc);
        out[i] = acc;
    }
}

}  // namespace llvq
