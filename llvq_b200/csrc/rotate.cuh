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
#include <cstdint>
#include <cuda_fp16.h>

#include "portable.h"

namespace llvq {

constexpr int kRotThreads = 1024;

// Coordinate i of the vector lives at word i + i / 8 of shared memory: the radix-8 passes touch eight
// coordinates 1, 8, 64... apart per thread, and the skew keeps the 32 lanes of a warp on 32 different banks
// in the first two passes (without it they are 8-way and 4-way conflicts).
__host__ __device__ inline int rot_at(int i) { return i + (i >> 3); }

template <int R>
__device__ __forceinline__ void wht_radix(float* s, int base, int stride) {
    float v[R];
#pragma unroll
    for (int j = 0; j < R; ++j) v[j] = s[rot_at(base + j * stride)];
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
    for (int j = 0; j < R; ++j) s[rot_at(base + j * stride)] = v[j];
}

// Row stride of Q_odd in shared memory: k rounded up to the compile-time bound of rot_mix (zero padded).
__host__ __device__ inline int rot_qstride(int k) { return k <= 1 ? 1 : k <= 4 ? 4 : k <= 8 ? 8 : k <= 16 ? 16 : k <= 24 ? 24 : 32; }

// Odd mix: thread j owns column j of the k x m matrix held in s: its k values go to registers once, every
// output row is one ascending chain of fused multiply-adds over them (the zero padding adds nothing), and the
// rows of Q_odd come from shared memory four at a time (all threads read the same address: a broadcast).
template <int KB>
__device__ __forceinline__ void rot_mix(const float* s, const float* q, float* __restrict__ out, int m, int k, float inv,
                                        int tid) {
    for (int j = tid; j < m; j += kRotThreads) {
        float col[KB];
#pragma unroll
        for (int t = 0; t < KB; ++t) col[t] = t < k ? s[rot_at(t * m + j)] * inv : 0.0f;
        for (int g = 0; g < k; ++g) {
            float acc = 0.0f;
#pragma unroll
            for (int t = 0; t < KB; t += 4) {
                const float4 qq = *reinterpret_cast<const float4*>(q + g * KB + t);
                acc = __fmaf_rn(qq.x, col[t], acc);
                acc = __fmaf_rn(qq.y, col[t + 1], acc);
                acc = __fmaf_rn(qq.z, col[t + 2], acc);
                acc = __fmaf_rn(qq.w, col[t + 3], acc);
            }
            out[g * m + j] = acc;
        }
    }
}

// The transform proper, for a CTA of kRotThreads threads whose signed vector already sits in s[0, n)
// and whose Q_odd sits in q, k rows of rot_qstride(k) floats, zero padded and 16-byte aligned (a barrier
// after both were written is the caller's): Hadamard
// passes, then scale and odd mix into out.
__device__ __forceinline__ void rot_transform(float* s, const float* q, float* __restrict__ out, int n, int m, int k,
                                              float inv, int tid, int first_stride = 1) {
    for (int stride = first_stride; stride < m;) {
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
        for (int i = tid; i < n; i += kRotThreads) out[i] = s[rot_at(i)] * inv;
        return;
    }
    if (k <= 4) rot_mix<4>(s, q, out, m, k, inv, tid);
    else if (k <= 8) rot_mix<8>(s, q, out, m, k, inv, tid);
    else if (k <= 16) rot_mix<16>(s, q, out, m, k, inv, tid);
    else if (k <= 24) rot_mix<24>(s, q, out, m, k, inv, tid);
    else rot_mix<32>(s, q, out, m, k, inv, tid);
}

__device__ __forceinline__ void rot_stage_q(float* q, const float* __restrict__ small, int k, int tid) {
    const int stride = rot_qstride(k);
    for (int i = tid; i < k * stride; i += kRotThreads) {
        const int g = i / stride, t = i - g * stride;
        q[i] = t < k ? small[g * k + t] : 0.0f;
    }
}

// Floats of dynamic shared memory a rotation of width n needs: the vector (rounded up to a multiple of 4 so
// that Q_odd starts 16-byte aligned) and the padded Q_odd.
__host__ __device__ inline int rot_vec_words(int n) { return (rot_at(n) + 4) & ~3; }
__host__ __device__ inline size_t rot_smem_floats(int n, int k) { return (size_t)rot_vec_words(n) + (size_t)k * rot_qstride(k); }

__device__ __forceinline__ float rot_signed(const unsigned int* __restrict__ signbits, int i, float v) {
    return ((signbits[i >> 5] >> (i & 31)) & 1u) ? -v : v;
}

// Eight consecutive coordinates in registers: signs from one byte of the bitmap, then the first three butterfly
// stages (len 1, 2, 4: the stride-1 radix-8 pass) before the values ever reach shared memory. i % 8 == 0.
__device__ __forceinline__ void rot_first_pass_store(float* s, const unsigned int* __restrict__ signbits, int i, float (&v)[8]) {
    const unsigned int bits = (signbits[i >> 5] >> (i & 31)) & 0xffu;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = ((bits >> j) & 1u) ? -v[j] : v[j];
#pragma unroll
    for (int len = 1; len < 8; len <<= 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if ((j & len) == 0) {
                const float a = v[j], b = v[j + len];
                v[j] = a + b;
                v[j + len] = a - b;
            }
        }
    }
    const int w = rot_at(i);  // i + j stays inside one skew step: eight consecutive words
#pragma unroll
    for (int j = 0; j < 8; ++j) s[w + j] = v[j];
}

// grid = rows of the batch (one CTA rotates one activation). Dynamic shared memory: n floats of the
// vector, then k * k floats of Q_odd.
__global__ void __launch_bounds__(kRotThreads)
rot_apply_kernel(const __half* __restrict__ x, const unsigned int* __restrict__ signbits, const float* __restrict__ small,
                 float* __restrict__ out, int n, int m, int k, float inv) {
    llvq_dependent_enter();
    extern __shared__ float rot_s[];
    float* s = rot_s;
    float* q = rot_s + rot_vec_words(n);
    const int tid = threadIdx.x;
    x += (size_t)blockIdx.x * n;
    out += (size_t)blockIdx.x * n;
    // 16-byte loads and the first pass in registers when the group width allows (every model width does)
    const bool fast = m >= 8 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    if (fast) {
        for (int i = tid * 8; i < n; i += kRotThreads * 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + i);
            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
            float v[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h2[j]);
                v[2 * j] = f.x;
                v[2 * j + 1] = f.y;
            }
            rot_first_pass_store(s, signbits, i, v);
        }
    } else {
        for (int i = tid; i < n; i += kRotThreads) s[rot_at(i)] = rot_signed(signbits, i, __half2float(x[i]));
    }
    rot_stage_q(q, small, k, tid);
    __syncthreads();
    rot_transform(s, q, out, n, m, k, inv, tid, fast ? 8 : 1);
}

// add + RMSNorm of the residual stream (as add_rmsnorm_kernel: x += delta in f16, y = f16(x / rms * w)) with
// the rotation of y folded in: the normalised activation never goes to memory, its rotated f32 form does.
// One CTA of 1024 threads; the f16 rounding of y is kept, so the result equals the two-kernel sequence bit for bit.
__global__ void __launch_bounds__(kRotThreads)
add_rmsnorm_rotate_kernel(__half* __restrict__ x, const __half* __restrict__ delta, const __half* __restrict__ w,
                          const unsigned int* __restrict__ signbits, const float* __restrict__ small,
                          float* __restrict__ out, int n, int m, int k, float inv, float eps) {
    llvq_dependent_enter();
    extern __shared__ float rot_s[];
    __shared__ float red[32];
    float* s = rot_s;
    float* q = rot_s + rot_vec_words(n);
    const int tid = threadIdx.x;
    constexpr int kMaxPairs = 8;  // up to 16 384 elements
    const int pairs = n >> 1;
    float2 v[kMaxPairs];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPairs; ++j) {
        const int i = tid + j * kRotThreads;
        v[j] = make_float2(0.0f, 0.0f);
        if (i < pairs) {
            v[j] = __half22float2(reinterpret_cast<const __half2*>(x)[i]);
            if (delta) {
                const float2 d = __half22float2(reinterpret_cast<const __half2*>(delta)[i]);
                const __half2 sum = __floats2half2_rn(v[j].x + d.x, v[j].y + d.y);  // the stream stays f16
                reinterpret_cast<__half2*>(x)[i] = sum;
                v[j] = __half22float2(sum);
            }
            ss += v[j].x * v[j].x + v[j].y * v[j].y;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    rot_stage_q(q, small, k, tid);
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) tot += red[j];
    const float r = rsqrtf(tot / (float)n + eps);
#pragma unroll
    for (int j = 0; j < kMaxPairs; ++j) {
        const int i = tid + j * kRotThreads;
        if (i < pairs) {
            const float2 wf = __half22float2(reinterpret_cast<const __half2*>(w)[i]);
            const float2 y = __half22float2(__floats2half2_rn(v[j].x * r * wf.x, v[j].y * r * wf.y));
            s[rot_at(2 * i)] = rot_signed(signbits, 2 * i, y.x);
            s[rot_at(2 * i + 1)] = rot_signed(signbits, 2 * i + 1, y.y);
        }
    }
    __syncthreads();
    rot_transform(s, q, out, n, m, k, inv, tid);
}

// y = silu(gate) * up rounded to f16 (as silu_mul_kernel), rotated: the input of the down projection.
__global__ void __launch_bounds__(kRotThreads)
silu_mul_rotate_kernel(const __half* __restrict__ gu, const unsigned int* __restrict__ signbits,
                       const float* __restrict__ small, float* __restrict__ out, int n, int m, int k, float inv) {
    llvq_dependent_enter();
    extern __shared__ float rot_s[];
    float* s = rot_s;
    float* q = rot_s + rot_vec_words(n);
    const int tid = threadIdx.x;
    const bool fast = m >= 8 && (reinterpret_cast<uintptr_t>(gu) & 15u) == 0;  // then n % 8 == 0 and gu + n is aligned too
    if (fast) {
        for (int i = tid * 8; i < n; i += kRotThreads * 8) {
            const uint4 gr = *reinterpret_cast<const uint4*>(gu + i), ur = *reinterpret_cast<const uint4*>(gu + n + i);
            const __half2* g2 = reinterpret_cast<const __half2*>(&gr);
            const __half2* u2 = reinterpret_cast<const __half2*>(&ur);
            float v[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 g = __half22float2(g2[j]), u = __half22float2(u2[j]);
                v[2 * j] = __half2float(__float2half_rn(g.x / (1.0f + __expf(-g.x)) * u.x));
                v[2 * j + 1] = __half2float(__float2half_rn(g.y / (1.0f + __expf(-g.y)) * u.y));
            }
            rot_first_pass_store(s, signbits, i, v);
        }
    } else {
        for (int i = tid; i < n; i += kRotThreads) {
            const float g = __half2float(gu[i]), u = __half2float(gu[n + i]);
            s[rot_at(i)] = rot_signed(signbits, i, __half2float(__float2half_rn(g / (1.0f + __expf(-g)) * u)));
        }
    }
    rot_stage_q(q, small, k, tid);
    __syncthreads();
    rot_transform(s, q, out, n, m, k, inv, tid, fast ? 8 : 1);
}

}  // namespace llvq
