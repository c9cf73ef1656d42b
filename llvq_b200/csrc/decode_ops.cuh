// The non-projection half of one batch-1 decode step of a Qwen3 block, as four small fused
// kernels (f16 tensors, f32 arithmetic). The reference leaves these steps to stock candle ops
// (llvq-llm/src/model.rs:778-834) and only *simulates* the int8 KV cache (llvq-llm/src/kvq.rs:
// 110-165); here the cache really holds u8 codes with an f16 scale and bias per group of 64
// along head_dim, written by the rope kernel and read by the attention kernel.
//
//   add_rmsnorm_kernel     x += delta (optional); y = x / rms(x) * w
//   qkv_rope_cache_kernel  per head: q/k RMSNorm over head_dim, RoPE (rotate-half) at the
//                          position read from device memory, q out; k and v quantised into the cache
//   attn_splitkv_kernel    (attn_splitkv.cuh) split-KV attention over the int8 cache, one CTA per
//   attn_combine_kernel    (KV head, slice of positions) serving all query heads of the group
//   silu_mul_kernel        y = silu(gate) * up
//
// The position is always read from device memory so that a captured CUDA graph replays unchanged.
#pragma once
#include <cuda_fp16.h>

#include "attn_splitkv.cuh"

namespace llvq {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// One CTA of 1024 threads, two f16 per thread and step (n even). x: residual stream, updated in
// place when delta != nullptr; each thread keeps its elements in registers between the two passes.
__global__ void __launch_bounds__(1024)
add_rmsnorm_kernel(__half* __restrict__ x, const __half* __restrict__ delta, const __half* __restrict__ w,
                   __half* __restrict__ y, int n, float eps) {
    llvq_dependent_enter();
    __shared__ float red[32];
    constexpr int kMaxPairs = 8;  // up to 16 384 elements
    const int pairs = n >> 1;
    float2 v[kMaxPairs];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kMaxPairs; ++k) {
        const int i = threadIdx.x + k * 1024;
        v[k] = make_float2(0.0f, 0.0f);
        if (i < pairs) {
            v[k] = __half22float2(reinterpret_cast<const __half2*>(x)[i]);
            if (delta) {
                const float2 d = __half22float2(reinterpret_cast<const __half2*>(delta)[i]);
                const __half2 sum = __floats2half2_rn(v[k].x + d.x, v[k].y + d.y);  // the stream stays f16
                reinterpret_cast<__half2*>(x)[i] = sum;
                v[k] = __half22float2(sum);
            }
            ss += v[k].x * v[k].x + v[k].y * v[k].y;
        }
    }
    ss = warp_sum_f(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int k = 0; k < 32; ++k) tot += red[k];
    const float r = rsqrtf(tot / (float)n + eps);
#pragma unroll
    for (int k = 0; k < kMaxPairs; ++k) {
        const int i = threadIdx.x + k * 1024;
        if (i < pairs) {
            const float2 wf = __half22float2(reinterpret_cast<const __half2*>(w)[i]);
            reinterpret_cast<__half2*>(y)[i] = __floats2half2_rn(v[k].x * r * wf.x, v[k].y * r * wf.y);
        }
    }
}


// Quantise the head_dim values of one head held by a warp (V values per lane, dims lane + 32 j) into
// groups of 64: group g covers j in {2g, 2g + 1}. u8 affine, scale = range / 255 through f16, bias = min
// through f16, round half away from zero (candle's round(), kvq.rs:149-152); a group whose scale rounds to
// zero stores code 0 (kvq.rs:133-160).
template <int V>
__device__ __forceinline__ void quantize_head(const float (&v)[V], unsigned char* q, __half* s, __half* b, int lane) {
#pragma unroll
    for (int g = 0; g < V / 2; ++g) {
        const float a0 = v[2 * g], a1 = v[2 * g + 1];
        const float mn = warp_min_f(fminf(a0, a1)), mx = warp_max_f(fmaxf(a0, a1));
        const __half sh = __float2half_rn((mx - mn) / 255.0f), bh = __float2half_rn(mn);
        const float sf = __half2float(sh), bf = __half2float(bh);
        const float safe = sf > 0.0f ? sf : 1.0f;
        const float c0 = sf > 0.0f ? fminf(fmaxf(roundf((a0 - bf) / safe), 0.0f), 255.0f) : 0.0f;
        const float c1 = sf > 0.0f ? fminf(fmaxf(roundf((a1 - bf) / safe), 0.0f), 255.0f) : 0.0f;
        q[lane + 64 * g] = (unsigned char)c0;
        q[lane + 32 + 64 * g] = (unsigned char)c1;
        if (lane == 0) {
            s[g] = sh;
            b[g] = bh;
        }
    }
}

// grid = n_heads + 2 n_kv CTAs of one warp. HD = head_dim (64 or 128).
template <int HD>
__global__ void qkv_rope_cache_kernel(const __half* __restrict__ qkv, const __half* __restrict__ q_norm,
                                      const __half* __restrict__ k_norm, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, const long long* __restrict__ pos_ptr,
                                      __half* __restrict__ q_out, KvCacheView kc, KvCacheView vc, int n_heads, int n_kv,
                                      float eps) {
    llvq_dependent_enter();
    constexpr int V = HD / 32;
    const int head = blockIdx.x, lane = threadIdx.x;
    const long long pos = *pos_ptr;
    const bool is_q = head < n_heads, is_k = !is_q && head < n_heads + n_kv;
    const __half* src = qkv + (size_t)head * HD;
    float v[V];
#pragma unroll
    for (int j = 0; j < V; ++j) v[j] = __half2float(src[lane + 32 * j]);
    if (is_q || is_k) {
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < V; ++j) ss += v[j] * v[j];
        const float r = rsqrtf(warp_sum_f(ss) / (float)HD + eps);
        const __half* w = is_q ? q_norm : k_norm;
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = __half2float(__float2half_rn(v[j] * r * __half2float(w[lane + 32 * j])));
        // rotate-half: dims d and d + HD/2 form a pair; lane holds both (j and j + V/2)
#pragma unroll
        for (int j = 0; j < V / 2; ++j) {
            const int d = lane + 32 * j;
            const float c = cos_t[pos * (HD / 2) + d], s = sin_t[pos * (HD / 2) + d];
            const float x1 = v[j], x2 = v[j + V / 2];
            v[j] = __half2float(__float2half_rn(x1 * c - x2 * s));
            v[j + V / 2] = __half2float(__float2half_rn(x2 * c + x1 * s));
        }
    }
    if (is_q) {
#pragma unroll
        for (int j = 0; j < V; ++j) q_out[(size_t)head * HD + lane + 32 * j] = __float2half_rn(v[j]);
        return;
    }
    const int kvh = is_k ? head - n_heads : head - n_heads - n_kv;
    KvCacheView c = is_k ? kc : vc;
    const size_t slot = (size_t)pos * n_kv + kvh;
    quantize_head<V>(v, c.q + slot * HD, c.s + slot * (HD / 64), c.b + slot * (HD / 64), lane);
}

__global__ void silu_mul_kernel(const __half* __restrict__ gu, __half* __restrict__ y, int inter) {
    llvq_dependent_enter();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const float g = __half2float(gu[i]), u = __half2float(gu[inter + i]);
    y[i] = __float2half_rn(g / (1.0f + __expf(-g)) * u);
}

}  // namespace llvq
