// The non-projection half of one batch-1 decode step of a Qwen3 block, as four small fused
// kernels (f16 tensors, f32 arithmetic). The reference leaves these steps to stock candle ops
// (llvq-llm/src/model.rs:778-834) and only *simulates* the int8 KV cache (llvq-llm/src/kvq.rs:
// 110-165); here the cache really holds u8 codes with an f16 scale and bias per group of 64
// along head_dim, written by the rope kernel and read by the attention kernel.
//
//   add_rmsnorm_kernel     x += delta (optional); y = x / rms(x) * w
//   qkv_rope_cache_kernel  per head: q/k RMSNorm over head_dim, RoPE (rotate-half) at the
//                          position read from device memory, q out; k and v quantised into the cache
//   attn_decode_kernel     split-KV attention: CTA (head, slice) runs an online softmax over its slice of
//   attn_combine_kernel    positions 0..pos with keys/values dequantised on the fly; slices merged after
//   silu_mul_kernel        y = silu(gate) * up
//
// The position is always read from device memory so that a captured CUDA graph replays unchanged.
#pragma once
#include <cuda_fp16.h>

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

struct KvCacheView {
    unsigned char* q;  // [capacity, n_kv, head_dim]
    __half* s;         // [capacity, n_kv, head_dim / 64]
    __half* b;
};

// Quantise the head_dim values of one head held by a warp (V values per lane, dims lane + 32 j) into
// groups of 64: group g covers j in {2g, 2g + 1}. u8 affine, scale = range / 255 through f16, bias = min
// through f16, round to nearest; a group whose scale rounds to zero stores code 0 (kvq.rs:133-160).
template <int V>
__device__ __forceinline__ void quantize_head(const float (&v)[V], unsigned char* q, __half* s, __half* b, int lane) {
#pragma unroll
    for (int g = 0; g < V / 2; ++g) {
        const float a0 = v[2 * g], a1 = v[2 * g + 1];
        const float mn = warp_min_f(fminf(a0, a1)), mx = warp_max_f(fmaxf(a0, a1));
        const __half sh = __float2half_rn((mx - mn) / 255.0f), bh = __float2half_rn(mn);
        const float sf = __half2float(sh), bf = __half2float(bh);
        const float safe = sf > 0.0f ? sf : 1.0f;
        const float c0 = sf > 0.0f ? fminf(fmaxf(rintf((a0 - bf) / safe), 0.0f), 255.0f) : 0.0f;
        const float c1 = sf > 0.0f ? fminf(fmaxf(rintf((a1 - bf) / safe), 0.0f), 255.0f) : 0.0f;
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

// Split-KV attention for one decoded token. grid = (n_heads, splits): CTA (h, s) covers the s-th
// equal slice of positions 0..pos with 4 warps (warp w takes every 4th position of the slice), an online
// softmax per warp merged through shared memory. With one split the result goes straight to `out`;
// otherwise the CTA stores its (max, sum, unnormalised accumulator) into `partial` and
// attn_combine_kernel merges the slices. Keys and values are dequantised on the fly.
template <int HD>
__global__ void attn_decode_kernel(const __half* __restrict__ q, KvCacheView kc, KvCacheView vc,
                                   const long long* __restrict__ pos_ptr, __half* __restrict__ out,
                                   float* __restrict__ partial, int n_heads, int n_kv) {
    constexpr int V = HD / 32;
    constexpr int kW = 4;
    __shared__ float sm_m[kW], sm_l[kW], sm_acc[kW][HD];
    const int head = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int splits = gridDim.y, split = blockIdx.y;
    const int kvh = head / (n_heads / n_kv);
    const int n_pos = (int)(*pos_ptr) + 1;
    const int slice = (n_pos + splits - 1) / splits;
    const int t0 = split * slice, t1 = min(n_pos, t0 + slice);
    const float scale = rsqrtf((float)HD);
    float qv[V], acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        qv[j] = __half2float(q[(size_t)head * HD + lane + 32 * j]) * scale;
        acc[j] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    for (int t = t0 + warp; t < t1; t += kW) {
        const size_t slot = (size_t)t * n_kv + kvh;
        const unsigned char* kq = kc.q + slot * HD;
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int g = j / 2;  // dims lane + 32 j: group of 64
            const float kval = __half2float(__float2half_rn(
                (float)kq[lane + 32 * j] * __half2float(kc.s[slot * (HD / 64) + g]) + __half2float(kc.b[slot * (HD / 64) + g])));
            dot += qv[j] * kval;
        }
        dot = warp_sum_f(dot);
        const float m_new = fmaxf(m, dot);
        const float corr = __expf(m - m_new), p = __expf(dot - m_new);
        l = l * corr + p;
        const unsigned char* vq = vc.q + slot * HD;
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int g = j / 2;
            const float vval = __half2float(__float2half_rn(
                (float)vq[lane + 32 * j] * __half2float(vc.s[slot * (HD / 64) + g]) + __half2float(vc.b[slot * (HD / 64) + g])));
            acc[j] = acc[j] * corr + p * vval;
        }
        m = m_new;
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int j = 0; j < V; ++j) sm_acc[warp][lane + 32 * j] = acc[j];
    __syncthreads();
    if (warp == 0) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kW; ++w) mm = fmaxf(mm, sm_m[w]);
        float ll = 0.0f, o[V];
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = 0.0f;
#pragma unroll
        for (int w = 0; w < kW; ++w) {
            const float f = sm_m[w] == -INFINITY ? 0.0f : __expf(sm_m[w] - mm);
            ll += sm_l[w] * f;
#pragma unroll
            for (int j = 0; j < V; ++j) o[j] += sm_acc[w][lane + 32 * j] * f;
        }
        if (splits == 1) {
#pragma unroll
            for (int j = 0; j < V; ++j) out[(size_t)head * HD + lane + 32 * j] = __float2half_rn(o[j] / ll);
        } else {
            float* dst = partial + ((size_t)head * splits + split) * (HD + 2);
            if (lane == 0) {
                dst[0] = mm;  // -inf for an empty slice
                dst[1] = ll;
            }
#pragma unroll
            for (int j = 0; j < V; ++j) dst[2 + lane + 32 * j] = o[j];
        }
    }
}

// grid = n_heads, HD threads: merge the slices of attn_decode_kernel in slice order.
template <int HD>
__global__ void attn_combine_kernel(const float* __restrict__ partial, __half* __restrict__ out, int splits) {
    const int head = blockIdx.x, d = threadIdx.x;
    const float* src = partial + (size_t)head * splits * (HD + 2);
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, src[(size_t)s * (HD + 2)]);
    float ll = 0.0f, o = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = src[(size_t)s * (HD + 2)];
        const float f = ms == -INFINITY ? 0.0f : __expf(ms - mm);
        ll += src[(size_t)s * (HD + 2) + 1] * f;
        o += src[(size_t)s * (HD + 2) + 2 + d] * f;
    }
    out[(size_t)head * HD + d] = __float2half_rn(o / ll);
}

__global__ void silu_mul_kernel(const __half* __restrict__ gu, __half* __restrict__ y, int inter) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const float g = __half2float(gu[i]), u = __half2float(gu[inter + i]);
    y[i] = __float2half_rn(g / (1.0f + __expf(-g)) * u);
}

}  // namespace llvq
