// Split-KV attention of one decoded token over the int8 KV cache (u8 codes, f16 scale and bias per
// group of 64 along head_dim; the scheme of llvq-llm/src/kvq.rs:110-165, which the reference only
// simulates). The work is one pass over the cached bytes, so the kernel is laid out for HBM:
//
//   grid = (n_kv, splits), 256 threads. A CTA owns one KV head and one slice of the positions and
//   serves all G = n_heads / n_kv query heads of that KV head from a single read of the slice
//   (grouped-query attention: the cache bytes cross the memory system once, not G times).
//   Each warp walks tiles of 32 positions:
//     scores   lane = position: the lane reads its key row (head_dim bytes, 16-byte loads),
//              dequantises pairs with half2 arithmetic (exact u8 -> f16, then one f16 fma: the
//              f16-rounded value the cache stands for) and accumulates G dot products in f32
//              against the query held in shared memory (broadcast reads);
//     softmax  online, base 2 (log2 e folded into the query scale), per warp and query head;
//     values   the tile's value rows are fetched with cp.async into the warp's shared-memory
//              stripe before the scores are computed, so both streams are in flight together;
//              then lane = head_dim / 32 dims: one row per step, dequantised and added as
//              p[g] * v to G accumulators; p and the value scales go through the same stripe.
//   The 8 warps merge through shared memory, the CTA writes (max, sum, accumulator) per query head,
//   and attn_combine_kernel merges the slices. With one slice the CTA writes the result itself.
//
// The position is read from device memory, so a captured graph replays unchanged; slices beyond the
// write head store an empty partial (max = -inf).
#pragma once
#include <cuda_fp16.h>

#include "portable.h"

namespace llvq {

struct KvCacheView {
    unsigned char* q;  // [capacity, n_kv, head_dim]
    __half* s;         // [capacity, n_kv, head_dim / 64]
    __half* b;
};

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnTile = 32;   // positions per warp step
constexpr int kAttnMaxG = 8;    // query heads per KV head

__device__ __forceinline__ float attn_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float attn_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Two cache bytes -> two dequantised values, f16(code * s + b), widened to f32. `sel` picks the bytes:
// 0x4140 for bytes 0,1 and 0x4342 for bytes 2,3 (0x64 in the high byte of each half makes 1024 + code).
__device__ __forceinline__ float2 kv_dequant2(unsigned int word, unsigned int sel, __half2 s2, __half2 b2) {
    const unsigned int packed = __byte_perm(word, 0x64646464u, sel);
    const __half2 code = __hsub2(*reinterpret_cast<const __half2*>(&packed), __half2half2(__ushort_as_half(0x6400)));
    return __half22float2(__hfma2(code, s2, b2));
}

template <int HD, int G>
struct AttnSmem {
    static constexpr int NG = HD / 64;
    float qs[HD][kAttnMaxG];                      // query * scale * log2(e), [dim][query head]
    union {
        struct {
            float p[kAttnWarps][kAttnTile][kAttnMaxG];   // softmax weights of the warp's tile
            __half2 vsb[kAttnWarps][kAttnTile][NG][2];   // (s, s) and (b, b) of each value group
            unsigned char v[kAttnWarps][kAttnTile][HD];  // value codes of the warp's tile (cp.async)
        } tile;
        struct {
            float m[kAttnWarps][G], l[kAttnWarps][G];
            float acc[kAttnWarps][G][HD];
        } merge;
    } u;
};

template <int HD, int G>
__global__ void __launch_bounds__(kAttnThreads)
attn_splitkv_kernel(const __half* __restrict__ q, KvCacheView kc, KvCacheView vc, const long long* __restrict__ pos_ptr,
                    __half* __restrict__ out, float* __restrict__ partial, int n_kv) {
    llvq_dependent_enter();
    constexpr int NG = HD / 64;
    constexpr int VB = HD / 32;       // value bytes (dims) per lane
    constexpr int KW = HD / 4;        // 32-bit words of a key row
    extern __shared__ __align__(16) unsigned char attn_raw[];
    AttnSmem<HD, G>& S = *reinterpret_cast<AttnSmem<HD, G>*>(attn_raw);
    const int kvh = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_pos = (int)(*pos_ptr) + 1;
    int slice = (n_pos + splits - 1) / splits;
    slice = (slice + kAttnTile - 1) / kAttnTile * kAttnTile;
    const int t0 = split * slice, t1 = min(n_pos, t0 + slice);

    // softmax(q k / sqrt(d)) in base 2: fold the scale and log2(e) into the query once
    const float qscale = rsqrtf((float)HD) * 1.4426950408889634f;
    for (int i = tid; i < HD * kAttnMaxG; i += kAttnThreads) {
        const int d = i / kAttnMaxG, g = i % kAttnMaxG;
        S.qs[d][g] = g < G ? __half2float(q[((size_t)kvh * G + g) * HD + d]) * qscale : 0.0f;
    }
    __syncthreads();

    float m[G], l[G], acc[G][VB];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int c = 0; c < VB; ++c) acc[g][c] = 0.0f;
    }

    for (int base = t0 + warp * kAttnTile; base < t1; base += kAttnWarps * kAttnTile) {
        const int t = base + lane;
        const bool valid = t < t1;
        const size_t slot = (size_t)(valid ? t : t1 - 1) * n_kv + kvh;
        const int n_here = min(kAttnTile, t1 - base);
        // ---- start the value rows of the tile on their way into the stripe ----
        {
            constexpr int CPR = HD / 16;  // 16-byte chunks per row
#pragma unroll
            for (int i = 0; i < CPR; ++i) {
                const int c = lane + 32 * i, r = c / CPR, k = c % CPR;
                if (r < n_here) {
                    const unsigned char* src = vc.q + ((size_t)(base + r) * n_kv + kvh) * HD + 16 * k;
                    const unsigned int dst = (unsigned int)__cvta_generic_to_shared(&S.u.tile.v[warp][r][16 * k]);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        // ---- scores: this lane's key row against the G queries ----
        float sc[G];
#pragma unroll
        for (int g = 0; g < G; ++g) sc[g] = 0.0f;
        {
            const uint4* row = reinterpret_cast<const uint4*>(kc.q + slot * HD);
            uint4 kw[KW / 4];
#pragma unroll
            for (int i = 0; i < KW / 4; ++i) kw[i] = __ldg(row + i);
            __half2 s2[NG], b2[NG];
#pragma unroll
            for (int gi = 0; gi < NG; ++gi) {
                s2[gi] = __half2half2(kc.s[slot * NG + gi]);
                b2[gi] = __half2half2(kc.b[slot * NG + gi]);
            }
#pragma unroll
            for (int i = 0; i < KW / 4; ++i) {
                const unsigned int w4[4] = {kw[i].x, kw[i].y, kw[i].z, kw[i].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int d = 16 * i + 4 * j;
                    const float2 k01 = kv_dequant2(w4[j], 0x4140u, s2[d / 64], b2[d / 64]);
                    const float2 k23 = kv_dequant2(w4[j], 0x4342u, s2[d / 64], b2[d / 64]);
                    const float kv4[4] = {k01.x, k01.y, k23.x, k23.y};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float4 qa = *reinterpret_cast<const float4*>(&S.qs[d + c][0]);
                        const float qv[4] = {qa.x, qa.y, qa.z, qa.w};
#pragma unroll
                        for (int g = 0; g < (G < 4 ? G : 4); ++g) sc[g] = fmaf(kv4[c], qv[g], sc[g]);
                        if (G > 4) {
                            const float4 qb = *reinterpret_cast<const float4*>(&S.qs[d + c][4]);
                            const float qw[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                            for (int g = 4; g < G; ++g) sc[g] = fmaf(kv4[c], qw[g - 4], sc[g]);
                        }
                    }
                }
            }
        }
        // ---- online softmax of the tile, per query head ----
        float corr[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float s = valid ? sc[g] : -INFINITY;
            const float m_new = fmaxf(m[g], attn_warp_max(s));  // finite: the tile holds a valid position
            corr[g] = exp2f(m[g] - m_new);
            const float p = exp2f(s - m_new);
            l[g] = l[g] * corr[g] + attn_warp_sum(p);
            m[g] = m_new;
            S.u.tile.p[warp][lane][g] = p;
        }
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
            S.u.tile.vsb[warp][lane][gi][0] = __half2half2(vc.s[slot * NG + gi]);
            S.u.tile.vsb[warp][lane][gi][1] = __half2half2(vc.b[slot * NG + gi]);
        }
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int c = 0; c < VB; ++c) acc[g][c] *= corr[g];
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        // ---- values: one row per step, lane = VB consecutive dims ----
        const int vgroup = (lane * VB) / 64;
#pragma unroll 4
        for (int j = 0; j < n_here; ++j) {
            const unsigned char* vrow = &S.u.tile.v[warp][j][lane * VB];
            float v[VB];
            const __half2 s2 = S.u.tile.vsb[warp][j][vgroup][0], b2 = S.u.tile.vsb[warp][j][vgroup][1];
            if constexpr (VB == 4) {
                const unsigned int w = *reinterpret_cast<const unsigned int*>(vrow);
                const float2 a = kv_dequant2(w, 0x4140u, s2, b2), b = kv_dequant2(w, 0x4342u, s2, b2);
                v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
            } else {
                const unsigned int w = *reinterpret_cast<const unsigned short*>(vrow);
                const float2 a = kv_dequant2(w, 0x4140u, s2, b2);
                v[0] = a.x, v[1] = a.y;
            }
            const float4 pa = *reinterpret_cast<const float4*>(&S.u.tile.p[warp][j][0]);
            const float pv[4] = {pa.x, pa.y, pa.z, pa.w};
#pragma unroll
            for (int g = 0; g < (G < 4 ? G : 4); ++g)
#pragma unroll
                for (int c = 0; c < VB; ++c) acc[g][c] = fmaf(pv[g], v[c], acc[g][c]);
            if (G > 4) {
                const float4 pb = *reinterpret_cast<const float4*>(&S.u.tile.p[warp][j][4]);
                const float pw[4] = {pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                for (int g = 4; g < G; ++g)
#pragma unroll
                    for (int c = 0; c < VB; ++c) acc[g][c] = fmaf(pw[g - 4], v[c], acc[g][c]);
            }
        }
        __syncwarp();  // the stripe is rewritten by the next tile
    }

    // ---- merge the warps (the tile stripes are dead from here on) ----
    __syncthreads();
#pragma unroll
    for (int g = 0; g < G; ++g) {
        if (lane == 0) {
            S.u.merge.m[warp][g] = m[g];
            S.u.merge.l[warp][g] = l[g];
        }
#pragma unroll
        for (int c = 0; c < VB; ++c) S.u.merge.acc[warp][g][lane * VB + c] = acc[g][c];
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += kAttnThreads) {
        const int g = i / HD, d = i % HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, S.u.merge.m[w][g]);
        float ll = 0.0f, o = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float mw = S.u.merge.m[w][g];
            const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mm);
            ll = fmaf(S.u.merge.l[w][g], f, ll);
            o = fmaf(S.u.merge.acc[w][g][d], f, o);
        }
        const int head = kvh * G + g;
        if (splits == 1) {
            out[(size_t)head * HD + d] = __float2half_rn(o / ll);
        } else {
            float* dst = partial + ((size_t)head * splits + split) * (HD + 2);
            if (d == 0) {
                dst[0] = mm;  // -inf for a slice beyond the write head
                dst[1] = ll;
            }
            dst[2 + d] = o;
        }
    }
}

// grid = n_heads, HD threads: merge the slices (base-2 maxima) in slice order.
template <int HD>
__global__ void __launch_bounds__(HD)
attn_combine_kernel(const float* __restrict__ partial, __half* __restrict__ out, int splits) {
    llvq_dependent_enter();
    extern __shared__ float f_s[];  // splits weights
    __shared__ float red[HD / 32];
    __shared__ float bcast[2];
    const int head = blockIdx.x, d = threadIdx.x, lane = d & 31, warp = d >> 5;
    const float* src = partial + (size_t)head * splits * (HD + 2);
    float mm = -INFINITY;
    for (int s = d; s < splits; s += HD) mm = fmaxf(mm, src[(size_t)s * (HD + 2)]);
    mm = attn_warp_max(mm);
    if (lane == 0) red[warp] = mm;
    __syncthreads();
    if (d == 0) {
        float v = red[0];
        for (int w = 1; w < HD / 32; ++w) v = fmaxf(v, red[w]);
        bcast[0] = v;
    }
    __syncthreads();
    mm = bcast[0];
    float ll = 0.0f;
    for (int s = d; s < splits; s += HD) {
        const float ms = src[(size_t)s * (HD + 2)];
        const float f = ms == -INFINITY ? 0.0f : exp2f(ms - mm);
        f_s[s] = f;
        ll = fmaf(src[(size_t)s * (HD + 2) + 1], f, ll);
    }
    ll = attn_warp_sum(ll);
    __syncthreads();  // red[] is read above; f_s complete below
    if (lane == 0) red[warp] = ll;
    __syncthreads();
    if (d == 0) {
        float v = 0.0f;
        for (int w = 0; w < HD / 32; ++w) v += red[w];
        bcast[1] = v;
    }
    __syncthreads();
    float o = 0.0f;
#pragma unroll 8
    for (int s = 0; s < splits; ++s) o = fmaf(src[(size_t)s * (HD + 2) + 2 + d], f_s[s], o);
    out[(size_t)head * HD + d] = __float2half_rn(o / bcast[1]);
}

}  // namespace llvq
