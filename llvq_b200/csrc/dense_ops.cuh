// Two helpers around the fused projections that are not on the batch-1 hot path:
//
//   dequant_dense_kernel   writes a matrix as dense f16 [d_out, d_in] (codes decoded once, gain, row
//                          scale and shell norm applied, tail columns copied). It feeds a transient
//                          cuBLAS GEMM for long prompts, where the contraction is compute-bound and a
//                          dense tile is the right operand; the reference's dense-decoded run
//                          (llvq-llm/src/bin/fusedrun.rs:263-278) is the same weights kept resident.
//   lm_head_argmax_kernel  greedy head over a tied f16 embedding: logits = E h in f32 with a fixed
//   lm_head_pick_kernel    summation order per row, argmax with the lowest index on ties. A row's logit
//                          does not depend on how the vocabulary is split over CTAs or GPUs, so a
//                          sharded head picks the same token as a whole one (the reference reads the
//                          logits back and takes the argmax on the host, llvq-llm/src/model.rs:1041-1073).
#pragma once
#include <cuda_fp16.h>

#include "decode_tab.cuh"
#include "kernels_generic.cuh"

namespace llvq {

// Persistent CTAs of 512 threads with the decoder tables in shared memory; a thread takes one block at a time
// (class search, then its family's decoder: the lanes of a warp may run different families one after the other,
// which this transient path accepts) and writes its 24 weights with three 16-byte stores when the row allows.
constexpr int kDenseThreads = 512;
__global__ void __launch_bounds__(kDenseThreads)
dequant_dense_kernel(const unsigned char* __restrict__ blob_g, const OffEntry* __restrict__ lut_off,
                     const unsigned long long* __restrict__ lut_on3, TabLayout L, MatrixView mv, __half* __restrict__ out,
                     int* __restrict__ err_flag) {
    extern __shared__ __align__(128) unsigned char dense_smem[];
    for (unsigned int o = threadIdx.x * 16u; o < L.total_bytes; o += kDenseThreads * 16u)
        *reinterpret_cast<uint4*>(dense_smem + o) = __ldg(reinterpret_cast<const uint4*>(blob_g + o));
    __syncthreads();
    TabView T;
    T.base = (unsigned int)__cvta_generic_to_shared(dense_smem);
    T.lut_off = lut_off;
    T.lut_on3 = lut_on3;
    T.L = L;
    const int per_row = mv.nb + (mv.tail_w ? 1 : 0);
    const size_t n_items = (size_t)mv.d_out * per_row;
    const bool vec_ok = (mv.d_in & 7) == 0 && ((uintptr_t)out & 15u) == 0;  // 48-byte blocks on 16-byte boundaries
    for (size_t item = (size_t)blockIdx.x * kDenseThreads + threadIdx.x; item < n_items; item += (size_t)gridDim.x * kDenseThreads) {
        const int r = (int)(item / per_row), b = (int)(item % per_row);
        __half* dst = out + (size_t)r * mv.d_in + (size_t)b * kDim;
        if (b == mv.nb) {  // the tail columns of this row, already in weight units
            for (int t = 0; t < mv.tail_w; ++t) {
                const float w = mv.tail_f16 ? __half2float(((const __half*)mv.tail)[(size_t)r * mv.tail_w + t])
                                            : ((const float*)mv.tail)[(size_t)r * mv.tail_w + t];
                dst[t] = __float2half_rn(w);
            }
            continue;
        }
        const unsigned long long v = load_code48(mv.codes, (size_t)r * mv.nb + b);
        const float2 cent = mv.cent[r];
        unsigned int V[6];
        float scale = 0.0f;
        const int fam = tab_decode_any(T, v >> 1, V, &scale);
        if (fam == -2 && err_flag) atomicExch(err_flag, 1);  // an index outside the ball decodes to zeros
        const float f = ((v & 1ull) ? cent.y : cent.x) * scale * mv.rscale[r];
        unsigned int h[12];
#pragma unroll
        for (int k = 0; k < 6; ++k) {
            const int w = (int)V[k];
            const __half2 lo = __floats2half2_rn((float)(signed char)(w & 0xff) * f, (float)(signed char)((w >> 8) & 0xff) * f);
            const __half2 hi = __floats2half2_rn((float)(signed char)((w >> 16) & 0xff) * f, (float)(w >> 24) * f);
            h[2 * k] = *reinterpret_cast<const unsigned int*>(&lo);
            h[2 * k + 1] = *reinterpret_cast<const unsigned int*>(&hi);
        }
        if (vec_ok) {
#pragma unroll
            for (int j = 0; j < 3; ++j) reinterpret_cast<uint4*>(dst)[j] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 12; ++j) {
                reinterpret_cast<unsigned short*>(dst)[2 * j] = (unsigned short)(h[j] & 0xffffu);
                reinterpret_cast<unsigned short*>(dst)[2 * j + 1] = (unsigned short)(h[j] >> 16);
            }
        }
    }
}

constexpr int kHeadThreads = 256;   // 8 warps, one embedding row per warp and step
constexpr int kHeadMaxGrid = 1024;  // partial (value, row) pairs the pick kernel merges
constexpr int kHeadMaxHidden = 8192;

struct HeadBest {
    float val;
    int row;
};

__device__ __forceinline__ bool head_better(float v, int r, float bv, int br) { return v > bv || (v == bv && r < br); }

// embed: [rows, hidden] f16 (16-byte aligned rows: hidden % 8 == 0); h: [hidden] f16.
__global__ void __launch_bounds__(kHeadThreads)
lm_head_argmax_kernel(const __half* __restrict__ embed, const __half* __restrict__ h, int rows, int hidden,
                      HeadBest* __restrict__ partial) {
    llvq_dependent_enter();
    __shared__ __align__(16) __half hs[kHeadMaxHidden];
    __shared__ HeadBest red[kHeadThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < hidden / 8; i += kHeadThreads)
        reinterpret_cast<uint4*>(hs)[i] = reinterpret_cast<const uint4*>(h)[i];
    __syncthreads();
    const int vec = hidden / 8;
    float best = -INFINITY;
    int best_row = 0x7fffffff;
    for (int r = blockIdx.x * (kHeadThreads / 32) + warp; r < rows; r += gridDim.x * (kHeadThreads / 32)) {
        const uint4* src = reinterpret_cast<const uint4*>(embed + (size_t)r * hidden);
        float acc = 0.0f;
#pragma unroll 4
        for (int i = lane; i < vec; i += 32) {
            const uint4 e = __ldg(src + i);
            const uint4 a = reinterpret_cast<const uint4*>(hs)[i];
            const __half2* eh = reinterpret_cast<const __half2*>(&e);
            const __half2* ah = reinterpret_cast<const __half2*>(&a);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 ef = __half22float2(eh[j]), af = __half22float2(ah[j]);
                acc = fmaf(ef.x, af.x, acc);
                acc = fmaf(ef.y, af.y, acc);
            }
        }
        acc = warp_sum_f(acc);  // xor butterfly: every lane ends with the same sum, same order for every row
        if (head_better(acc, r, best, best_row)) {
            best = acc;
            best_row = r;
        }
    }
    if (lane == 0) red[warp] = HeadBest{best, best_row};
    __syncthreads();
    if (threadIdx.x == 0) {
        HeadBest b = red[0];
        for (int w = 1; w < kHeadThreads / 32; ++w)
            if (head_better(red[w].val, red[w].row, b.val, b.row)) b = red[w];
        partial[blockIdx.x] = b;
    }
}

// ---- the tied embedding carried as int8 g64 (the reference's emb_q8.cu: w = scale * q + bias per group
// of 64 along the row, f16 scale and bias, one f32 multiply and one f32 add, never contracted) ----

__device__ __forceinline__ float q8_deq(unsigned int q, float s, float b) { return __fadd_rn(__fmul_rn(s, (float)q), b); }

// Greedy head over the int8 embedding: one row per warp and step, 16 codes (one 16-byte load, inside one
// group) per lane and step, f32 accumulation in a fixed order, argmax with the lowest row on ties.
// wq: [rows, hidden] u8, hidden % 16 == 0; scales / biases: [rows, hidden / 64] f16 (hidden % 64 == 0).
__global__ void __launch_bounds__(kHeadThreads)
lm_head_argmax_q8_kernel(const unsigned char* __restrict__ wq, const __half* __restrict__ scales,
                         const __half* __restrict__ biases, const __half* __restrict__ h, int rows, int hidden,
                         HeadBest* __restrict__ partial) {
    llvq_dependent_enter();
    __shared__ __align__(16) float hs[kHeadMaxHidden];
    __shared__ HeadBest red[kHeadThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < hidden; i += kHeadThreads) hs[i] = __half2float(h[i]);
    __syncthreads();
    const int vec = hidden / 16, gpr = hidden / 64;
    float best = -INFINITY;
    int best_row = 0x7fffffff;
    for (int r = blockIdx.x * (kHeadThreads / 32) + warp; r < rows; r += gridDim.x * (kHeadThreads / 32)) {
        const uint4* src = reinterpret_cast<const uint4*>(wq + (size_t)r * hidden);
        float acc = 0.0f;
#pragma unroll 2
        for (int i = lane; i < vec; i += 32) {
            const uint4 e = __ldg(src + i);
            const int g = i >> 2;  // 16 codes per step, 64 per group
            const float s = __half2float(scales[(size_t)r * gpr + g]), b = __half2float(biases[(size_t)r * gpr + g]);
            const unsigned int w4[4] = {e.x, e.y, e.z, e.w};
            const float* hv = hs + 16 * i;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc = __fmaf_rn(q8_deq(w4[j] & 0xffu, s, b), hv[4 * j], acc);
                acc = __fmaf_rn(q8_deq((w4[j] >> 8) & 0xffu, s, b), hv[4 * j + 1], acc);
                acc = __fmaf_rn(q8_deq((w4[j] >> 16) & 0xffu, s, b), hv[4 * j + 2], acc);
                acc = __fmaf_rn(q8_deq(w4[j] >> 24, s, b), hv[4 * j + 3], acc);
            }
        }
        acc = warp_sum_f(acc);
        if (head_better(acc, r, best, best_row)) {
            best = acc;
            best_row = r;
        }
    }
    if (lane == 0) red[warp] = HeadBest{best, best_row};
    __syncthreads();
    if (threadIdx.x == 0) {
        HeadBest b = red[0];
        for (int w = 1; w < kHeadThreads / 32; ++w)
            if (head_better(red[w].val, red[w].row, b.val, b.row)) b = red[w];
        partial[blockIdx.x] = b;
    }
}

// Token ids -> dequantised f16 rows, one CTA per token (emb_q8_gather): y[t, c] = f16(scale * q + bias).
__global__ void embed_gather_q8_kernel(const unsigned char* __restrict__ wq, const __half* __restrict__ scales,
                                       const __half* __restrict__ biases, const long long* __restrict__ ids,
                                       __half* __restrict__ y, int hidden, int rows) {
    llvq_dependent_enter();
    long long row = ids[blockIdx.x];
    if (row < 0 || row >= rows) row = 0;  // a token outside the vocabulary reads row 0 instead of foreign memory
    const int gpr = (hidden + 63) / 64;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const size_t g = (size_t)row * gpr + (c >> 6);
        y[(size_t)blockIdx.x * hidden + c] =
            __float2half_rn(q8_deq(wq[(size_t)row * hidden + c], __half2float(scales[g]), __half2float(biases[g])));
    }
}

// One CTA: merge the partials; the row index is reported with `row_offset` added (a vocabulary shard).
__global__ void __launch_bounds__(kHeadMaxGrid)
lm_head_pick_kernel(const HeadBest* __restrict__ partial, int n, long long row_offset, float* __restrict__ val_out,
                    long long* __restrict__ idx_out) {
    llvq_dependent_enter();
    __shared__ HeadBest red[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    HeadBest b = threadIdx.x < n ? partial[threadIdx.x] : HeadBest{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, b.val, o);
        const int r = __shfl_xor_sync(0xffffffffu, b.row, o);
        if (head_better(v, r, b.val, b.row)) b = HeadBest{v, r};
    }
    if (lane == 0) red[warp] = b;
    __syncthreads();
    if (warp == 0) {
        b = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float v = __shfl_xor_sync(0xffffffffu, b.val, o);
            const int r = __shfl_xor_sync(0xffffffffu, b.row, o);
            if (head_better(v, r, b.val, b.row)) b = HeadBest{v, r};
        }
        if (lane == 0) {
            *val_out = b.val;
            *idx_out = row_offset + (b.row == 0x7fffffff ? 0 : b.row);  // all-NaN logits: row 0
        }
    }
}

}  // namespace llvq
