// Class-sorted fused dequant-GEMV for sm_100a.
//
// One CTA owns kRows consecutive output rows. Their packed codes (a contiguous,
// 16-byte aligned slab of the archive stream) are brought into shared memory by
// one bulk asynchronous copy (cp.async.bulk, completion on an mbarrier). The row
// tile is then processed in chunks of up to kChunk column blocks:
//
//   phase 1  every thread takes blocks of the chunk: 48-bit big-endian record ->
//            (index, gain) -> class search -> local rank -> decode family. The
//            block's item is stored at its own position; its position is appended
//            to the list of its family (match.any + one shared-memory atomic per
//            family and warp).
//   phase 2  warps pull batches of 32 same-family items and run that family's
//            branch-free decoder (decode_fast.cuh) with the dot product against
//            the staged activation fused into its position loop; the block's
//            contribution, scaled by gain centroid / sqrt(16 m), goes to part[].
//   phase 3  one warp per row adds the chunk's partials in a fixed order.
//
// Sorting by family is what keeps the 32 lanes of a warp on one instruction
// stream: blocks of the odd coset (24-slot unranking) and of the even coset
// (table look-ups) cost very different amounts of work.
//
// The activation chunk is staged transposed, xs[pos][block] with an odd row
// stride, so that lanes holding different blocks read different banks; that
// transposition is why x takes ordinary loads rather than a bulk copy.
#pragma once
#include <cuda_fp16.h>

#include "decode_fast.cuh"
#include "decode_generic.cuh"
#include "kernels_generic.cuh"

namespace llvq {

constexpr int kChunk = 128;                    // column blocks per chunk
constexpr int kChunkPad = kChunk + 1;          // xs row stride (odd: conflict-free transposition)
constexpr int kThreads = 256;                  // 8 warps
constexpr int kWarps = kThreads / 32;
constexpr unsigned int kSpinLimit = 1u << 22;  // bounded wait on the bulk copy

// ROWS = rows per CTA (8 or 16; a multiple of 8 keeps the code slab 16-byte aligned).
// More rows per CTA mean more batches per chunk and so a better balance between the
// warps of phase 2; fewer rows mean more CTAs for matrices with few rows.
template <int ROWS>
struct alignas(16) SortedSmem {
    static constexpr int kItems = ROWS * kChunk;
    unsigned long long mbar;
    int count[4];  // items per family in this chunk
    int ticket;    // next batch to hand out
    int error;
    int pad[2];
    float2 cent[ROWS];
    float rscale[ROWS];
    float xs_tail[32];
    float part[kItems];
    uint2 items[kItems];  // local rank (47 bits) | class << 47 | gain << 56, at the block's own slot
    // Slots (row << 7 | block) of each family's blocks. Two families share one array, one
    // growing from the front and one from the back: even / odd-2 in list_a, odd-3 / generic in list_b.
    unsigned short list_a[kItems];
    unsigned short list_b[kItems];
    float xs[kDim * kChunkPad];
    // followed by the code slab (dynamic size)
};

__device__ __forceinline__ unsigned int smem_addr(const void* p) {
    return (unsigned int)__cvta_generic_to_shared(p);
}

// Starts the bulk copy of `bytes` (a multiple of 16) from 16-byte aligned global memory into shared
// memory; completion is signalled on `mbar`. Call from one thread, after the barrier has been
// initialised and that initialisation made visible by a __syncthreads().
__device__ __forceinline__ void bulk_load_issue(unsigned char* dst, const unsigned char* src, unsigned int bytes,
                                                unsigned long long* mbar) {
    const unsigned int bar = smem_addr(mbar);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// Bounded wait for phase `parity` of an mbarrier; false when the spin limit ran out. Meant for ONE
// polling thread: the rest of the CTA waits at the __syncthreads_and() that spreads the verdict.
__device__ __forceinline__ bool mbar_wait(unsigned long long* mbar, unsigned int parity) {
    const unsigned int bar = smem_addr(mbar);
    unsigned int done = 0;
    for (unsigned int spin = 0; spin < kSpinLimit && !done; ++spin) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
    }
    return done != 0;
}

// 48-bit big-endian record at byte offset 6 * f of the slab (2-byte aligned).
__device__ __forceinline__ unsigned long long slab_code48(const unsigned char* slab, int f) {
    const unsigned short* h = reinterpret_cast<const unsigned short*>(slab + 6 * f);
    const unsigned int h0 = h[0], h1 = h[1], h2 = h[2];
    const unsigned int hi = __byte_perm(h0, 0, 0x4401);                 // bytes 0,1 -> big-endian 16 bits
    const unsigned int lo = __byte_perm(h1, h2, 0x0145);                // bytes 2..5 -> big-endian 32 bits
    return ((unsigned long long)hi << 32) | lo;
}

// xs[pos * kChunkPad + b] = x[b * 24 + pos] for the n = 24 * blocks activations of a chunk.
// Eight consecutive activations (8 | 24, so they stay inside one block) per thread and step.
template <typename XT>
__device__ __forceinline__ void stage_x_chunk(float* xs, const XT* __restrict__ x, int n, int tid) {
    for (int i = tid * 8; i < n; i += kThreads * 8) {
        const int b = i / kDim, pos = i - b * kDim;
        float v[8];
        if constexpr (sizeof(XT) == 2) {
            const uint4 raw = *reinterpret_cast<const uint4*>(x + i);  // 16-byte aligned: i % 8 == 0
            const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f2 = __half22float2(h[k]);
                v[2 * k] = f2.x;
                v[2 * k + 1] = f2.y;
            }
        } else {
            const float4 lo = *reinterpret_cast<const float4*>(x + i);
            const float4 hi = *reinterpret_cast<const float4*>(x + i + 4);
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w;
            v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) xs[(pos + k) * kChunkPad + b] = v[k];
    }
}

// Position of entry i of a family's list inside its shared array.
template <int ROWS>
__device__ __forceinline__ unsigned short* list_slot(SortedSmem<ROWS>& S, unsigned int fam, int i) {
    constexpr int kItems = SortedSmem<ROWS>::kItems;
    unsigned short* base = (fam == kPathEven || fam == kPathOdd2) ? S.list_a : S.list_b;
    const bool front = fam == kPathEven || fam == kPathOdd3;
    return base + (front ? i : kItems - 1 - i);
}

template <typename XT, typename YT, int ROWS>
__global__ void __launch_bounds__(kThreads, 5)
gemv_sorted_kernel(FastTables F, DevTables G, MatrixView mv, const XT* __restrict__ x, YT* __restrict__ y,
                   int* __restrict__ err_flag, int split_range, float* __restrict__ split_ws,
                   int* __restrict__ split_counter) {
    using Smem = SortedSmem<ROWS>;
    constexpr int kRowsPerWarp = ROWS / kWarps;
    static_assert(ROWS % kWarps == 0 && sizeof(Smem) % 16 == 0, "rows split evenly; slab starts 16-byte aligned");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Smem& S = *reinterpret_cast<Smem*>(smem_raw);
    unsigned char* slab = smem_raw + sizeof(Smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = mv.nb;
    const int row0 = blockIdx.x * ROWS;
    const int rows = min(ROWS, mv.d_out - row0);

    if (tid < ROWS) {
        const int r = min(row0 + tid, mv.d_out - 1);
        S.cent[tid] = mv.cent[r];
        S.rscale[tid] = mv.rscale[r];
    }
    if (tid < 32) S.xs_tail[tid] = tid < mv.tail_w ? to_f32<XT>(x[nb * kDim + tid]) : 0.0f;
    if (tid == 0) {
        S.error = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&S.mbar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Column split: blockIdx.y owns the column blocks [cs0, cs1). A CTA that owns whole rows stages
    // their codes with one bulk copy; a CTA that owns a column range reads its codes from global
    // memory (its part of each row is neither contiguous with the next row's nor 16-byte aligned).
    const int cs0 = blockIdx.y * split_range, cs1 = min(nb, cs0 + split_range);
    const unsigned char* codes = mv.codes + (size_t)row0 * nb * 6;
    const bool use_slab = gridDim.y == 1 && nb > 0;
    if (use_slab) {
        // the slab start is 16-byte aligned because row0 is a multiple of 8 (48 * nb bytes per 8 rows);
        // the copy runs while the first activation chunk is being staged
        if (tid == 0) bulk_load_issue(slab, codes, ((unsigned int)rows * nb * 6 + 15u) & ~15u, &S.mbar);
        codes = slab;
    }

    float row_acc[kRowsPerWarp];  // phase 3: lane-replicated sums of the rows owned by this warp
#pragma unroll
    for (int q = 0; q < kRowsPerWarp; ++q) row_acc[q] = 0.0f;

    for (int cb0 = cs0; cb0 < cs1; cb0 += kChunk) {
        const int cbn = min(kChunk, cs1 - cb0);

        // ---- stage the activation chunk (transposed) and reset the queues ----
        stage_x_chunk<XT>(S.xs, x + (size_t)cb0 * kDim, cbn * kDim, tid);
        if (tid < 4) S.count[tid] = 0;
        if (tid == 0) S.ticket = 0;
        if (use_slab && cb0 == cs0) {
            // one thread waits (bounded) for the code slab; the barrier spreads its verdict
            const bool landed = tid != 0 || mbar_wait(&S.mbar, 0);
            if (!__syncthreads_and(landed)) {
                if (tid == 0) atomicOr(err_flag, 2);
                return;  // the copy never landed: report, do not touch the slab
            }
        } else {
            __syncthreads();
        }

        // ---- phase 1: classify; a warp takes rows warp, warp + 8, ..., a lane every 32nd block ----
#pragma unroll 1
        for (int k = 0; k < kRowsPerWarp * (kChunk / 32); ++k) {
            const int lr = warp + kWarps * (k / (kChunk / 32)), bl = lane + 32 * (k % (kChunk / 32));
            const int f = lr * kChunk + bl;
            unsigned int path = 4u;  // 4: nothing to decode
            if (lr < rows && bl < cbn) {
                const unsigned long long v = slab_code48(codes, lr * nb + cb0 + bl);
                const Classified c = classify12(F, v >> 1);
                if (c.ci >= 0) {
                    path = c.path;
                    const unsigned long long loc = c.local;
                    S.items[f] = make_uint2((unsigned int)loc, (unsigned int)(loc >> 32) | (unsigned int)c.ci << 15 |
                                                                   (unsigned int)(v & 1ull) << 24);
                } else {
                    S.part[f] = 0.0f;  // origin, or refused index: contributes nothing
                    if (c.ci == -2) S.error = 1;
                }
            }
            // lanes of the same family find each other; the lowest one reserves their list slots
            const unsigned int peers = __match_any_sync(0xffffffffu, path);
            const int leader = __ffs(peers) - 1;
            int first = 0;
            if (path < 4u && lane == leader) first = atomicAdd(&S.count[path], __popc(peers));
            first = __shfl_sync(0xffffffffu, first, leader);
            if (path < 4u) *list_slot<ROWS>(S, path, first + __popc(peers & ((1u << lane) - 1u))) = (unsigned short)f;
        }
        __syncthreads();

        // ---- phase 2: decode + dot, one family per batch; longest batches first ----
        const int n_slow = S.count[kPathSlow], n_o3 = S.count[kPathOdd3], n_o2 = S.count[kPathOdd2],
                  n_ev = S.count[kPathEven];
        const int b_slow = (n_slow + 31) >> 5, b_o3 = (n_o3 + 31) >> 5, b_o2 = (n_o2 + 31) >> 5, b_ev = (n_ev + 31) >> 5;
        const int total_batches = b_slow + b_o3 + b_o2 + b_ev;
        for (;;) {
            int t = 0;
            if (lane == 0) t = atomicAdd(&S.ticket, 1);
            t = __shfl_sync(0xffffffffu, t, 0);
            if (t >= total_batches) break;
            unsigned int fam;
            int first, count;
            if (t < b_slow) {
                fam = kPathSlow; first = 32 * t; count = n_slow - first;
            } else if (t < b_slow + b_o3) {
                fam = kPathOdd3; first = 32 * (t - b_slow); count = n_o3 - first;
            } else if (t < b_slow + b_o3 + b_o2) {
                fam = kPathOdd2; first = 32 * (t - b_slow - b_o3); count = n_o2 - first;
            } else {
                fam = kPathEven; first = 32 * (t - b_slow - b_o3 - b_o2); count = n_ev - first;
            }
            if (lane < count) {  // the last batch of a family may be ragged
                const int f = *list_slot<ROWS>(S, fam, first + lane);
                const uint2 it = S.items[f];
                const unsigned long long local = (unsigned long long)(it.y & 0x7fffu) << 32 | it.x;
                const int ci = (int)((it.y >> 15) & 0x1ffu);
                const unsigned int gain = (it.y >> 24) & 1u;
                const int lr = f >> 7, bl = f & (kChunk - 1);
                const float* xb = S.xs + bl;
                float acc = 0.0f, scale;
                auto dot = [&](int pos, float v) { acc = fmaf(v, xb[pos * kChunkPad], acc); };
                const FastClass* rec = F.cls + ci;
                if (fam == kPathEven) {
                    const Quad q0 = load_quad(rec, 0), q1 = load_quad(rec, 1), q2 = load_quad(rec, 2),
                               q3 = load_quad(rec, 3);
                    scale = bits_to_float(q3.x);
                    even_fast(F, local, q0.z, q1, q2, dot);
                } else if (fam == kPathSlow) {
                    decode_class12(G, ci, local, [&](int pos, int v) { acc = fmaf((float)v, xb[pos * kChunkPad], acc); },
                                   &scale);
                } else {
                    const Quad q0 = load_quad(rec, 0), q1 = load_quad(rec, 1);
                    unsigned int g, r;
                    divmod_odd(local, q0.z, bits_to_float(q1.w), &g, &r);
                    const unsigned int cw = __ldg(F.golay + g);
                    scale = bits_to_float(q1.z);
                    if (fam == kPathOdd2)
                        odd_fast<2>(r, q0.z, q1.x, q1.y, cw, dot);
                    else
                        odd_fast<3>(r, q0.z, q1.x, q1.y, cw, dot);
                }
                const float2 cg = S.cent[lr];
                S.part[f] = acc * (scale * (gain ? cg.y : cg.x));
            }
        }
        __syncthreads();

        // ---- phase 3: fixed-order row sums ----
#pragma unroll
        for (int q = 0; q < kRowsPerWarp; ++q) {
            const int lr = warp + kWarps * q;
            if (lr < rows) {
                float s = 0.0f;
                for (int b = lane; b < cbn; b += 32) s += S.part[lr * kChunk + b];
                row_acc[q] += warp_sum(s);
            }
        }
        // the next chunk's staging overwrites xs/items only; part is rewritten after two barriers
    }

    if (gridDim.y == 1) {
#pragma unroll
        for (int q = 0; q < kRowsPerWarp; ++q) {
            const int lr = warp + kWarps * q;
            if (lr < rows) {
                const int r = row0 + lr;
                const float t = tail_dot(mv, r, S.xs_tail, lane);
                if (lane == 0) store_y<YT>(y, r, fmaf(row_acc[q], S.rscale[lr], t));
            }
        }
    } else {
        // column split: publish this CTA's partial row sums; the CTA that arrives last at the row
        // tile's counter adds the partials in split order (so the result does not depend on which
        // CTA that is), finishes the rows and re-arms the counter for the next launch.
#pragma unroll
        for (int q = 0; q < kRowsPerWarp; ++q) {
            const int lr = warp + kWarps * q;
            if (lr < rows && lane == 0) split_ws[(size_t)blockIdx.y * mv.d_out + row0 + lr] = row_acc[q];
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) S.ticket = atomicAdd(&split_counter[blockIdx.x], 1) == (int)gridDim.y - 1;
        __syncthreads();
        if (S.ticket) {
            __threadfence();
#pragma unroll
            for (int q = 0; q < kRowsPerWarp; ++q) {
                const int lr = warp + kWarps * q;
                if (lr < rows) {
                    const int r = row0 + lr;
                    float s = 0.0f;
                    for (unsigned int k = 0; k < gridDim.y; ++k) s += __ldcg(split_ws + (size_t)k * mv.d_out + r);
                    const float t = tail_dot(mv, r, S.xs_tail, lane);
                    if (lane == 0) store_y<YT>(y, r, fmaf(s, S.rscale[lr], t));
                }
            }
            if (tid == 0) split_counter[blockIdx.x] = 0;
        }
    }
    __syncthreads();
    if (tid == 0 && S.error) atomicOr(err_flag, 1);
}

template <int ROWS>
inline size_t sorted_smem_bytes(int nb) {
    return sizeof(SortedSmem<ROWS>) + (((size_t)ROWS * nb * 6 + 15) & ~(size_t)15) + 16;
}

}  // namespace llvq
