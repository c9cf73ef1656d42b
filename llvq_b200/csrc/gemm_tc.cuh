// Batched dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   Y[B, d_out] = X[B, d_in] * W^T,  B >= 16 (speculative tree verify, prefill slices)
//
// Every code is decoded ONCE per batch: a CTA owns 128 rows of W and a range of
// column chunks (192 columns = 8 blocks per row = 1024 blocks per chunk). Per chunk
//   phase 1  classify the 1024 blocks into decode families (as the GEMV does);
//   phase 2  decode them family by family, 32 blocks per warp step, and write the
//            values, already scaled by gain centroid / sqrt(16 m), as f16 into the
//            A tile in shared memory (K-major, 128-byte swizzle, three 64-column panels);
//            the X chunk goes into the B tile in the same layout;
//   MMA      one thread issues 12 tcgen05.mma (M = 128, N = padded batch, K = 16) that
//            accumulate in TMEM, then tcgen05.commit onto an mbarrier. The next chunk's
//            classification overlaps the tensor work; its tile writes wait on the mbarrier.
// The f32 accumulators are read back with tcgen05.ld and stored as split-K partials; a
// second kernel adds the partials in a fixed order, applies the row scale and the f32/f16
// tail columns, and narrows to f16 once.
//
// Every wait is bounded; on a time-out the kernel raises the error word, still frees its
// TMEM columns and returns.
#pragma once
#include <cuda_fp16.h>

#include "decode_fast.cuh"
#include "decode_generic.cuh"
#include "gemv_sorted.cuh"  // smem_addr, kSpinLimit, warp helpers

namespace llvq {

constexpr int kGM = 128;                  // rows of W per CTA = MMA M
constexpr int kGKB = 8;                   // blocks per row and chunk: 8 * 24 = 192 = 3 * 64 columns
constexpr int kGItems = kGM * kGKB;       // 1024 blocks per chunk
constexpr int kGThreads = 512;
constexpr int kGMaxN = 64;                // padded batch per launch = MMA N
constexpr int kGPanelA = kGM * 128;       // bytes of one 64-column A panel
constexpr int kGPanelB = kGMaxN * 128;    // bytes of one 64-column B panel
constexpr unsigned int kGTmemCols = 64;   // accumulator columns (power of two >= 32)

struct alignas(1024) GemmSmem {
    unsigned char a[3][kGPanelA];  // 48 KB
    unsigned char b[3][kGPanelB];  // 24 KB
    uint2 items[kGItems];
    unsigned short list_a[kGItems];
    unsigned short list_b[kGItems];
    float2 cent[kGM];
    unsigned long long mbar;
    unsigned int tmem_base;
    int count[4];
    int ticket;
    int error;
};

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc_k128_at(unsigned long long addr) {
    unsigned long long d = (addr & 0x3FFFFull) >> 4;  // start address, 16-byte units
    d |= 1ull << 16;                                   // leading byte offset (unused with swizzle)
    d |= (1024ull >> 4) << 32;                         // stride byte offset between 8-row groups
    d |= 1ull << 46;                                   // descriptor version of sm_100
    d |= 2ull << 61;                                   // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ unsigned long long umma_desc_k128(const void* smem_ptr) {
    return umma_desc_k128_at(smem_addr(smem_ptr));
}

// Byte offset of 16-byte chunk `gc` (0..23 over the three panels) of row `r` in a swizzled tile.
__device__ __forceinline__ unsigned int swz_offset(int r, int gc, int panel_bytes) {
    return (unsigned int)((gc >> 3) * panel_bytes + r * 128 + (((gc & 7) ^ (r & 7)) << 4));
}

// Collects the 24 values of one block and writes them as three 16-byte chunks of f16.
struct TileWriter {
    unsigned int h[12];
    float even;
    float scale;
    __device__ __forceinline__ void put(int pos, float v) {
        if ((pos & 1) == 0) {
            even = v * scale;
        } else {
            const __half2 p = __floats2half2_rn(even, v * scale);
            h[pos >> 1] = *reinterpret_cast<const unsigned int*>(&p);
        }
    }
    __device__ __forceinline__ void store(unsigned char* a_tile, int row, int kb) const {
#pragma unroll
        for (int j = 0; j < 3; ++j)
            *reinterpret_cast<uint4*>(a_tile + swz_offset(row, 3 * kb + j, kGPanelA)) =
                make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
    }
};

struct GemmArgs {
    const __half* x;     // [batch, d_in]
    float* ws;           // [splits, n_pad, d_out] split-K partials
    int batch;           // valid rows of x
    int n_pad;           // batch rounded up to 16 (MMA N)
    int chunks_per_split;
    int x_vec_ok;        // x rows allow 16-byte loads
};

__device__ __forceinline__ unsigned short* gemm_list_slot(GemmSmem& S, unsigned int fam, int i) {
    unsigned short* base = (fam == kPathEven || fam == kPathOdd2) ? S.list_a : S.list_b;
    const bool front = fam == kPathEven || fam == kPathOdd3;
    return base + (front ? i : kGItems - 1 - i);
}

__global__ void __launch_bounds__(kGThreads, 2)
gemm_tc_kernel(FastTables F, DevTables G, MatrixView mv, GemmArgs ga, int* __restrict__ err_flag) {
    extern __shared__ unsigned char gsm_raw[];
    // the swizzled panels need 1024-byte alignment in the shared window: round the base up by hand
    GemmSmem& S = *reinterpret_cast<GemmSmem*>(gsm_raw + ((1024u - (smem_addr(gsm_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = mv.nb;
    const int row0 = blockIdx.x * kGM;
    const int split = blockIdx.y;
    const int n_chunks = (nb + kGKB - 1) / kGKB;
    const int c_begin = split * ga.chunks_per_split;
    const int c_end = min(n_chunks, c_begin + ga.chunks_per_split);

    if (tid < kGM) S.cent[tid] = mv.cent[min(row0 + tid, mv.d_out - 1)];
    if (tid == 0) {
        S.error = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&S.mbar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // one warp allocates the accumulator columns and gives the permit back
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&S.tmem_base)),
                     "r"(kGTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned int tmem = S.tmem_base;
    // instruction descriptor: D = f32, A = B = f16, both K-major, N = n_pad, M = 128
    const unsigned int idesc = (1u << 4) | ((unsigned int)(ga.n_pad >> 3) << 17) | ((unsigned int)(kGM >> 4) << 24);
    bool ok = true;

    for (int c = c_begin; c < c_end && ok; ++c) {
        const int cb0 = c * kGKB;
        if (tid < 4) S.count[tid] = 0;
        if (tid == 0) S.ticket = 0;
        __syncthreads();

        // ---- phase 1: classify (touches neither tile, so it overlaps the previous chunk's MMAs) ----
        unsigned int zero_mask = 0;  // my blocks that decode to nothing: their tile entries must read zero
#pragma unroll 1
        for (int k = 0; k < kGItems / kGThreads; ++k) {
            const int f = tid + k * kGThreads;
            const int lr = f >> 3, kb = f & 7;
            unsigned int path = 4u;
            if (row0 + lr < mv.d_out && cb0 + kb < nb) {
                const unsigned long long v = load_code48(mv.codes, (size_t)(row0 + lr) * nb + cb0 + kb);
                const Classified cl = classify12(F, v >> 1);
                if (cl.ci >= 0) {
                    path = cl.path;
                    const unsigned long long loc = path == kPathSlow ? (v >> 1) : cl.local;
                    S.items[f] = make_uint2((unsigned int)loc, (unsigned int)(loc >> 32) | (unsigned int)cl.ci << 15 |
                                                                   (unsigned int)(v & 1ull) << 24);
                } else if (cl.ci == -2) {
                    S.error = 1;
                }
            }
            if (path == 4u) zero_mask |= 1u << k;
            const unsigned int peers = __match_any_sync(0xffffffffu, path);
            const int leader = __ffs(peers) - 1;
            int first = 0;
            if (path < 4u && lane == leader) first = atomicAdd(&S.count[path], __popc(peers));
            first = __shfl_sync(0xffffffffu, first, leader);
            if (path < 4u) *gemm_list_slot(S, path, first + __popc(peers & ((1u << lane) - 1u))) = (unsigned short)f;
        }

        // ---- the tiles are free once the previous chunk's MMAs have completed ----
        if (c > c_begin && tid == 0) ok = mbar_wait(&S.mbar, (unsigned int)((c - c_begin - 1) & 1));  // one poller
        ok = __syncthreads_and(ok);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // zero the blocks nobody decodes; stage the X chunk as the B tile (rows beyond the batch and
        // columns beyond the last block read zero so that no stray NaN meets a zero weight)
#pragma unroll
        for (int k = 0; k < kGItems / kGThreads; ++k)
            if (zero_mask >> k & 1u) {
                const int f = tid + k * kGThreads;
#pragma unroll
                for (int j = 0; j < 3; ++j)
                    *reinterpret_cast<uint4*>(&S.a[0][0] + swz_offset(f >> 3, 3 * (f & 7) + j, kGPanelA)) =
                        make_uint4(0, 0, 0, 0);
            }
        for (int i = tid; i < ga.n_pad * 24; i += kGThreads) {
            const int n = i / 24, gc = i - n * 24;
            const int col = cb0 * kDim + gc * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (n < ga.batch && col + 8 <= nb * kDim) {
                const __half* src = ga.x + (size_t)n * mv.d_in + col;
                if (ga.x_vec_ok) {
                    v = *reinterpret_cast<const uint4*>(src);
                } else {
                    unsigned short e[8];
#pragma unroll
                    for (int t = 0; t < 8; ++t) e[t] = reinterpret_cast<const unsigned short*>(src)[t];
                    v = make_uint4(e[0] | (unsigned int)e[1] << 16, e[2] | (unsigned int)e[3] << 16,
                                   e[4] | (unsigned int)e[5] << 16, e[6] | (unsigned int)e[7] << 16);
                }
            }
            *reinterpret_cast<uint4*>(&S.b[0][0] + swz_offset(n, gc, kGPanelB)) = v;
        }
        __syncthreads();

        // ---- phase 2: decode, one family per batch of 32 blocks, into the A tile ----
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
            if (lane < count) {
                const int f = *gemm_list_slot(S, fam, first + lane);
                const uint2 it = S.items[f];
                const unsigned long long local = (unsigned long long)(it.y & 0x7fffu) << 32 | it.x;
                const int ci = (int)((it.y >> 15) & 0x1ffu);
                const unsigned int gain = (it.y >> 24) & 1u;
                const int lr = f >> 3, kb = f & 7;
                const float2 cg = S.cent[lr];
                const float gsel = gain ? cg.y : cg.x;
                const FastClass* rec = F.cls + ci;
                TileWriter tw;
                tw.even = 0.0f;
                auto put = [&](int pos, float v) { tw.put(pos, v); };
                if (fam == kPathEven) {
                    const Quad q0 = load_quad(rec, 0), q1 = load_quad(rec, 1), q2 = load_quad(rec, 2),
                               q3 = load_quad(rec, 3);
                    tw.scale = bits_to_float(q3.x) * gsel;
                    even_fast(F, local, q0.z, q1, q2, put);
                } else if (fam == kPathSlow) {
                    // the generic decoder reports the scale only at the end: collect raw values first
                    float sc;
                    tw.scale = 1.0f;
                    decode_generic12(G, local, [&](int pos, int v) { tw.put(pos, (float)v); }, &sc);
                    const __half2 s2 = __float2half2_rn(sc * gsel);
#pragma unroll
                    for (int q = 0; q < 12; ++q) {
                        const __half2 p = __hmul2(*reinterpret_cast<const __half2*>(&tw.h[q]), s2);
                        tw.h[q] = *reinterpret_cast<const unsigned int*>(&p);
                    }
                } else {
                    const Quad q0 = load_quad(rec, 0), q1 = load_quad(rec, 1);
                    unsigned int g, r;
                    divmod_odd(local, q0.z, bits_to_float(q1.w), &g, &r);
                    const unsigned int cw = __ldg(F.golay + g);
                    tw.scale = bits_to_float(q1.z) * gsel;
                    if (fam == kPathOdd2)
                        odd_fast<2>(r, q0.z, q1.x, q1.y, cw, put);
                    else
                        odd_fast<3>(r, q0.z, q1.x, q1.y, cw, put);
                }
                tw.store(&S.a[0][0], lr, kb);
            }
        }
        // generic-proxy writes must be visible to the tensor core's asynchronous reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();

        // ---- MMA: 3 panels x 4 K-steps of 16, accumulating in TMEM ----
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                const unsigned long long da = umma_desc_k128(&S.a[p][0]), db = umma_desc_k128(&S.b[p][0]);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const unsigned int accumulate = (c > c_begin || p > 0 || kk > 0) ? 1u : 0u;
                    // +32 bytes (two 16-byte units) per K-step inside a swizzled 128-byte row
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                        ::"r"(tmem), "l"(da + 2ull * kk), "l"(db + 2ull * kk), "r"(idesc), "r"(accumulate), "r"(0u),
                        "r"(0u), "r"(0u), "r"(0u)
                        : "memory");
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_addr(&S.mbar))
                         : "memory");
        }
    }

    // ---- epilogue: wait for the last MMAs, read the accumulators, store the split-K partials ----
    if (ok && c_end > c_begin && tid == 0) ok = mbar_wait(&S.mbar, (unsigned int)((c_end - c_begin - 1) & 1));
    ok = __syncthreads_and(ok);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok && warp < 4 && c_end > c_begin) {
        const int row = row0 + 32 * warp + lane;  // warp w may touch TMEM lanes 32w .. 32w + 31
        float* dst = ga.ws + (size_t)split * ga.n_pad * mv.d_out;
        for (int n0 = 0; n0 < ga.n_pad; n0 += 8) {
            unsigned int r[8];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                         : "r"(tmem + ((unsigned int)(32 * warp) << 16) + (unsigned int)n0));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < mv.d_out) {
#pragma unroll
                for (int q = 0; q < 8; ++q) dst[(size_t)(n0 + q) * mv.d_out + row] = __uint_as_float(r[q]);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGTmemCols) : "memory");
    if (tid == 0) {
        if (!ok) atomicOr(err_flag, 2);
        if (S.error) atomicOr(err_flag, 1);
    }
}

// y[n, r] = f16( (sum_s ws[s, n, r]) * rscale[r] + tail[r, :] . x[n, 24 nb :] ), partials added in split order.
__global__ void gemm_reduce_kernel(MatrixView mv, const __half* __restrict__ x, const float* __restrict__ ws,
                                   __half* __restrict__ y, int batch, int n_pad, int splits) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = blockIdx.y;
    if (r >= mv.d_out || n >= batch) return;
    float s = 0.0f;
    for (int k = 0; k < splits; ++k) s += ws[((size_t)k * n_pad + n) * mv.d_out + r];
    float t = 0.0f;
    const __half* xt = x + (size_t)n * mv.d_in + (size_t)mv.nb * kDim;
    for (int q = 0; q < mv.tail_w; ++q) {
        const float w = mv.tail_f16 ? __half2float(((const __half*)mv.tail)[(size_t)r * mv.tail_w + q])
                                    : ((const float*)mv.tail)[(size_t)r * mv.tail_w + q];
        t = fmaf(w, __half2float(xt[q]), t);
    }
    y[(size_t)n * mv.d_out + r] = __float2half_rn(fmaf(s, mv.rscale[r], t));
}

inline size_t gemm_smem_bytes() { return sizeof(GemmSmem) + 1024; }

}  // namespace llvq
