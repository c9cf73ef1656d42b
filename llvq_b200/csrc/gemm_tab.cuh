// Batched dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a,
// decoding with the state-table decoders of decode_tab.cuh.
//
//   Y[B, d_out] = X[B, d_in] * W^T,  B >= 16 (speculative tree verify, prefill slices)
//
// Every code is decoded ONCE per batch. One persistent CTA of 1024 threads per SM keeps
// the decoder tables in shared memory and runs as TWO independent halves of 16 warps, each
// with its own operand tiles, lists, barriers and accumulator columns (what two CTAs per
// SM would be, if two copies of the tables fitted): while one half waits for its slowest
// warp or for its tensor-core work to drain, the other half decodes. A half walks a static
// list of work units: a unit is 128 rows of W times a range of column chunks (96 columns =
// 4 blocks per row = 512 blocks per chunk, one per thread of the half). Per chunk
//   decode    warps draw batches of 32 same-family blocks (lists written one chunk
//             ahead), run that family's decoder, scale the 24 signed bytes by
//             gain centroid / sqrt(16 m) and write them as f16 into the A tile in shared
//             memory (K-major, 64-byte swizzle, three 32-column panels); the X chunk goes
//             into the B tile in the same layout by cp.async, under the decoding;
//   classify  the warps that are done classify the NEXT chunk (48-bit record -> class ->
//             family list) instead of waiting at the barrier: items, lists and counters
//             are double (triple) buffered, the groups of 32 blocks are handed out by tickets;
//   MMA       one thread issues 6 tcgen05.mma (M = 128, N = padded batch, K = 16) that
//             accumulate in TMEM and commits them onto an mbarrier; the tiles are free
//             again when that barrier completes.
// After the last chunk of a unit the f32 accumulators are read back with tcgen05.ld and
// stored as split-K partials; gemm_reduce_kernel adds the partials in a fixed
// order, applies the row scale and the tail columns, and narrows to f16 once.
//
// Every wait is bounded; on a time-out the half raises the error word and stops, the CTA still
// frees its TMEM columns and returns.
#pragma once
#include <cuda_fp16.h>

#include "gemv_pipe.cuh"  // bulk copies, bounded mbarrier waits, group barriers

namespace llvq {

constexpr int kGM = 128;                  // rows of W per unit = MMA M
constexpr int kGKB = 4;                   // blocks per row and chunk: 4 * 24 = 96 = 3 * 32 columns
constexpr int kGItems = kGM * kGKB;       // 512 blocks per chunk
constexpr int kGMaxN = 64;                // padded batch per launch = MMA N
constexpr int kGPanelA = kGM * 64;        // bytes of one 32-column A panel
constexpr int kGPanelB = kGMaxN * 64;     // bytes of one 32-column B panel
constexpr unsigned int kGTmemCols = 64;   // accumulator columns of one half (power of two >= 32)
constexpr int kTGThreads = 1024;
constexpr int kTGHalves = 2;
constexpr int kTGHalfThreads = kTGThreads / kTGHalves;
constexpr int kTGHalfWarps = kTGHalfThreads / 32;
static_assert(kGItems == kTGHalfThreads, "one block of a chunk per thread of a half");
static_assert(kGMaxN * 12 <= 2 * kTGHalfThreads, "two pieces of the B tile per thread");
static_assert(kTGHalfThreads == kGroupThreads, "the halves use the group barriers of gemv_pipe.cuh");
// A row's 4 records of a chunk (24 bytes, 2-byte aligned) are fetched as the 16-byte aligned range around
// them: at most 14 + 24 bytes, rounded up to 48.
constexpr unsigned int kGSlabLine = 48;
constexpr int kGSlabThreads = kGM * 3;  // one 16-byte piece of the slab per thread

// Shared-memory matrix descriptor: K-major operand, 64-byte swizzle, 8-row groups 512 bytes apart.
__device__ __forceinline__ unsigned long long umma_desc_k64_at(unsigned long long addr) {
    unsigned long long d = (addr & 0x3FFFFull) >> 4;  // start address, 16-byte units
    d |= 1ull << 16;                                   // leading byte offset (unused with swizzle)
    d |= (512ull >> 4) << 32;                          // stride byte offset between 8-row groups
    d |= 1ull << 46;                                   // descriptor version of sm_100
    d |= 4ull << 61;                                   // SWIZZLE_64B
    return d;
}

// Byte offset of 16-byte piece `gc` (0..11 over the three panels) of row `r` in a tile of 64-byte rows with
// the 64-byte swizzle: inside every 512-byte group of 8 rows, address bits 4-5 are XORed with bits 7-8.
__device__ __forceinline__ unsigned int swz_offset(int r, int gc, int panel_bytes) {
    return (unsigned int)((gc >> 2) * panel_bytes + r * 64 + (((gc & 3) ^ ((r >> 1) & 3)) << 4));
}

struct GemmArgs {
    const __half* x;     // [batch, d_in]
    float* ws;           // [splits, n_pad, d_out] split-K partials
    int batch;           // valid rows of x
    int n_pad;           // batch rounded up to 16 (MMA N)
    int x_vec_ok;        // x rows allow 16-byte loads
};

struct GemmTabPlan {
    unsigned int blob;    // decoder tables
    unsigned int tiles;   // per half: A panels (3 x 8 KB) then B panels (3 x 4 KB); 1024-byte aligned in the shared window
    unsigned int items;   // per half: 2 x 512 x 8
    unsigned int lists;   // per half: 2 x 2 x 512 x 2
    unsigned int slab;    // per half: packed codes of one chunk, 128 lines of 48 bytes
    unsigned int ctrl;
    unsigned int total;
    int units, splits, chunks_per_split, row_tiles;
};

// Position of a half in its sequence of chunks: unit = row tile * splits + split.
struct alignas(16) GemmTabIt {
    int unit, useq, c, c_end, row0, split;
    int valid, first, last, pad;
    __device__ __forceinline__ void open(int u, int seq, const GemmTabPlan& P, int n_chunks) {
        unit = u;
        useq = seq;
        valid = u < P.units ? 1 : 0;
        const int rt = u / P.splits;
        split = u - rt * P.splits;
        row0 = rt * kGM;
        c = split * P.chunks_per_split;
        c_end = min(n_chunks, c + P.chunks_per_split);
        first = 1;
        last = c + 1 >= c_end ? 1 : 0;
    }
    __device__ __forceinline__ void step(const GemmTabPlan& P, int n_chunks, int stride) {
        if (c + 1 < c_end) {
            ++c;
            first = 0;
            last = c + 1 >= c_end ? 1 : 0;
        } else {
            open(unit + stride, useq + 1, P, n_chunks);
        }
    }
};

struct alignas(16) GemmTabShared {
    unsigned long long mbar_tab[2];  // decoder tables: classification part, decode part
    unsigned int tmem_base;
    int error;
};
struct alignas(16) GemmTabCtrl {     // one per half
    unsigned long long mbar_mma;
    unsigned long long mbar_slab;    // codes of chunk q: completion number q
    alignas(16) int count[3][4];     // items per family of chunk q at count[q % 3]
    int ticket[3];
    int cticket[3];                  // groups of 32 blocks of chunk q handed out for classification
    unsigned int zero[2][kTGHalfWarps];  // blocks of chunk q that decode to nothing, one bit per block, at zero[q & 1]
    int done_row0, done_split;       // the unit whose accumulators are read back next (written by the half's thread 0)
    GemmTabIt it[3];                 // chunk q of this half at it[q % 3]; thread 0 writes chunk q + 2 during iteration q
    float2 cent[2][kGM];             // gain centroids of the rows of the k-th unit of this half at cent[k & 1]
};

__device__ __forceinline__ unsigned int gemm_tab_list_slot(unsigned int lists, unsigned int fam, int i) {
    // the rare and four-kind lists share one array from both ends, the three-kind and even lists the other
    const unsigned int arr = lists + ((fam == kFamOdd3 || fam == kFamEven) ? 2u * kGItems : 0u);
    const bool front = fam == kFamOdd4 || fam == kFamEven;
    return arr + 2u * (unsigned int)(front ? i : kGItems - 1 - i);
}

__global__ void __launch_bounds__(kTGThreads, 1)
llvq_gemm_tab_kernel(const unsigned char* __restrict__ blob_g, const OffEntry* __restrict__ lut_off,
                     const unsigned long long* __restrict__ lut_on3, TabLayout L, MatrixView mv, GemmArgs ga, GemmTabPlan P,
                     int* __restrict__ err_flag) {
    extern __shared__ __align__(128) unsigned char gts_raw[];
    const unsigned int sbase = pipe_smem_addr(gts_raw);
    const int tid = threadIdx.x;
    const int half = tid / kTGHalfThreads;
    const int gt = tid - half * kTGHalfThreads, lane = gt & 31, warp = gt >> 5;  // position inside the half
    // the swizzled panels need 1024-byte alignment in the shared window
    const unsigned int pad = (1024u - ((sbase + P.tiles) & 1023u)) & 1023u;
    const unsigned int a_tile = sbase + P.tiles + pad + (unsigned int)half * (3u * kGPanelA + 3u * kGPanelB);  // shared-window addresses
    const unsigned int b_tile = a_tile + 3u * kGPanelA;
    GemmTabShared& S = *reinterpret_cast<GemmTabShared*>(gts_raw + P.ctrl);
    GemmTabCtrl& C = reinterpret_cast<GemmTabCtrl*>(gts_raw + P.ctrl + sizeof(GemmTabShared))[half];
    const int nb = mv.nb;
    const int n_chunks = (nb + kGKB - 1) / kGKB;

    TabView T;
    T.base = sbase + P.blob;
    T.lut_off = lut_off;
    T.lut_on3 = lut_on3;
    T.L = L;

    if (tid == 0) {
        S.error = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pipe_smem_addr(&S.mbar_tab[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pipe_smem_addr(&S.mbar_tab[1])));
    }
    if (gt == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pipe_smem_addr(&C.mbar_mma)));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pipe_smem_addr(&C.mbar_slab)), "r"(kGSlabThreads));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The half's position in its chunk sequence lives in shared memory (every thread would otherwise carry it
        // in registers across the decoders): thread 0 steps it two chunks ahead, barriers publish it.
        GemmTabIt it;
        it.open((int)blockIdx.x * kTGHalves + half, 0, P, n_chunks);
        it.pad = 0;
        C.it[0] = it;
        if (it.valid) it.step(P, n_chunks, (int)gridDim.x * kTGHalves);
        C.it[1] = it;
    }
    if (gt < 12) (&C.count[0][0])[gt] = 0;
    if (gt < 3) C.ticket[gt] = C.cticket[gt] = 0;
    if (tid < 32) {  // one warp allocates the accumulator columns of both halves and gives the permit back
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pipe_smem_addr(&S.tmem_base)),
                     "r"(kGTmemCols * kTGHalves)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // Programmatic dependent launch: the next kernel of the stream (the reduce kernel, then the next projection)
    // may be scheduled as soon as this CTA leaves its SM; this launch came this far under the previous kernel's tail.
    asm volatile("griddepcontrol.launch_dependents;");
    if (tid == 0) {
        pipe_expect_tx(pipe_smem_addr(&S.mbar_tab[0]), L.classify_bytes);
        pipe_bulk_copy(T.base, blob_g, L.classify_bytes, pipe_smem_addr(&S.mbar_tab[0]));
        pipe_expect_tx(pipe_smem_addr(&S.mbar_tab[1]), L.total_bytes - L.classify_bytes);
        pipe_bulk_copy(T.base + L.classify_bytes, blob_g + L.classify_bytes, L.total_bytes - L.classify_bytes,
                       pipe_smem_addr(&S.mbar_tab[1]));
    }
    bool ok = true;
    {
        const bool landed = tid != 0 || pipe_mbar_wait(pipe_smem_addr(&S.mbar_tab[0]));
        ok = __syncthreads_and(landed);
    }

    // Asynchronous copy of a chunk's packed codes into the slab: threads 0 .. 383 of the half bring one 16-byte
    // piece each (three pieces per row: the 16-byte aligned range around the row's 24 bytes; the code stream
    // carries 64 bytes of padding, so the last piece may run past the last record) and arrive on the slab barrier
    // when their piece has landed. A bulk copy per row would be 128 small requests per chunk, which the copy
    // engine serves slower than a chunk is decoded.
    const unsigned int slab = sbase + P.slab + (unsigned int)half * (kGM * kGSlabLine), bar_slab = pipe_smem_addr(&C.mbar_slab);
    auto issue_slab = [&](const GemmTabIt& it) {
        if (gt < kGSlabThreads) {
            const int lr = gt / 3, piece = gt - 3 * lr;
            const int ncols = min(kGKB, nb - it.c * kGKB);
            if (it.row0 + lr < mv.d_out) {
                const unsigned char* src = mv.codes + ((size_t)(it.row0 + lr) * nb + (size_t)it.c * kGKB) * 6;
                const unsigned int sh = (unsigned int)((uintptr_t)src & 15u);
                if (16u * piece < sh + (unsigned int)ncols * 6u)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(slab + (unsigned int)lr * kGSlabLine + 16u * piece),
                                 "l"(src - sh + 16 * piece)
                                 : "memory");
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_slab) : "memory");
        }
    };

    // Classification of chunk `it` (sequence number q, codes in the slab). Warps draw groups of 32 blocks from a
    // ticket counter, so the warps that finish their decode batches early classify more of the next chunk and
    // the warps with the long batches none. A block that decodes to nothing is noted in C.zero (its A entries
    // must read zero). Returns false when the wait for the codes ran out.
    auto classify = [&](const GemmTabIt& it, int q) -> bool {
        const unsigned int items = sbase + P.items + (unsigned int)(2 * half + (q & 1)) * (8u * kGItems);
        const unsigned int lists = sbase + P.lists + (unsigned int)(2 * half + (q & 1)) * (4u * kGItems);
        int* count = C.count[q % 3];
        if (it.first && gt < kGM) C.cent[it.useq & 1][gt] = __ldg(mv.cent + min(it.row0 + gt, mv.d_out - 1));
        if (!__all_sync(0xffffffffu, pipe_mbar_wait(bar_slab, (unsigned int)q & 1u))) return false;  // warp-uniform
        for (;;) {
            int g = 0;
            if (lane == 0) g = atomicAdd(&C.cticket[q % 3], 1);
            g = __shfl_sync(0xffffffffu, g, 0);
            if (g >= kTGHalfWarps) break;
            const int f = 32 * g + lane, lr = f >> 2, kb = f & 3;
            unsigned int fam = 4u;
            if (it.row0 + lr < mv.d_out && it.c * kGKB + kb < nb) {
                const unsigned int sh = (unsigned int)((uintptr_t)(mv.codes + ((size_t)(it.row0 + lr) * nb + (size_t)it.c * kGKB) * 6) & 15u);
                const unsigned int ca = slab + (unsigned int)lr * kGSlabLine + sh + 6u * (unsigned int)kb;  // 2-byte aligned
                unsigned int h0, h1, h2;
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(h0) : "r"(ca));
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(h1) : "r"(ca + 2u));
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(h2) : "r"(ca + 4u));
                const unsigned int hi = __byte_perm(h0, 0, 0x4401);   // bytes 0,1 -> big-endian 16 bits
                const unsigned int lo = __byte_perm(h1, h2, 0x0145);  // bytes 2..5 -> big-endian 32 bits
                const TabClassified cl = tab_classify(T, ((unsigned long long)hi << 32) | lo);
                if (cl.fam >= 0) {
                    fam = (unsigned int)cl.fam;
                    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(items + 8u * f), "r"((unsigned int)cl.local2),
                                 "r"((unsigned int)(cl.local2 >> 32) | (unsigned int)cl.ci << 13)
                                 : "memory");
                } else if (cl.fam == -2) {
                    S.error = 1;
                }
            }
            const unsigned int none = __ballot_sync(0xffffffffu, fam == 4u);
            if (lane == 0) C.zero[q & 1][g] = none;
            const unsigned int peers = __match_any_sync(0xffffffffu, fam);
            const int leader = __ffs(peers) - 1;
            int first = 0;
            if (fam < 4u && lane == leader) first = atomicAdd(&count[fam], __popc(peers));
            first = __shfl_sync(0xffffffffu, first, leader);
            if (fam < 4u) {
                const unsigned int a = gemm_tab_list_slot(lists, fam, first + __popc(peers & ((1u << lane) - 1u)));
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"((unsigned short)f) : "memory");
            }
        }
        return true;
    };

    // The X chunk of a chunk becomes the B tile: piece i (of n_pad * 12 16-byte pieces) goes from global memory
    // straight to its swizzled place with cp.async, so the copy runs under the decode phase and takes no register;
    // rows beyond the batch and columns beyond the last block are zero-filled (src-size 0) so that no stray NaN
    // meets a zero weight. Activations whose rows do not allow 16-byte loads take the slow path through registers.
    auto stage_x = [&](const GemmTabIt& it) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = gt + k * kTGHalfThreads;
            if (i >= ga.n_pad * 12) break;
            const int n = i / 12, gc = i - n * 12;
            const int col = it.c * kGKB * kDim + gc * 8;
            const bool live = n < ga.batch && col + 8 <= nb * kDim;
            const __half* src = ga.x + (live ? (size_t)n * mv.d_in + col : 0);
            const unsigned int dst = b_tile + swz_offset(n, gc, kGPanelB);
            if (ga.x_vec_ok) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0) : "memory");
            } else {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (live) {
                    const unsigned short* e = reinterpret_cast<const unsigned short*>(src);
                    v.x = e[0] | (unsigned int)e[1] << 16;
                    v.y = e[2] | (unsigned int)e[3] << 16;
                    v.z = e[4] | (unsigned int)e[5] << 16;
                    v.w = e[6] | (unsigned int)e[7] << 16;
                }
                sts128(dst, v);
            }
        }
    };

    // Accumulators of a finished unit -> split-K partials ws[split][n][row] (warps 0-3 of the half: a warp may
    // touch the TMEM lanes 32 (warp % 4) .. + 31, and warps 0-3 of either half have warp % 4 = their index).
    auto store_unit = [&]() {
        if (warp < 4) {
            const unsigned int tmem = S.tmem_base + (unsigned int)half * kGTmemCols;
            const int row = C.done_row0 + 32 * warp + lane;
            float* dst = ga.ws + (size_t)C.done_split * ga.n_pad * mv.d_out + row;
            for (int n0 = 0; n0 < ga.n_pad; n0 += 4) {
                unsigned int r[4];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                             : "r"(tmem + ((unsigned int)(32 * warp) << 16) + (unsigned int)n0));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < mv.d_out) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) dst[(size_t)(n0 + k) * mv.d_out] = __uint_as_float(r[k]);
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    bool prev_last = false;  // the previous chunk closed its unit: read the accumulators back before the next MMA
    {
        bool landed = true;
        if (ok && C.it[0].valid) issue_slab(C.it[0]);
        // x may be the previous kernel's output and the split-K workspace may still be read by the previous
        // projection's reduce kernel: from here on the previous kernel of the stream has completed (no-op for an
        // ordinary launch). Tables and codes, all that was touched so far, are constant.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (ok && C.it[0].valid) {
            landed = classify(C.it[0], 0);
        }
        // the decode tables must have landed before the first decode; the first chunk's lists are complete
        landed = landed && (tid != 0 || pipe_mbar_wait(pipe_smem_addr(&S.mbar_tab[1])));
        ok = __syncthreads_and(landed && ok);
    }

    int q = 0;  // chunks issued so far by this half = groups of MMAs committed on its mbar_mma
    for (; ok && C.it[q % 3].valid; ++q) {
        const GemmTabIt& cur = C.it[q % 3];
        // ---- the tiles are free once the previous chunk's MMAs have completed ----
        if (q > 0) {  // chunk q - 1 was commit number q - 1 on the barrier
            const bool done = gt != 0 || pipe_mbar_wait(pipe_smem_addr(&C.mbar_mma), (unsigned int)((q - 1) & 1));
            ok = pipe_group_sync_and(half, done);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        if (gt == 0) {  // counters and position of the chunk after the next one
#pragma unroll
            for (int k = 0; k < 4; ++k) C.count[(q + 2) % 3][k] = 0;
            C.ticket[(q + 2) % 3] = 0;
            C.cticket[(q + 2) % 3] = 0;
            GemmTabIt it = C.it[(q + 1) % 3];
            if (it.valid) it.step(P, n_chunks, (int)gridDim.x * kTGHalves);
            C.it[(q + 2) % 3] = it;
        }
        const unsigned int items = sbase + P.items + (unsigned int)(2 * half + (q & 1)) * (8u * kGItems);
        const unsigned int lists = sbase + P.lists + (unsigned int)(2 * half + (q & 1)) * (4u * kGItems);
        // the slab is free (chunk q was classified before the last barrier): fetch the next chunk's codes
        if (C.it[(q + 1) % 3].valid) issue_slab(C.it[(q + 1) % 3]);
        // zero the block nobody decodes; start the X chunk on its way into the B tile
        if ((C.zero[q & 1][warp] >> lane) & 1u) {
#pragma unroll
            for (int j = 0; j < 3; ++j)
                sts128(a_tile + swz_offset(gt >> 2, 3 * (gt & 3) + j, kGPanelA), make_uint4(0, 0, 0, 0));
        }
        stage_x(cur);  // lands while the chunk is decoded
        // the finished unit's accumulators are overwritten by this chunk's first MMA (after the next barrier)
        if (prev_last) store_unit();

        // ---- decode: one family per batch of 32 blocks, into the A tile ----
        // (the family counts are re-read from shared memory for every batch: nothing but the ticket stays in
        // registers across a decoder)
        for (;;) {
            int t = 0;
            if (lane == 0) t = atomicAdd(&C.ticket[q % 3], 1);
            t = __shfl_sync(0xffffffffu, t, 0);
            const int4 cn = *reinterpret_cast<const int4*>(C.count[q % 3]);  // rare, odd3, odd4, even (TabFamily order)
            const int b_rare = (cn.x + 31) >> 5, b_o4 = (cn.z + 31) >> 5, b_o3 = (cn.y + 31) >> 5, b_ev = (cn.w + 31) >> 5;
            if (t >= b_rare + b_o4 + b_o3 + b_ev) break;
            unsigned int fam;
            int first, cnt;
            if (t < b_rare) {
                fam = kFamRare; first = 32 * t; cnt = cn.x - first;
            } else if (t < b_rare + b_o4) {
                fam = kFamOdd4; first = 32 * (t - b_rare); cnt = cn.z - first;
            } else if (t < b_rare + b_o4 + b_o3) {
                fam = kFamOdd3; first = 32 * (t - b_rare - b_o4); cnt = cn.y - first;
            } else {
                fam = kFamEven; first = 32 * (t - b_rare - b_o4 - b_o3); cnt = cn.w - first;
            }
            if (lane < cnt) {
                unsigned int f;
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(f) : "r"(gemm_tab_list_slot(lists, fam, first + lane)));
                uint2 it;
                asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(it.x), "=r"(it.y) : "r"(items + 8u * f));
                const unsigned long long local = ((unsigned long long)(it.y & 0x1fffu) << 32 | it.x) >> 1;
                const int ci = (int)(it.y >> 13);
                f |= (it.x & 1u) << 16;  // the gain bit rides along
                unsigned int V[6];
                float scale;
                if (fam == kFamEven)
                    scale = tab_decode_even<false>(T, ci, local, V);
                else if (fam == kFamOdd3)
                    scale = tab_decode_odd3(T, ci, local, V);
                else if (fam == kFamOdd4)
                    scale = tab_decode_odd4(T, ci, local, V);
                else {
                    const TabRareBlock r = tab_decode_rare_call(T.base, lut_off, lut_on3, L, ci, local);
                    V[0] = r.v0; V[1] = r.v1; V[2] = r.v2; V[3] = r.v3; V[4] = r.v4; V[5] = r.v5;
                    scale = r.scale;
                }
                const int lr = (int)((f & 0xffffu) >> 2), kb = (int)(f & 3u);
                const float2 cg = C.cent[cur.useq & 1][lr];
                const __half2 s2 = __float2half2_rn(scale * ((f >> 16) ? cg.y : cg.x));
                // signed byte b -> f16: the byte, offset to 0..255, dropped into the mantissa of 1024 gives
                // 1152 + b exactly; subtract, then one rounding in the product with the scale
                const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0xE480u));  // -1152
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    unsigned int h[4];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const unsigned int u = V[2 * j + k] ^ 0x80808080u;
                        const unsigned int p01 = __byte_perm(u, 0x64646464u, 0x5140), p23 = __byte_perm(u, 0x64646464u, 0x5342);
                        const __half2 a = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&p01), bias), s2);
                        const __half2 b = __hmul2(__hadd2(*reinterpret_cast<const __half2*>(&p23), bias), s2);
                        h[2 * k] = *reinterpret_cast<const unsigned int*>(&a);
                        h[2 * k + 1] = *reinterpret_cast<const unsigned int*>(&b);
                    }
                    sts128(a_tile + swz_offset(lr, 3 * kb + j, kGPanelA), make_uint4(h[0], h[1], h[2], h[3]));
                }
            }
        }

        // ---- classify the next chunk while the other warps finish their batches ----
        const GemmTabIt& nxt = C.it[(q + 1) % 3];
        bool landed = true;
        if (nxt.valid) {
            landed = classify(nxt, q + 1);
        }

        // this thread's pieces of the B tile have landed; generic-proxy writes must be visible to the tensor core's
        // asynchronous reads
        asm volatile("cp.async.wait_all;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        ok = pipe_group_sync_and(half, landed);
        if (!ok) break;

        // ---- MMA: 3 panels x 2 K-steps of 16, accumulating in TMEM ----
        if (gt == 0) {
            if (cur.last) {  // read by warps 0-3 after the next barrier
                C.done_row0 = cur.row0;
                C.done_split = cur.split;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned int tmem = S.tmem_base + (unsigned int)half * kGTmemCols;
            // instruction descriptor: D = f32, A = B = f16, both K-major, N = n_pad, M = 128
            const unsigned int idesc = (1u << 4) | ((unsigned int)(ga.n_pad >> 3) << 17) | ((unsigned int)(kGM >> 4) << 24);
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                const unsigned long long da = umma_desc_k64_at(a_tile + p * kGPanelA), db = umma_desc_k64_at(b_tile + p * kGPanelB);
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const unsigned int accumulate = (cur.first == 0 || p > 0 || kk > 0) ? 1u : 0u;
                    // +32 bytes (two 16-byte units) per K-step inside a swizzled 64-byte row
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
                             pipe_smem_addr(&C.mbar_mma))
                         : "memory");
        }
        prev_last = cur.last != 0;
    }

    // ---- the half's last unit: wait for its MMAs, read the accumulators, store the partials ----
    if (ok && q > 0) {
        const bool done = gt != 0 || pipe_mbar_wait(pipe_smem_addr(&C.mbar_mma), (unsigned int)((q - 1) & 1));
        ok = pipe_group_sync_and(half, done);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) store_unit();
    }
    // the halves meet again: the table copy must not outlive the CTA, TMEM is freed once nobody reads it
    if (tid == 0) pipe_mbar_wait(pipe_smem_addr(&S.mbar_tab[1]));
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    const bool any_failed = __syncthreads_or(!ok);
    if (tid < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(S.tmem_base), "r"(kGTmemCols * kTGHalves) : "memory");
    if (tid == 0) {
        if (any_failed) atomicOr(err_flag, 2);
        if (S.error) atomicOr(err_flag, 1);
    }
}

// y[n, r] = f16( (sum_s ws[s, n, r]) * rscale[r] + tail[r, :] . x[n, 24 nb :] ), partials added in split order.
__global__ void gemm_reduce_kernel(MatrixView mv, const __half* __restrict__ x, const float* __restrict__ ws,
                                   __half* __restrict__ y, int batch, int n_pad, int splits) {
    llvq_dependent_enter();
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

// Shared-memory plan and the split of the column chunks into work units for a grid of `grid` CTAs (two halves
// each): the split count that minimises the chunks of the busiest half (plus a small charge per unit for its
// read-back), fewer splits on a tie.
inline GemmTabPlan gemm_tab_plan(const TabLayout& L, int d_out, int nb, int grid) {
    GemmTabPlan p{};
    unsigned int at = 0;
    p.blob = at;
    at += (L.total_bytes + 127u) & ~127u;
    p.items = at;
    at += kTGHalves * 2u * 8u * kGItems;
    p.lists = at;
    at += kTGHalves * 2u * 4u * kGItems;
    p.slab = at;
    at += kTGHalves * kGM * kGSlabLine;
    p.ctrl = at;
    at += (unsigned int)((sizeof(GemmTabShared) + kTGHalves * sizeof(GemmTabCtrl) + 15) & ~(size_t)15);
    p.tiles = at;
    at += kTGHalves * (3u * kGPanelA + 3u * kGPanelB) + 1024u;  // room to round the panels up to a 1024-byte boundary
    p.total = at;
    p.row_tiles = (d_out + kGM - 1) / kGM;
    const int chunks = (nb + kGKB - 1) / kGKB;
    const int streams = grid * kTGHalves;
    p.splits = 0;
    p.chunks_per_split = 1;
    double best = 0.0;
    for (int s = 1; s <= chunks; ++s) {
        const int cps = (chunks + s - 1) / s;
        const int real = (chunks + cps - 1) / cps;
        if (real != s) continue;
        const long long units = (long long)p.row_tiles * s;
        const long long waves = (units + streams - 1) / streams;
        const double cost = (double)waves * (cps + 0.5);
        if (p.splits == 0 || cost < best - 1e-9) {
            best = cost;
            p.splits = s;
            p.chunks_per_split = cps;
        }
    }
    p.units = p.row_tiles * p.splits;
    return p;
}

}  // namespace llvq
