// Persistent fused dequant-GEMV for sm_100a.
//
// One CTA of 1024 threads per SM owns a contiguous range of output rows and keeps
// the decoder tables (tab_tables.h, 106 KB) in shared memory. The CTA runs as
// kPipeGroups groups of warps, each with its own share of the rows, its own tile
// buffers and its own named barrier. A group's rows are cut into tiles of at most
// tile_max blocks (rows x a chunk of the columns: the whole row where its activation
// digits fit the digit buffer; as many blocks as the group's share of the remaining
// shared memory holds: about 2 400). A tile goes through three phases separated by
// the group's barrier:
//
//   classify   the tile's packed codes are already in shared memory (one bulk
//              asynchronous copy per contiguous range, cp.async.bulk completing on an
//              mbarrier, started while the previous tile was being decoded). Every
//              warp takes 32 blocks at a time: 48-bit record -> class -> family, an
//              8-byte item at the block's own slot, the slot appended to its family's
//              list (ballots + one shared-memory atomic per family and warp).
//   decode     a few warps first form this tile's row scales and tail-column products
//              (only the row sums read them) and stage the next tile's centroids and,
//              for rows cut into column chunks, its activation digits. Then all warps
//              draw batches of 32 same-family items, longest family first,
//              run that family's branch-free decoder (decode_tab.cuh) and dot the 24
//              signed bytes against the activation digits with dp4a; the scaled block
//              sum replaces the item.
//   row sums   one warp per row adds the block sums in a fixed order; the last column
//              chunk of a row applies the row scale and the tail product and stores y.
//
// The integer dot product: per 24-column block the activations are scaled by their
// largest magnitude to 16 bits (f16 activations) or 24 bits (f32 activations) and
// split into byte digits; sum_j v_j x_j is then exact in integers for the quantised
// x (relative error per term 2^-16 resp. 2^-24 of the block's largest activation),
// and independent of the order of evaluation.
//
// The kernel is launched with programmatic stream serialisation: it lets the next
// launch of the stream start at once, and itself waits for the previous launch only
// before it first touches the activation: table copies, tile layout, the first code
// slab and a prefetch of the first rows' data all come before that wait. The
// activation may also be formed in the staging step from the tensors an elementwise
// step would have read (PipeXOp: RMSNorm of residual + delta, or silu(gate) * up).
#pragma once
#include <cuda_fp16.h>

#include "decode_tab.cuh"
#include "kernels_generic.cuh"

namespace llvq {

constexpr int kPipeThreads = 1024;
constexpr int kPipeWarps = kPipeThreads / 32;
// The CTA runs as kPipeGroups independent groups of warps that share the decoder tables: each group owns a
// part of the CTA's rows, its own tile buffers and its own named barrier, so the groups drift out of phase
// and one group's decode phase fills the issue slots another leaves empty while it classifies, sums rows or
// waits at a barrier (what two CTAs per SM would do, if two copies of the tables fitted).
#ifndef LLVQ_PIPE_GROUPS
#define LLVQ_PIPE_GROUPS 2
#endif
constexpr int kPipeGroups = LLVQ_PIPE_GROUPS;
constexpr int kGroupThreads = kPipeThreads / kPipeGroups;
constexpr int kGroupWarps = kGroupThreads / 32;
constexpr int kDigitBytes = 24576;    // shared memory given to the activation digits
constexpr int kTileRowsMax = 128;     // rows per tile
constexpr int kStageWarps = 4 / kPipeGroups > 0 ? 4 / kPipeGroups : 1;  // warps of a group that stage the next tile's digits and row data
constexpr unsigned int kPipeSpinLimit = 1u << 22;
#ifndef LLVQ_CLS_GROUPS
#define LLVQ_CLS_GROUPS 2
#endif
constexpr int kClsGroups = LLVQ_CLS_GROUPS;  // groups of 32 blocks a warp classifies per iteration (independent look-up chains)

template <typename XT>
struct XDigits;
// Bytes per column in shared memory: an odd multiple of 16, so that the 16-byte loads of eight
// consecutive columns fall into eight different bank groups. The f16 layout keeps the column's
// scale in a separate float array (kScaleInline = false); the f32 layout has room for it.
template <>
struct XDigits<__half> {
    static constexpr int kDigits = 2, kColBytes = 48;
    static constexpr bool kScaleInline = false;
};
template <>
struct XDigits<float> {
    static constexpr int kDigits = 3, kColBytes = 80;
    static constexpr bool kScaleInline = true;
};

// Shared-memory plan of one launch (byte offsets from the start of dynamic shared memory).
struct PipePlan {
    unsigned int blob;        // decoder tables
    unsigned int xbuf;        // one or two digit buffers of cols_max columns (column bytes, then one float each)
    unsigned int ctrl;        // PipeCtrl
    unsigned int items;       // tile_max x 8
    unsigned int lists;       // 2 x tile_max x 2
    unsigned int slab;        // the packed codes of a tile
    unsigned int slab_bytes;
    unsigned int total;
    int tile_max;             // blocks per tile
    int cols_max, ncc;        // columns per chunk, column chunks (two digit buffers when ncc > 1)
    int rows_per_cta;
    int tcn;                  // columns of a full chunk
    int fit;                  // rows of a tile (as many as the tile memory holds, at most kTileRowsMax)
    unsigned int mdiv_full, mdiv_last;  // PipeTile::mdiv of a full chunk and of the last chunk
    int probe;                // attribution probes: bit 0 = leave the decoders out, bit 1 = leave the class search out
    unsigned long long* trace;  // per CTA kTraceEvents time stamps (ns), or null
};
constexpr int kTraceEvents = 64;

// One tile: rows [row0, row0 + rows) x column blocks [col0, col0 + cols) of the matrix.
struct PipeTile {
    int row0, rows, col0, cols, blocks;
    unsigned int mdiv;  // ceil(2^32 / cols): f / cols == umulhi(f, mdiv) for f < 2^16; 0 stands for cols == 1
    int first_chunk, last_chunk;
    int rg_first, same_cols;  // first row group; every tile of the CTA spans the same columns (one column chunk)
};

// The tiles of a CTA whose rows are [r0, r0 + nr) run row group by row group and, inside a row
// group, column chunk by column chunk. next() steps to the following tile without a division.
struct PipeGeom {
    int r0, nr;       // rows of this CTA
    int ncc, tcn;     // column chunks and their width (the last may be narrower)
    int nrg, rpt;     // row groups and their height (the last may be shorter)
    int nb;
    unsigned int mdiv_full, mdiv_last;
    int rg, cc;       // the tile next() returns
    __device__ __forceinline__ int tiles() const { return nrg * ncc; }
    __device__ __forceinline__ PipeTile next() {
        PipeTile t;
        t.row0 = r0 + rg * rpt;
        t.rows = min(rpt, r0 + nr - t.row0);
        t.col0 = cc * tcn;
        t.last_chunk = cc == ncc - 1;
        t.first_chunk = cc == 0;
        t.cols = t.last_chunk ? nb - t.col0 : tcn;
        t.mdiv = t.last_chunk ? mdiv_last : mdiv_full;
        t.blocks = t.rows * t.cols;
        t.rg_first = rg == 0;
        t.same_cols = ncc == 1;
        if (++cc == ncc) {
            cc = 0;
            ++rg;
        }
        return t;
    }
};

struct alignas(16) PipeShared {
    unsigned long long mbar[2];       // decoder tables: classification part, decode part
    int error;
    float xs_tail[32];
    float red[32];                    // per-warp sums of squares (activation produced in the kernel)
};
struct alignas(16) PipeCtrl {         // one per group
    unsigned long long slab_bar;      // code slab
    int ticket;
    int count[4];                     // items per family in the tile
    int2 list_lut[4];                 // per family: shared-window address of list entry 0, byte step to the next entry
    float rowacc[kTileRowsMax];
    float2 cent[2][kTileRowsMax];     // gain centroids of the rows of tile k at cent[k & 1]
    float2 rowfix[2][kTileRowsMax];   // (row scale, tail-column product) of the rows of tile k at rowfix[k & 1]
    PipeTile tile[2];                 // geometry of tile k at tile[k & 1], written by the group's thread 0 one tile ahead
    PipeGeom geo;                     // stepped by the group's thread 0 only
};

// Barrier over the kGroupThreads threads of group g (named barrier g + 1; barrier 0 stays the CTA's).
__device__ __forceinline__ void pipe_group_sync(int g) {
    asm volatile("bar.sync %0, %1;" ::"r"(g + 1), "n"(kGroupThreads) : "memory");
}
__device__ __forceinline__ bool pipe_group_sync_and(int g, bool pred) {
    unsigned int r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %2, 0;\n\t"
        "bar.red.and.pred q, %1, %3, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(g + 1), "r"((unsigned int)pred), "n"(kGroupThreads)
        : "memory");
    return r != 0;
}

__device__ __forceinline__ unsigned long long pipe_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ unsigned int pipe_smem_addr(const void* p) {
    return (unsigned int)__cvta_generic_to_shared(p);
}

// Bounded wait for the phase of the given parity of an mbarrier; false when the spin limit ran out.
__device__ __forceinline__ bool pipe_mbar_wait(unsigned int bar, unsigned int parity = 0) {
    unsigned int done = 0;
    for (unsigned int spin = 0; spin < kPipeSpinLimit && !done; ++spin) {
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

__device__ __forceinline__ void pipe_expect_tx(unsigned int bar, unsigned int bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pipe_bulk_copy(unsigned int dst, const void* src, unsigned int bytes, unsigned int bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ int dp4a_ss(unsigned int a, unsigned int b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(unsigned int a, unsigned int b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint4 lds128(unsigned int addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(unsigned int addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Where the f16 activation comes from. kXPlain: x itself. kXNorm: x is the residual stream and the activation is
// RMSNorm(x + delta) * w, computed by every CTA for itself with add_rmsnorm_kernel's arithmetic and order of
// operations (same bits); CTA 0 also writes x + delta to x_out, which must not alias x (the other CTAs
// still read x). kXSilu: x holds gate (n values) then up (n values) and the activation is silu(gate) * up,
// rounded to f16 as silu_mul_kernel stores it.
enum { kXPlain = 0, kXNorm = 1, kXSilu = 2 };
struct PipeXOp {
    const __half* delta;  // kXNorm: added to x first; may be null
    const __half* w;      // kXNorm: norm weights
    __half* x_out;        // kXNorm: the updated residual stream
    float eps;            // kXNorm
    int n;                // length of the activation
};

__device__ __forceinline__ float pipe_round_h(float v) { return __half2float(__float2half_rn(v)); }

// Element e of the activation (r: 1 / rms of the updated residual stream, kXNorm only).
template <int XOP>
__device__ __forceinline__ float pipe_x_elem(const __half* __restrict__ x, int e, const PipeXOp& xop, float r) {
    float v = __half2float(x[e]);
    if constexpr (XOP == kXNorm) {
        if (xop.delta) v = pipe_round_h(v + __half2float(xop.delta[e]));
        v = pipe_round_h(v * r * __half2float(xop.w[e]));
    } else if constexpr (XOP == kXSilu) {
        const float u = __half2float(x[xop.n + e]);
        v = pipe_round_h(v / (1.0f + __expf(-v)) * u);
    }
    return v;
}

__device__ __forceinline__ void pipe_load24_h(const __half* __restrict__ p, float (&v)[kDim]) {
#pragma unroll
    for (int q = 0; q < 3; ++q) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p + 8 * q);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f2 = __half22float2(h[k]);
            v[8 * q + 2 * k] = f2.x;
            v[8 * q + 2 * k + 1] = f2.y;
        }
    }
}

// Digits of one 24-column block of the activation, written to `dst` (shared-window address):
// kDigits planes of 24 bytes (most significant first: signed, then unsigned), then the float
// that turns the integer dot product back into the activation's units.
template <typename XT, int XOP>
__device__ __forceinline__ void pipe_prep_column(const XT* __restrict__ x, size_t e0, const PipeXOp& xop, float r, unsigned int dst,
                                                 unsigned int dst_scale) {
    const XT* xcol = x + e0;
    float v[kDim];
    __half2 vh[XOP == kXSilu ? kDim / 2 : 1];  // kXSilu keeps its values packed (they are f16 anyway): fewer live registers
    auto val = [&](int j) -> float {
        if constexpr (XOP == kXSilu)
            return (j & 1) ? __high2float(vh[j >> 1]) : __low2float(vh[j >> 1]);
        else
            return v[j];
    };
    if constexpr (sizeof(XT) == 2 && XOP == kXSilu) {
        // eight values at a time: gate and up of a piece are consumed before the next piece is loaded
        const __half* g = reinterpret_cast<const __half*>(xcol);
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            const uint4 graw = *reinterpret_cast<const uint4*>(g + 8 * q);
            const uint4 uraw = *reinterpret_cast<const uint4*>(g + xop.n + 8 * q);
            const __half2* gh = reinterpret_cast<const __half2*>(&graw);
            const __half2* uh = reinterpret_cast<const __half2*>(&uraw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 gf = __half22float2(gh[k]), uf = __half22float2(uh[k]);
                vh[4 * q + k] = __floats2half2_rn(gf.x / (1.0f + __expf(-gf.x)) * uf.x, gf.y / (1.0f + __expf(-gf.y)) * uf.y);
            }
        }
    } else if constexpr (sizeof(XT) == 2) {
        pipe_load24_h(reinterpret_cast<const __half*>(xcol), v);
        if constexpr (XOP == kXNorm) {
            float t[kDim];
            if (xop.delta) {
                pipe_load24_h(xop.delta + e0, t);
#pragma unroll
                for (int j = 0; j < kDim; ++j) v[j] = pipe_round_h(v[j] + t[j]);
            }
            pipe_load24_h(xop.w + e0, t);
#pragma unroll
            for (int j = 0; j < kDim; ++j) v[j] = pipe_round_h(v[j] * r * t[j]);
        }
    } else {
#pragma unroll
        for (int q = 0; q < 6; ++q) {
            const float4 f4 = *reinterpret_cast<const float4*>(xcol + 4 * q);
            v[4 * q] = f4.x;
            v[4 * q + 1] = f4.y;
            v[4 * q + 2] = f4.z;
            v[4 * q + 3] = f4.w;
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < kDim; ++j) amax = fmaxf(amax, fabsf(val(j)));
    constexpr int kDigits = XDigits<XT>::kDigits;
    constexpr float kFull = kDigits == 2 ? 32767.0f : 8388607.0f;
    // a zero block scales by 0; an infinite or NaN activation makes the block's factor NaN or inf,
    // which the product with the (zero) integer sum turns into NaN, as floating-point sums would
    const float s = amax > 0.0f ? kFull / amax : 0.0f;
    const float inv = amax / kFull;
    unsigned int w[kDigits][6];
#pragma unroll
    for (int d = 0; d < kDigits; ++d)
#pragma unroll
        for (int q = 0; q < 6; ++q) w[d][q] = 0;
#pragma unroll
    for (int j = 0; j < kDim; ++j) {
        // the product of the largest magnitude with s may round one past kFull: clamp, or the top
        // digit would change sign
        const int q = max(-(int)kFull, min((int)kFull, __float2int_rn(val(j) * s)));
#pragma unroll
        for (int d = 0; d < kDigits; ++d) {
            const unsigned int byte = ((unsigned int)q >> (8 * (kDigits - 1 - d))) & 0xffu;  // top digit keeps the sign
            w[d][j >> 2] |= byte << (8 * (j & 3));
        }
    }
    if constexpr (kDigits == 2) {
        sts128(dst, make_uint4(w[0][0], w[0][1], w[0][2], w[0][3]));
        sts128(dst + 16, make_uint4(w[0][4], w[0][5], w[1][0], w[1][1]));
        sts128(dst + 32, make_uint4(w[1][2], w[1][3], w[1][4], w[1][5]));
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst_scale), "r"(__float_as_uint(inv)) : "memory");
    } else {
        sts128(dst, make_uint4(w[0][0], w[0][1], w[0][2], w[0][3]));
        sts128(dst + 16, make_uint4(w[0][4], w[0][5], w[1][0], w[1][1]));
        sts128(dst + 32, make_uint4(w[1][2], w[1][3], w[1][4], w[1][5]));
        sts128(dst + 48, make_uint4(w[2][0], w[2][1], w[2][2], w[2][3]));
        sts128(dst + 64, make_uint4(w[2][4], w[2][5], __float_as_uint(inv), 0u));
    }
}

// sum_j V_j x_j for the digits at `xb`, in the activation's units.
template <typename XT>
__device__ __forceinline__ float pipe_dot(const unsigned int* V, unsigned int xb, unsigned int xscale) {
    if constexpr (XDigits<XT>::kDigits == 2) {
        const uint4 a = lds128(xb), b = lds128(xb + 16), c = lds128(xb + 32);
        float inv;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(inv) : "r"(xscale));
        int hi = dp4a_ss(V[0], a.x, 0);
        hi = dp4a_ss(V[1], a.y, hi);
        hi = dp4a_ss(V[2], a.z, hi);
        hi = dp4a_ss(V[3], a.w, hi);
        hi = dp4a_ss(V[4], b.x, hi);
        hi = dp4a_ss(V[5], b.y, hi);
        int lo = dp4a_su(V[0], b.z, 0);
        lo = dp4a_su(V[1], b.w, lo);
        lo = dp4a_su(V[2], c.x, lo);
        lo = dp4a_su(V[3], c.y, lo);
        lo = dp4a_su(V[4], c.z, lo);
        lo = dp4a_su(V[5], c.w, lo);
        return (float)(hi * 256 + lo) * inv;  // |hi * 256 + lo| < 2^24: exact
    } else {
        const uint4 a = lds128(xb), b = lds128(xb + 16), c = lds128(xb + 32), d = lds128(xb + 48), e = lds128(xb + 64);
        int d0 = dp4a_ss(V[0], a.x, 0);
        d0 = dp4a_ss(V[1], a.y, d0);
        d0 = dp4a_ss(V[2], a.z, d0);
        d0 = dp4a_ss(V[3], a.w, d0);
        d0 = dp4a_ss(V[4], b.x, d0);
        d0 = dp4a_ss(V[5], b.y, d0);
        int d1 = dp4a_su(V[0], b.z, 0);
        d1 = dp4a_su(V[1], b.w, d1);
        d1 = dp4a_su(V[2], c.x, d1);
        d1 = dp4a_su(V[3], c.y, d1);
        d1 = dp4a_su(V[4], c.z, d1);
        d1 = dp4a_su(V[5], c.w, d1);
        int d2 = dp4a_su(V[0], d.x, 0);
        d2 = dp4a_su(V[1], d.y, d2);
        d2 = dp4a_su(V[2], d.z, d2);
        d2 = dp4a_su(V[3], d.w, d2);
        d2 = dp4a_su(V[4], e.x, d2);
        d2 = dp4a_su(V[5], e.y, d2);
        // each partial sum is below 2^24 in magnitude, so its conversion is exact
        const float t = fmaf((float)d0, 65536.0f, fmaf((float)d1, 256.0f, (float)d2));
        return t * __uint_as_float(e.z);
    }
}

// Starts the bulk copies of a tile's packed codes into a slab (call with a whole warp). A tile that
// spans whole rows is one contiguous range of the code stream; a column chunk is one range per row.
// Ranges start and end on 16-byte boundaries of global memory (the stream carries 64 bytes of
// padding), so the records of row lr begin pipe_row_shift() bytes into that row's slab line.
struct PipeSlabGeom {
    unsigned int row_stride;  // bytes between the slab lines of consecutive rows
    bool contiguous;
};
__device__ __forceinline__ PipeSlabGeom pipe_slab_geom(const PipeTile& t, int nb) {
    PipeSlabGeom g;
    g.contiguous = t.cols == nb;
    g.row_stride = g.contiguous ? (unsigned int)t.cols * 6u : (((unsigned int)t.cols * 6u + 30u + 15u) & ~15u);
    return g;
}
__device__ __forceinline__ unsigned int pipe_row_shift(const unsigned char* codes, const PipeTile& t, int nb, bool contiguous,
                                                       unsigned int lr) {
    const size_t first = contiguous ? (size_t)t.row0 * nb * 6 : ((size_t)(t.row0 + lr) * nb + t.col0) * 6;
    return (unsigned int)((uintptr_t)(codes + first) & 15u);
}
__device__ __forceinline__ void pipe_issue_slab(const unsigned char* codes, const PipeTile& t, int nb, unsigned int slab,
                                                unsigned int bar, int lane) {
    const PipeSlabGeom g = pipe_slab_geom(t, nb);
    if (g.contiguous) {
        if (lane == 0) {
            const unsigned char* src = codes + (size_t)t.row0 * nb * 6;
            const unsigned int sh = (unsigned int)((uintptr_t)src & 15u);
            const unsigned int bytes = (sh + (unsigned int)t.blocks * 6u + 15u) & ~15u;
            pipe_expect_tx(bar, bytes);
            pipe_bulk_copy(slab, src - sh, bytes, bar);
        }
        return;
    }
    unsigned int total = 0;
    for (int lr = lane; lr < t.rows; lr += 32) {
        const unsigned char* src = codes + ((size_t)(t.row0 + lr) * nb + t.col0) * 6;
        const unsigned int sh = (unsigned int)((uintptr_t)src & 15u);
        total += (sh + (unsigned int)t.cols * 6u + 15u) & ~15u;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) pipe_expect_tx(bar, total);
    __syncwarp();
    for (int lr = lane; lr < t.rows; lr += 32) {
        const unsigned char* src = codes + ((size_t)(t.row0 + lr) * nb + t.col0) * 6;
        const unsigned int sh = (unsigned int)((uintptr_t)src & 15u);
        pipe_bulk_copy(slab + (unsigned int)lr * g.row_stride, src - sh, (sh + (unsigned int)t.cols * 6u + 15u) & ~15u, bar);
    }
}

// List slot of entry k of a family: the rare and four-kind lists share one array from both ends,
// the three-kind and even lists the other. (address of entry 0, byte step)
__device__ __forceinline__ int2 pipe_list_geom(unsigned int lists, int tile_max, unsigned int fam) {
    const unsigned int arr = lists + ((fam == kFamOdd3 || fam == kFamEven) ? (unsigned int)tile_max * 2u : 0u);
    const bool front = fam == kFamOdd4 || fam == kFamEven;
    return make_int2((int)(front ? arr : arr + 2u * (unsigned int)(tile_max - 1)), front ? 2 : -2);
}

// Staging of a tile's per-column and per-row data: activation digits of column c of the tile, and for row c
// of the tile its centroids and, for the last column chunk of a row, its row scale and tail-column product.
template <typename XT, int XOP>
__device__ __forceinline__ void pipe_stage_col(const XT* __restrict__ x, const PipeXOp& xop, float r, const PipeTile& t, unsigned int xbuf,
                                               unsigned int xscl, int c) {
    constexpr int kColBytes = XDigits<XT>::kColBytes;
    if (c < t.cols) pipe_prep_column<XT, XOP>(x, (size_t)(t.col0 + c) * kDim, xop, r, xbuf + c * kColBytes, xscl + 4u * c);
}
// PARTS: bit 0 = the centroids (the decode phase reads them), bit 1 = row scale and tail product (the row sums do).
template <int PARTS>
__device__ __forceinline__ void pipe_stage_row(const MatrixView& mv, const PipeTile& t, PipeCtrl& C, const float* xs_tail, int slot, int c) {
    if (c < t.rows) {
        const int r = t.row0 + c;
        if (PARTS & 1) C.cent[slot][c] = __ldg(mv.cent + r);
        if ((PARTS & 2) && t.last_chunk) {
            // tail columns in ascending order, one fused multiply-add each: what the reference's
            // tail_dot_h (llvq-cuda/kernels/matvec.cu:329-341) compiles to under NVRTC's default
            // --fmad=true
            const float rs = __ldg(mv.rscale + r);
            float tv = 0.0f;
            // eight loads in flight at a time: this runs beside the decode phase, where registers are scarcer
            // than time
#pragma unroll
            for (int k0 = 0; k0 < kDim - 1; k0 += 8) {
                float w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int k = k0 + j;
                    w[j] = k >= mv.tail_w ? 0.0f
                           : mv.tail_f16  ? __half2float(__ldg((const __half*)mv.tail + (size_t)r * mv.tail_w + k))
                                          : __ldg((const float*)mv.tail + (size_t)r * mv.tail_w + k);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (k0 + j < mv.tail_w) tv = fmaf(w[j], xs_tail[k0 + j], tv);
            }
            C.rowfix[slot][c] = make_float2(rs, tv);
        }
    }
}

// Before the kernel may read the activation it can already pull the constant row data of its first tile towards
// the SM: prefetches hold no register across the wait for the previous launch.
__device__ __forceinline__ void pipe_prefetch_row(const MatrixView& mv, const PipeTile& t, int c) {
    if (c < t.rows) {
        const int r = t.row0 + c;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(mv.cent + r));
        if (t.last_chunk) {
            asm volatile("prefetch.global.L2 [%0];" ::"l"(mv.rscale + r));
            if (mv.tail_w > 0) {
                const size_t row_bytes = (size_t)mv.tail_w * (mv.tail_f16 ? 2u : 4u);
                const char* p = (const char*)mv.tail + (size_t)r * row_bytes;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(p + row_bytes - 1));
            }
        }
    }
}

template <typename XT, typename YT, int XOP>
__global__ void __launch_bounds__(kPipeThreads, 1)
llvq_gemv_pipe_kernel(const unsigned char* __restrict__ blob_g, const OffEntry* __restrict__ lut_off,
                      const unsigned long long* __restrict__ lut_on3, TabLayout L, MatrixView mv,
                      const XT* __restrict__ x, YT* __restrict__ y, PipePlan plan, PipeXOp xop,
                      int* __restrict__ err_flag) {
    static_assert(XOP == kXPlain || sizeof(XT) == 2, "an activation produced in the kernel is f16");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const unsigned int sbase = pipe_smem_addr(smem_raw);
    constexpr int kColBytes = XDigits<XT>::kColBytes;
    const int tid = threadIdx.x;
    const int grp = tid / kGroupThreads;                      // this thread's group
    const int gt = tid - grp * kGroupThreads, lane = gt & 31, warp = gt >> 5;  // position inside the group
    PipeShared& S = *reinterpret_cast<PipeShared*>(smem_raw + plan.ctrl);
    PipeCtrl& C = reinterpret_cast<PipeCtrl*>(smem_raw + plan.ctrl + sizeof(PipeShared))[grp];
    const int tile_max = plan.tile_max;

    TabView T;
    T.base = sbase + plan.blob;
    T.lut_off = lut_off;
    T.lut_on3 = lut_on3;
    T.L = L;
    // time stamps of thread 0 (group 0): entry, tables landed, then the end of every phase
    unsigned long long* trace = plan.trace ? plan.trace + (size_t)blockIdx.x * kTraceEvents : nullptr;
    int trace_n = 0;
    auto stamp = [&]() {
        if (trace && tid == 0 && trace_n < kTraceEvents) trace[trace_n] = pipe_now_ns();
        ++trace_n;
    };
    stamp();
    // The decoder tables start travelling before anything else is computed: the thread that initialises their
    // mbarriers also issues the copies (what classification reads first), the others meet them at the first
    // CTA barrier. The tables are constant, so this needs no ordering against the previous launch of the stream.
    if (tid == 0) {
        S.error = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pipe_smem_addr(&S.mbar[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pipe_smem_addr(&S.mbar[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pipe_expect_tx(pipe_smem_addr(&S.mbar[0]), L.classify_bytes);
        pipe_bulk_copy(T.base, blob_g, L.classify_bytes, pipe_smem_addr(&S.mbar[0]));
        pipe_expect_tx(pipe_smem_addr(&S.mbar[1]), L.total_bytes - L.classify_bytes);
        pipe_bulk_copy(T.base + L.classify_bytes, blob_g + L.classify_bytes, L.total_bytes - L.classify_bytes,
                       pipe_smem_addr(&S.mbar[1]));
    }

    // ---- rows of this CTA, of this group, and their tiling ----
    const int cta_r0 = blockIdx.x * plan.rows_per_cta;
    const int cta_nr = max(0, min(plan.rows_per_cta, mv.d_out - cta_r0));
    const int rpg = (cta_nr + kPipeGroups - 1) / kPipeGroups;
    const int grp_r0 = cta_r0 + grp * rpg;
    const int grp_nr = max(0, min(rpg, cta_r0 + cta_nr - grp_r0));
    const int ncc = plan.ncc;
    const int tcn = plan.tcn;
    const int fit = plan.fit;
    const int nrg = (grp_nr + fit - 1) / fit;
    const int nt = grp_nr > 0 ? nrg * ncc : 0;
    // activation digits: buffers of cols_max columns (digits, then one float per column). A matrix with a single
    // column chunk stages its digits once for the whole CTA; otherwise every group alternates between two
    // buffers of its own.
    const unsigned int xdig_bytes = (unsigned int)plan.cols_max * kColBytes;
    const unsigned int xbuf_bytes = ((unsigned int)plan.cols_max * (kColBytes + 4) + 15u) & ~15u;  // 16-byte loads
    const unsigned int items = sbase + plan.items + (unsigned int)grp * (unsigned int)tile_max * 8u,
                       lists = sbase + plan.lists + (unsigned int)grp * (unsigned int)tile_max * 4u,
                       xbuf = sbase + plan.xbuf + (ncc > 1 ? (unsigned int)grp * 2u * xbuf_bytes : 0u), xscl = xbuf + xdig_bytes,
                       slab = sbase + plan.slab + (unsigned int)grp * plan.slab_bytes;
    const unsigned int bar_slab = pipe_smem_addr(&C.slab_bar);
    bool failed = false;

    // ---- prologue: the first tile's codes start travelling, then the activation is staged ----
    // Programmatic dependent launch: the next launch of the stream may take this SM as soon as this CTA
    // leaves it, and this launch comes as far as griddepcontrol.wait below while the previous one is still running.
    // Nothing before that wait reads what a previous kernel writes (tables and codes are constant).
    asm volatile("griddepcontrol.launch_dependents;");
    if (warp == 1) {
        // the group's second warp lays out the tiles and starts the first code slab on its own (thread 0 of the
        // CTA, in the first warp, is busy issuing the table copies)
        if (lane < 4) C.list_lut[lane] = pipe_list_geom(lists, tile_max, (unsigned int)lane);
        if (lane == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_slab));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            PipeGeom geo;
            geo.nb = mv.nb;
            geo.r0 = grp_r0;
            geo.nr = grp_nr;
            geo.ncc = ncc;
            geo.tcn = tcn;
            geo.nrg = nrg;
            geo.rpt = (grp_nr + nrg - 1) / max(nrg, 1);
            geo.mdiv_full = plan.mdiv_full;
            geo.mdiv_last = plan.mdiv_last;
            geo.rg = 0;
            geo.cc = 0;
            if (nt > 0) C.tile[0] = geo.next();
            C.geo = geo;
        }
        __syncwarp();
        if (nt > 0) {
            const PipeTile t0 = C.tile[0];
            pipe_issue_slab(mv.codes, t0, mv.nb, slab, bar_slab, lane);
        }
    }
    __syncthreads();  // the tile geometry (and S.error = 0) is visible to every warp
    // the staging warps pull the first tile's row data (constant) towards the SM before the wait
    const bool stager = warp >= kGroupWarps - kStageWarps;
    if (stager && nt > 0) {
        const PipeTile t0 = C.tile[0];
        for (int c = 32 * (kGroupWarps - 1 - warp) + lane; c < t0.rows; c += 32 * kStageWarps) pipe_prefetch_row(mv, t0, c);
    }
    // the activation may be the previous kernel's output, and y may be its input: from here on the previous
    // launch of the stream has completed and its writes are visible (no-op for an ordinary launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float xr = 0.0f;  // kXNorm: 1 / rms of the updated residual stream
    if constexpr (XOP == kXNorm) {
        // add_rmsnorm_kernel's first pass with its partition (thread t: pairs t, t + 1024, ...), its order of
        // additions and its warp and CTA reductions, so that every CTA arrives at the bits that kernel produces
        const __half2* x2 = reinterpret_cast<const __half2*>(x);
        const __half2* d2 = reinterpret_cast<const __half2*>(xop.delta);
        const int pairs = xop.n >> 1;
        float ss = 0.0f;
        for (int i = tid; i < pairs; i += kPipeThreads) {
            __half2 h = x2[i];
            if (d2) {
                const float2 a = __half22float2(h), d = __half22float2(d2[i]);
                h = __floats2half2_rn(a.x + d.x, a.y + d.y);
            }
            if (blockIdx.x == 0) reinterpret_cast<__half2*>(xop.x_out)[i] = h;
            const float2 v = __half22float2(h);
            ss += v.x * v.x + v.y * v.y;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((tid & 31) == 0) S.red[tid >> 5] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int k = 0; k < 32; ++k) tot += S.red[k];
        xr = rsqrtf(tot / (float)xop.n + xop.eps);
    }
    // the tail activations: every staging warp writes the same values and reads them back after its own
    // warp barrier (no CTA barrier stands between here and the staging below)
    if (warp >= kGroupWarps - kStageWarps) {
        float tv = 0.0f;
        if (lane < mv.tail_w) {
            if constexpr (XOP == kXPlain)
                tv = to_f32<XT>(x[mv.nb * kDim + lane]);
            else
                tv = pipe_x_elem<XOP>(reinterpret_cast<const __half*>(x), mv.nb * kDim + lane, xop, xr);
        }
        S.xs_tail[lane] = tv;
        __syncwarp();
    }
    // the first tile's digits and row data are staged while the tables travel
    if (ncc == 1) {
        // one column chunk: the digits of the whole row, once, by every thread of the CTA (nothing else has
        // work before the tables land)
        PipeTile all;
        all.col0 = 0;
        all.cols = mv.nb;
        for (int c = tid; c < mv.nb; c += kPipeThreads) pipe_stage_col<XT, XOP>(x, xop, xr, all, xbuf, xscl, c);
    }
    if (stager && nt > 0) {
        const PipeTile t0 = C.tile[0];
        for (int c = 32 * (kGroupWarps - 1 - warp) + lane; c < max(t0.cols, t0.rows); c += 32 * kStageWarps) {
            if (ncc > 1) pipe_stage_col<XT, XOP>(x, xop, xr, t0, xbuf, xscl, c);
            pipe_stage_row<1>(mv, t0, C, S.xs_tail, 0, c);  // row scale and tail product follow under the decode phase
        }
    }
    {
        const bool landed = tid != 0 || pipe_mbar_wait(pipe_smem_addr(&S.mbar[0]));
        if (!__syncthreads_and(landed)) failed = true;  // uniform over the CTA
    }
    stamp();

    for (int i = 0; i < nt && !failed; ++i) {
        const PipeTile& tc = C.tile[i & 1];
        const bool has_next = i + 1 < nt;
        // ================= phase 1: digits, row data, classification =================
        if (gt == 0) {
            C.ticket = 0;
#pragma unroll
            for (int k = 0; k < 4; ++k) C.count[k] = 0;
            if (has_next) {  // geometry of the next tile (its codes are fetched during phase 2)
                PipeGeom geo = C.geo;
                C.tile[(i + 1) & 1] = geo.next();
                C.geo = geo;
            }
        }
        {
            // the tile's codes: started a phase ago (or in the prologue)
            const bool landed = gt != 0 || pipe_mbar_wait(bar_slab, (unsigned int)i & 1u);
            if (!pipe_group_sync_and(grp, landed)) {
                failed = true;
                break;
            }
        }
        {
            // ---- classification: warp w takes blocks 32 w .. 32 w + 31, then 32 (w + warps) .., ... ----
            // item: 2 * (rank inside the class) + gain (45 bits: the largest class holds 8.83e12 points), class << 45
            const PipeSlabGeom sg = pipe_slab_geom(tc, mv.nb);
            const unsigned int blocks = (unsigned int)tc.blocks, cols = (unsigned int)tc.cols, mdiv = tc.mdiv;
            // byte offset of row lr's first record inside its slab line: (a0 + lr * pitch) & 15 for a column chunk
            const unsigned int a0 = pipe_row_shift(mv.codes, tc, mv.nb, sg.contiguous, 0);
            const unsigned int pitch = ((unsigned int)mv.nb * 6u) & 15u;
            const unsigned int probe = (unsigned int)plan.probe;
            // two groups of 32 blocks per iteration: their table look-ups are independent, so the scheduler can
            // overlap the shared-memory latency of one with the arithmetic of the other
#pragma unroll 1
            for (unsigned int f0 = 32u * warp; f0 < blocks; f0 += 32u * kClsGroups * kGroupWarps) {
                unsigned int fams[kClsGroups], fs[kClsGroups];
                uint2 its[kClsGroups];
#pragma unroll
                for (int u = 0; u < kClsGroups; ++u) {
                    const unsigned int f = f0 + 32u * kGroupWarps * u + lane;
                    fs[u] = f;
                    fams[u] = 4u;  // 4: nothing to decode
                    its[u] = make_uint2(0u, 0u);  // origin or refused index: a block sum of zero
                    if (f < blocks) {
                        unsigned int ca;  // shared-window address of the record, 2-byte aligned
                        if (sg.contiguous) {
                            ca = slab + a0 + 6u * f;
                        } else {
                            const unsigned int lr = mdiv ? __umulhi(f, mdiv) : f, lc = f - lr * cols;
                            ca = slab + lr * sg.row_stride + ((a0 + lr * pitch) & 15u) + 6u * lc;
                        }
                        // the slab is not written during this phase: plain (movable) loads
                        unsigned int h0, h1, h2;
                        asm("ld.shared.u16 %0, [%1];" : "=r"(h0) : "r"(ca));
                        asm("ld.shared.u16 %0, [%1];" : "=r"(h1) : "r"(ca + 2u));
                        asm("ld.shared.u16 %0, [%1];" : "=r"(h2) : "r"(ca + 4u));
                        const unsigned int hi = __byte_perm(h0, 0, 0x4401);   // bytes 0,1 -> big-endian 16 bits
                        const unsigned int lo = __byte_perm(h1, h2, 0x0145);  // bytes 2..5 -> big-endian 32 bits
                        if (probe & 2u) {
                            // stream probe: the codes are read, nothing is searched or decoded
                            its[u].y = lo & hi & 0x80000000u & (lo >> 1);  // keeps the loads alive
                        } else {
                            const TabClassified c = tab_classify(T, ((unsigned long long)hi << 32) | lo);
                            if (c.fam >= 0) {
                                fams[u] = (unsigned int)c.fam;
                                its[u].x = (unsigned int)c.local2;
                                its[u].y = (unsigned int)(c.local2 >> 32) | (unsigned int)c.ci << 13;
                            } else if (c.fam == -2) {
                                S.error = 1;
                            }
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kClsGroups; ++u) {
                    const unsigned int f = fs[u], fam = fams[u];
                    if (f < blocks)
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(items + 8u * f), "r"(its[u].x), "r"(its[u].y) : "memory");
                    // lanes of the same family find each other; the lowest one reserves their list slots
                    const unsigned int v0 = __ballot_sync(0xffffffffu, fam == 0u), v1 = __ballot_sync(0xffffffffu, fam == 1u),
                                       v2 = __ballot_sync(0xffffffffu, fam == 2u), v3 = __ballot_sync(0xffffffffu, fam == 3u);
                    const unsigned int peers = fam == 0u ? v0 : fam == 1u ? v1 : fam == 2u ? v2 : fam == 3u ? v3 : 1u << lane;
                    const int leader = __ffs(peers) - 1;
                    int slot = 0;
                    if (fam < 4u && lane == leader) slot = atomicAdd(&C.count[fam], __popc(peers));
                    slot = __shfl_sync(0xffffffffu, slot, leader);
                    if (fam < 4u) {
                        const int2 lg = C.list_lut[fam];
                        const unsigned int a = (unsigned int)(lg.x + lg.y * (slot + __popc(peers & ((1u << lane) - 1u))));
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"((unsigned short)f) : "memory");
                    }
                }
            }
        }
        {
            // the decode tables must have landed before the group's first decode phase
            const bool landed = i > 0 || gt != 0 || pipe_mbar_wait(pipe_smem_addr(&S.mbar[1]));
            if (!pipe_group_sync_and(grp, landed)) {
                failed = true;
                break;
            }
        }
        stamp();

        // ================= phase 2: decode + dot =================
        // the slab is free now: the next tile's codes travel while this one is decoded
        if (warp == 0 && has_next) {
            const PipeTile tn = C.tile[(i + 1) & 1];
            pipe_issue_slab(mv.codes, tn, mv.nb, slab, bar_slab, lane);
        }
        // ... and a few warps stage row data before they join the decoding: this tile's row scales and tail
        // products, which only the row sums below need, then the next tile's digits and centroids
        if (warp >= kGroupWarps - kStageWarps)
            for (int c = 32 * (kGroupWarps - 1 - warp) + lane; c < tc.rows; c += 32 * kStageWarps)
                pipe_stage_row<2>(mv, tc, C, S.xs_tail, i & 1, c);
        if (has_next && warp >= kGroupWarps - kStageWarps) {
            const PipeTile tn = C.tile[(i + 1) & 1];
            const unsigned int xo = ncc > 1 ? (unsigned int)((i + 1) & 1) * xbuf_bytes : 0u;
            for (int c = 32 * (kGroupWarps - 1 - warp) + lane; c < max(tn.cols, tn.rows); c += 32 * kStageWarps) {
                if (ncc > 1) pipe_stage_col<XT, XOP>(x, xop, xr, tn, xbuf + xo, xscl + xo, c);
                pipe_stage_row<1>(mv, tn, C, S.xs_tail, (i + 1) & 1, c);
            }
        }
        {
            const int n_rare = C.count[kFamRare], n_o4 = C.count[kFamOdd4], n_o3 = C.count[kFamOdd3], n_ev = C.count[kFamEven];
            const int b_rare = (n_rare + 31) >> 5, b_o4 = (n_o4 + 31) >> 5, b_o3 = (n_o3 + 31) >> 5, b_ev = (n_ev + 31) >> 5;
            const int n_dec = (plan.probe & 4) ? 0 : b_rare + b_o4 + b_o3 + b_ev;  // probe bit 2: no batches at all
            const unsigned int cols = (unsigned int)tc.cols, mdiv = tc.mdiv;
            const unsigned int xcur = xbuf + (ncc > 1 ? (unsigned int)(i & 1) * xbuf_bytes : 0u);
            for (;;) {
                int t = 0;
                if (lane == 0) t = atomicAdd(&C.ticket, 1);
                t = __shfl_sync(0xffffffffu, t, 0);
                if (t >= n_dec) break;
                // one family per batch, longest families first
                unsigned int fam;
                int first, count;
                if (t < b_rare) {
                    fam = kFamRare; first = 32 * t; count = n_rare - first;
                } else if (t < b_rare + b_o4) {
                    fam = kFamOdd4; first = 32 * (t - b_rare); count = n_o4 - first;
                } else if (t < b_rare + b_o4 + b_o3) {
                    fam = kFamOdd3; first = 32 * (t - b_rare - b_o4); count = n_o3 - first;
                } else {
                    fam = kFamEven; first = 32 * (t - b_rare - b_o4 - b_o3); count = n_ev - first;
                }
                if (lane < count) {  // the last batch of a family may be ragged
                    unsigned int f;
                    const int2 lg = C.list_lut[fam];
                    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(f) : "r"((unsigned int)(lg.x + lg.y * (first + lane))));
                    uint2 it;
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(it.x), "=r"(it.y) : "r"(items + 8u * f));
                    const unsigned long long local = ((unsigned long long)(it.y & 0x1fffu) << 32 | it.x) >> 1;
                    const int ci = (int)(it.y >> 13);
                    const unsigned int gain = it.x & 1u;
                    const unsigned int lr = mdiv ? __umulhi(f, mdiv) : f, lc = f - lr * cols;
                    unsigned int V[6];
                    float scale;
                    if (plan.probe & 1) {
                        // floor probe: everything but the decoders (an item still flows through the lists)
                        scale = 0.0f;
#pragma unroll
                        for (int k = 0; k < 6; ++k) V[k] = it.x;
                    } else if (fam == kFamEven)
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
                    const float dot = pipe_dot<XT>(V, xcur + lc * kColBytes, xcur + xdig_bytes + 4u * lc);
                    const float2 cg = C.cent[i & 1][lr];
                    const float part = dot * (scale * (gain ? cg.y : cg.x));
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(items + 8u * f), "r"(__float_as_uint(part)) : "memory");
                }
            }
        }
        pipe_group_sync(grp);
        stamp();

        // ================= phase 3: fixed-order row sums =================
        for (int lr = warp; lr < tc.rows; lr += kGroupWarps) {
            float s = 0.0f;
            // four loads in flight, added in column order (the order of a one-by-one loop)
            for (int c = lane; c < tc.cols; c += 128) {
                unsigned int u[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    u[k] = 0u;  // an absent column adds +0.0f, which changes nothing: s starts at +0.0f and so is never -0.0f
                    if (c + 32 * k < tc.cols)
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(u[k]) : "r"(items + 8u * (unsigned int)(lr * tc.cols + c + 32 * k)));
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) s += __uint_as_float(u[k]);
            }
            s = warp_sum(s);
            if (lane == 0) {
                const float acc = tc.first_chunk ? s : C.rowacc[lr] + s;
                if (tc.last_chunk) {
                    // y = acc * rscale + tail, contracted as the reference's epilogue is
                    // (llvq-llm/kernels/tv_planes_h.cu:67-71)
                    const float2 fx = C.rowfix[i & 1][lr];
                    store_y<YT>(y, tc.row0 + lr, fmaf(acc, fx.x, fx.y));
                } else {
                    C.rowacc[lr] = acc;
                }
            }
        }
        pipe_group_sync(grp);
        stamp();
    }
    // the groups meet again: neither table copy may outlive the CTA, and the error words are complete
    if (tid == 0) pipe_mbar_wait(pipe_smem_addr(&S.mbar[1]));
    const bool any_failed = __syncthreads_or(failed);
    if (tid == 0) {
        if (any_failed) atomicOr(err_flag, 2);
        if (S.error) atomicOr(err_flag, 1);
    }
}

// Shared-memory plan for a matrix of nb column blocks on a device with `smem_optin` bytes per CTA;
// tile_max = 0 when the tables leave no room for a tile.
template <typename XT>
inline PipePlan pipe_plan(const TabLayout& L, int smem_optin, int d_out, int nb, int sm_count) {
    PipePlan p{};
    constexpr int kPerCol = XDigits<XT>::kColBytes + 4;
    // the whole row in one chunk (digits shared by the groups) when its digits fit, else the fewest equal
    // chunks for which two buffers per group fit
    p.ncc = 1;
    if (nb * kPerCol > kDigitBytes)
        while (2 * kPipeGroups * ((nb + p.ncc - 1) / p.ncc) * kPerCol > kDigitBytes) ++p.ncc;
    p.cols_max = nb > 0 ? (nb + p.ncc - 1) / p.ncc : 1;
    unsigned int at = 0;
    p.blob = at;
    at += (L.total_bytes + 127u) & ~127u;
    p.xbuf = at;
    at += (unsigned int)(p.ncc > 1 ? 2 * kPipeGroups : 1) * (((unsigned int)p.cols_max * kPerCol + 15u) & ~15u);
    p.ctrl = at;
    at += (unsigned int)((sizeof(PipeShared) + kPipeGroups * sizeof(PipeCtrl) + 15) & ~(size_t)15);
    // per block of a group's tile: 8 bytes of item, 2 x 2 bytes of lists, 7 bytes of code slab (6 bytes of
    // record + the alignment slack of a column chunk's rows: at most 30 bytes per 65 blocks)
    const int room = smem_optin - (int)at - 128 - kPipeGroups * 96;
    int tile_max = room / (19 * kPipeGroups);
    tile_max &= ~31;
    if (tile_max > 65536 - 32) tile_max = 65536 - 32;  // list entries are 16 bits
    if (tile_max < p.cols_max) tile_max = 0;           // not even one row fits
    p.tile_max = tile_max > 0 ? tile_max : 0;
    p.items = at;
    at += (unsigned int)kPipeGroups * (unsigned int)p.tile_max * 8u;
    p.lists = at;
    at += (unsigned int)kPipeGroups * (unsigned int)p.tile_max * 4u;
    p.slab_bytes = ((unsigned int)p.tile_max * 7u + 64u + 15u) & ~15u;
    p.slab = at;
    at += (unsigned int)kPipeGroups * p.slab_bytes;
    p.total = at;
    p.rows_per_cta = (d_out + sm_count - 1) / sm_count;
    p.tcn = nb > 0 ? (nb + p.ncc - 1) / p.ncc : 1;
    auto reciprocal = [](int cols) { return cols > 1 ? (unsigned int)((0x100000000ull + cols - 1) / cols) : 0u; };
    p.fit = p.tile_max / p.tcn < 1 ? 1 : p.tile_max / p.tcn > kTileRowsMax ? kTileRowsMax : p.tile_max / p.tcn;
    p.mdiv_full = reciprocal(p.tcn);
    p.mdiv_last = reciprocal(nb - (p.ncc - 1) * p.tcn);
    p.probe = 0;
    p.trace = nullptr;
    return p;
}

// Integer dump of the decoders the fused kernels run: one thread per block, tables in shared memory,
// classification and family decoders exactly as in llvq_gemv_pipe_kernel. Writes 24 int8 per block,
// the shell (0 for the origin, 255 for a refused index) and the gain bit. The pattern is the
// reference's decode_probe (llvq-cuda/kernels/preflight.cu:39-60).
constexpr int kProbeThreads = 256;
__global__ void __launch_bounds__(kProbeThreads)
llvq_decode_tab_kernel(const unsigned char* __restrict__ blob_g, const OffEntry* __restrict__ lut_off,
                       const unsigned long long* __restrict__ lut_on3, TabLayout L, const unsigned char* __restrict__ codes, size_t n, signed char* __restrict__ points,
                       unsigned char* __restrict__ shell, unsigned char* __restrict__ gain) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    for (unsigned int o = threadIdx.x * 16u; o < L.total_bytes; o += kProbeThreads * 16u)
        *reinterpret_cast<uint4*>(smem_raw + o) = __ldg(reinterpret_cast<const uint4*>(blob_g + o));
    __syncthreads();
    TabView T;
    T.base = pipe_smem_addr(smem_raw);
    T.lut_off = lut_off;
    T.lut_on3 = lut_on3;
    T.L = L;
    for (size_t b = (size_t)blockIdx.x * kProbeThreads + threadIdx.x; b < n; b += (size_t)gridDim.x * kProbeThreads) {
        const unsigned long long v = load_code48(codes, b);
        unsigned int V[6];
        float scale;
        const TabClassified c = tab_classify(T, v);
        const unsigned long long local = c.local2 >> 1;
        unsigned int m = c.fam == -1 ? 0u : 255u;
        if (c.fam < 0) {
#pragma unroll
            for (int k = 0; k < 6; ++k) V[k] = 0u;
        } else {
            m = tab_ld32(T, L.cls + kClsStride * (unsigned int)c.ci + 56u);
            if (c.fam == (int)kFamEven)
                scale = tab_decode_even<false>(T, c.ci, local, V);
            else if (c.fam == (int)kFamOdd3)
                scale = tab_decode_odd3(T, c.ci, local, V);
            else if (c.fam == (int)kFamOdd4)
                scale = tab_decode_odd4(T, c.ci, local, V);
            else
                scale = tab_decode_rare(T, c.ci, local, V);
        }
        (void)scale;
        // 24 bytes per block: 8-byte aligned
        uint2* out = reinterpret_cast<uint2*>(points + b * kDim);
        out[0] = make_uint2(V[0], V[1]);
        out[1] = make_uint2(V[2], V[3]);
        out[2] = make_uint2(V[4], V[5]);
        shell[b] = (unsigned char)m;
        if (gain) gain[b] = (unsigned char)(v & 1ull);
    }
}

}  // namespace llvq
