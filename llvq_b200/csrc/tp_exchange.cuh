// All-gather of small row shards between the GPUs of one node through peer memory, for the
// tensor-parallel token step (the reference is single-GPU; this layer is new). The gathers of a
// decode step move 10-34 KB and are latency-bound, so the exchange is one small kernel per gather:
//
//   every rank owns a region = [flags | gather buffers], mapped into its peers (CUDA IPC);
//   warp p of the kernel copies this rank's shard into peer p's gather buffer at this rank's
//   offset with ordinary 16-byte peer stores, fences, and releases flag[site][rank] = seq on p;
//   then it waits until peer p's flag in the LOCAL region reaches seq: p's shard has landed here.
//
// `seq` counts the exchanges of this rank (device memory, so a captured graph replays); all ranks
// run the same sequence of exchanges, so equal counts name the same exchange. A site's buffer is
// written again only four exchanges later, after every rank has consumed it (each later exchange
// needed this rank's flag, which it sets after its consumers in stream order). No TMA, no multicast,
// no remote loads: plain stores to peers, polling on local memory only.
//
// Every wait is bounded: after `spin_limit` polls the warp records bit 2 of the error word and goes
// on, so the kernel always returns and the host reads the failure.
//
// One launch can carry several ranks (one CTA each): on a single GPU the ranks of a test are run
// as one cooperative launch over all ranks' regions, never as separate launches that wait on one
// another.
#pragma once
#include <cstdint>

#include "portable.h"

namespace llvq {

constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxSites = 16;
constexpr int kTpFlagBytes = kTpMaxSites * kTpMaxWorld * 4;  // flags[site][source rank], u32

struct TpRank {
    unsigned char* region[kTpMaxWorld];  // base of every rank's region as mapped here (own region included)
    unsigned int* seq;                   // exchanges done by this rank (local device memory)
    int* err;                            // sticky error word (bit 2: a peer's flag did not arrive)
    int rank, world;
    unsigned int spin_limit;
};

struct TpCall {
    TpRank r;
    const unsigned char* src;  // this rank's shard (local memory)
    unsigned int shard_bytes;
    unsigned int buf_offset;   // byte offset of the site's gather buffer inside a region
    int site;
};

struct TpCalls {
    TpCall c[kTpMaxWorld];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// grid = ranks carried by this launch (1 in production), block = 32 * kTpMaxWorld threads.
__global__ void __launch_bounds__(32 * kTpMaxWorld)
tp_exchange_kernel(TpCalls calls) {
    // launched as a programmatic dependent in production: the consumer of the gathered buffer may load its tables
    // while this kernel waits for the peers; nothing here runs before the kernels ahead in the stream are complete
    llvq_dependent_enter();
    const TpCall& c = calls.c[blockIdx.x];
    const int lane = threadIdx.x & 31, p = threadIdx.x >> 5;
    const unsigned int seq = *reinterpret_cast<volatile unsigned int*>(c.r.seq) + 1u;
    if (p < c.r.world) {
        unsigned char* dst = c.r.region[p] + c.buf_offset + (size_t)c.r.rank * c.shard_bytes;
        if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(c.src) | c.shard_bytes) & 15u) == 0) {
            const uint4* s4 = reinterpret_cast<const uint4*>(c.src);
            uint4* d4 = reinterpret_cast<uint4*>(dst);
            for (unsigned int i = lane; i < c.shard_bytes / 16; i += 32) d4[i] = s4[i];
        } else {
            for (unsigned int i = lane; i < c.shard_bytes; i += 32) dst[i] = c.src[i];
        }
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
            unsigned int* theirs = reinterpret_cast<unsigned int*>(c.r.region[p]) + c.site * kTpMaxWorld + c.r.rank;
            st_release_sys(theirs, seq);
            const unsigned int* mine = reinterpret_cast<const unsigned int*>(c.r.region[c.r.rank]) + c.site * kTpMaxWorld + p;
            unsigned int polls = 0;
            while ((int)(ld_acquire_sys(mine) - seq) < 0) {
                if (++polls >= c.r.spin_limit) {
                    atomicOr(c.r.err, 4);
                    break;
                }
                __nanosleep(100);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) *c.r.seq = seq;
}

}  // namespace llvq
