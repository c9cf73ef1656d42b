// Host launcher around the reference's own serving kernel, for the benchmark's reference arm and a parity test
// (test infrastructure: nothing of the library links or loads this).
//
// The reference serves a projection from its Planes14 layout with `tv_planes_h`
// (llvq-llm/kernels/tv_planes_h.cu:38-72 over llvq-cuda/kernels/llvq_planes.cuh, planes.cu, matvec.cu,
// llvq_slot.cuh) and compiles that text at run time with NVRTC, one concatenated translation unit with TILE_BLOCKS
// defined by the host (llvq-llm/src/fused_cuda.rs). This file is that translation unit for nvcc: it includes
// the kernel sources, unmodified, from a checkout of the reference (-I <checkout>) in the order the reference
// concatenates them, and adds the launch the reference's Rust host makes (one warp per row, 8 rows per 256-thread
// block, TILE_BLOCKS * 24 floats of dynamic shared memory; launch_planes_h, llvq-llm/src/fused_cuda.rs).
// `make -C oracle ref` builds it into oracle/_ref/libref_planes.so.
#include <cuda_runtime.h>

#define TILE_BLOCKS 128u
#include "llvq-cuda/kernels/llvq_slot.cuh"
#include "llvq-cuda/kernels/matvec.cu"
#include "llvq-cuda/kernels/llvq_planes.cuh"
#include "llvq-cuda/kernels/planes.cu"
#include "llvq-llm/kernels/tv_planes_h.cu"

extern "C" {

// sizeof(ClassRec): the table the caller uploads has 512 such records
int ref_class_rec_bytes(void) { return (int)sizeof(ClassRec); }

// y[d_out] (binary16) = W x for one matrix: words = Planes14 stream of d_out * nblocks records (padded by the
// caller for the four-word window), tab = 512 ClassRec, gscale = the two gain centroids, rscale = d_out row
// scales, tail = d_out * tail_w binary16, x = d_in floats. d_out must be a multiple of 8 (the kernel has no
// row guard). Returns the CUDA error code of the launch.
int ref_tv_planes_h(const unsigned int* words, const void* tab, const float* gscale, const float* rscale,
                    const unsigned short* tail, const float* x, unsigned short* y, unsigned int nblocks,
                    unsigned int tail_w, unsigned int d_out, void* stream) {
    if (d_out % 8u) return (int)cudaErrorInvalidValue;
    tv_planes_h<<<d_out / 8u, 256, TILE_BLOCKS * LLVQ_DIM * sizeof(float), (cudaStream_t)stream>>>(
        words, (const ClassRec*)tab, gscale, rscale, tail, x, y, nblocks, tail_w);
    return (int)cudaGetLastError();
}

}  // extern "C"
