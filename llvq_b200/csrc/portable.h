// Lets the scalar (one-thread) decoders compile both as CUDA device code and as
// plain host C++. The host build exists only so that the test-suite can run the
// very same decode source on a machine without a GPU and diff it against the
// CPU oracle; the library itself never calls the host build.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define LLVQ_DEV __device__ __forceinline__
#define LLVQ_HD __host__ __device__ __forceinline__
#define LLVQ_CONSTEXPR __host__ __device__ constexpr
#else
#define LLVQ_DEV inline
#define LLVQ_HD inline
#define LLVQ_CONSTEXPR constexpr
#endif

namespace llvq {

LLVQ_HD int popc32(unsigned int v) {
#if defined(__CUDA_ARCH__)
    return __popc(v);
#else
    return __builtin_popcount(v);
#endif
}

LLVQ_HD unsigned int umulhi32(unsigned int a, unsigned int b) {
#if defined(__CUDA_ARCH__)
    return __umulhi(a, b);
#else
    return (unsigned int)(((unsigned long long)a * b) >> 32);
#endif
}

}  // namespace llvq

#if defined(__CUDACC__)
// First statement of a kernel that is launched with programmatic stream serialisation: lets the next
// launch of the stream start its own preamble at once, then waits until the previous launch of the
// stream has completed and its writes are visible. A no-op pair in an ordinary launch.
__device__ __forceinline__ void llvq_dependent_enter() {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

