// C ABI of llvq_b200 (see include/llvq_b200.h). Host-side objects own the device
// buffers; every entry point validates its arguments, records a message on
// failure and returns a status instead of aborting.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/llvq_b200.h"
#include "codebook.h"
#include "decode_ops.cuh"
#include "dense_ops.cuh"
#include "archive.h"
#include "rotate.cuh"
#include "rotation.h"
#include "tp_exchange.cuh"
#include "gemm_tab.cuh"
#include "gemv_pipe.cuh"
#include "tab_tables.h"
#include "kernels_generic.cuh"

using namespace llvq;

namespace {

thread_local std::string g_error;
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return code;
}

#define CUDA_TRY(expr)                                                                          \
    do {                                                                                        \
        cudaError_t e_ = (expr);                                                                \
        if (e_ != cudaSuccess)                                                                  \
            return fail(LLVQ_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                        __FILE__, __LINE__);                                                    \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
    }
    ~DeviceGuard() {
        int cur = -1;
        cudaGetDevice(&cur);
        if (prev >= 0 && cur != prev) cudaSetDevice(prev);
    }
};

constexpr int kLutShift = 35;
constexpr int kManySegments = 8;  // segments of llvq_gemv_h_host_many (activations up, results back)

// Launch with programmatic stream serialisation (see llvq_runtime_set_overlap): the kernel may be scheduled
// while the previous kernel of the stream is still running; it orders itself behind that kernel with
// griddepcontrol.wait before it touches memory (llvq_dependent_enter, or the GEMV's own placement of the wait).
std::atomic<int> g_overlap_ops{1};
template <typename... KArgs, typename... Args>
cudaError_t launch_dep(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_overlap_ops.load(std::memory_order_relaxed) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device setting: remember, per (device, kernel),
// the largest size configured so far, so that a second runtime on another GPU raises it again.
std::mutex g_smem_mu;
std::map<std::pair<int, const void*>, size_t> g_smem_configured;

int ensure_dyn_smem(const void* func, size_t bytes) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_smem_mu);
    size_t& have = g_smem_configured[{dev, func}];
    if (bytes > have) {
        CUDA_TRY(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        have = bytes;
    }
    return LLVQ_OK;
}

}  // namespace

struct llvq_runtime {
    int device = 0;
    Codebook cb;
    DevTables T{};
    void* d_cls = nullptr;
    void* d_ends = nullptr;
    void* d_lut = nullptr;
    void* d_golay = nullptr;
    int* d_err = nullptr;  // sticky flag written by kernels: bit 0 index outside the ball, bit 1 copy timeout
    // state-table decoders: the blob the GEMV copies into shared memory, the off-support table
    TabLayout TL{};
    void* d_tab_blob = nullptr;
    void* d_tab_off = nullptr;
    void* d_tab_on3 = nullptr;
    struct KernelInfo {
        const char* name;
        int regs, local_bytes, static_smem, binary_version;
    };
    std::vector<KernelInfo> kernel_info;  // read back at start-up
    uint64_t fingerprint = 0;
    int max_smem_optin = 0;
    int sm_count = 0;
    int overlap_launches = 1;      // GEMV launches carry the programmatic-serialisation attribute
    // staging of llvq_gemv_h_host_many: one pinned host buffer and its device twin, grown on demand
    std::mutex many_mu;
    cudaStream_t many_stream = nullptr;   // copy streams of llvq_gemv_h_host_many (results back, activations up)
    cudaStream_t many_up = nullptr;       // and their per-segment events
    cudaEvent_t many_ready[kManySegments] = {}, many_done[kManySegments] = {}, many_in[kManySegments] = {};
    unsigned char* many_host = nullptr;
    unsigned char* many_dev = nullptr;
    size_t many_bytes = 0;
    // split-K partials of the batched GEMM; grown on demand, shared by all matrices of the runtime
    float* gemm_ws = nullptr;
    size_t gemm_ws_bytes = 0;
};

struct llvq_matrix {
    llvq_runtime* rt = nullptr;
    int d_out = 0, d_in = 0, nb = 0, tail_w = 0, tail_mode = 0;
    unsigned char* codes = nullptr;
    float2* cent = nullptr;
    float* rscale = nullptr;
    void* tail = nullptr;
    size_t codes_bytes = 0;
    // staging for the host-buffer entry points
    void* x_stage = nullptr;
    void* y_stage = nullptr;
    MatrixView view() const {
        MatrixView v;
        v.codes = codes;
        v.cent = cent;
        v.rscale = rscale;
        v.tail = tail;
        v.d_out = d_out;
        v.d_in = d_in;
        v.nb = nb;
        v.tail_w = tail_w;
        v.tail_f16 = tail_mode == LLVQ_TAIL_F16;
        return v;
    }
};

namespace {

size_t generic_smem_bytes(int nb) { return ((size_t)kDim * nb + 32 + (size_t)kGenRows * nb) * sizeof(float); }

template <typename XT, typename YT>
int launch_gemv_generic(llvq_matrix* m, const XT* x, YT* y, cudaStream_t s) {
    llvq_runtime* rt = m->rt;
    const size_t smem = generic_smem_bytes(m->nb);
    if (smem > (size_t)rt->max_smem_optin)
        return fail(LLVQ_ERR_UNSUPPORTED, "d_in %d needs %zu bytes of shared memory (limit %d)", m->d_in, smem,
                    rt->max_smem_optin);
    auto kern = gemv_generic_kernel<XT, YT>;
    {
        int st = ensure_dyn_smem((const void*)kern, smem);
        if (st) return st;
    }
    const int grid = (m->d_out + kGenRows - 1) / kGenRows;
    kern<<<grid, kGenThreads, smem, s>>>(rt->T, m->view(), x, y, kN12, rt->d_err);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

// The persistent pipelined kernel: one CTA per SM, rows split evenly over the CTAs.
template <typename XT, typename YT, int XOP = kXPlain>
int launch_pipe(llvq_matrix* m, const XT* x, YT* y, cudaStream_t s, PipePlan plan, int probe = 0,
                unsigned long long* trace = nullptr, PipeXOp xop = PipeXOp{}) {
    plan.probe = probe;
    plan.trace = trace;
    llvq_runtime* rt = m->rt;
    auto kern = llvq_gemv_pipe_kernel<XT, YT, XOP>;
    int st = ensure_dyn_smem((const void*)kern, plan.total);
    if (st) return st;
    const int grid = (m->d_out + plan.rows_per_cta - 1) / plan.rows_per_cta;
    // Launched with programmatic stream serialisation: when the previous kernel of the stream is another launch of
    // this kernel, the prologue of this one (tables and first codes into shared memory) runs on every SM the previous
    // launch has left, instead of after its last CTA; the kernel orders itself behind the previous launch with
    // griddepcontrol.wait before it touches x or y. After any other kernel the attribute changes nothing.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kPipeThreads);
    cfg.dynamicSmemBytes = plan.total;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = rt->overlap_launches ? 1 : 0;
    CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, (const unsigned char*)rt->d_tab_blob, (const OffEntry*)rt->d_tab_off,
                                (const unsigned long long*)rt->d_tab_on3, rt->TL, m->view(), x, y, plan, xop, rt->d_err));
    g_launches++;
    return LLVQ_OK;
}

template <typename XT, typename YT>
int launch_gemv(llvq_matrix* m, const XT* x, YT* y, cudaStream_t s) {
    llvq_runtime* rt = m->rt;
    // the fused kernels read the activation with 16-byte loads
    if ((uintptr_t)x & 15u) return launch_gemv_generic<XT, YT>(m, x, y, s);
    if (m->nb > 0) {
        const PipePlan plan = pipe_plan<XT>(rt->TL, rt->max_smem_optin, m->d_out, m->nb, rt->sm_count);
        if (plan.tile_max > 0) return launch_pipe<XT, YT>(m, x, y, s, plan);
    }
    // a matrix of tail columns only
    return launch_gemv_generic<XT, YT>(m, x, y, s);
}

template <typename XT, typename YT>
int gemv_entry(llvq_matrix* m, const XT* x, YT* y, llvq_stream_t stream) {
    if (!m || !x || !y) return fail(LLVQ_ERR_INVALID, "gemv: null argument");
    if (((uintptr_t)x % sizeof(XT)) || ((uintptr_t)y % sizeof(YT))) return fail(LLVQ_ERR_INVALID, "gemv: misaligned buffer");
    DeviceGuard g(m->rt->device);
    return launch_gemv<XT, YT>(m, x, y, (cudaStream_t)stream);
}

// The projection with its activation produced in the kernel's staging step (f16, pipelined kernel only).
template <int XOP>
int gemv_xop_entry(llvq_matrix* m, const __half* x, __half* y, const PipeXOp& xop, cudaStream_t s, const char* what) {
    llvq_runtime* rt = m->rt;
    DeviceGuard g(rt->device);
    const PipePlan plan = pipe_plan<__half>(rt->TL, rt->max_smem_optin, m->d_out, m->nb, rt->sm_count);
    if (m->nb == 0 || plan.tile_max == 0) return fail(LLVQ_ERR_UNSUPPORTED, "%s: matrix not served by the pipelined kernel", what);
    return launch_pipe<__half, __half, XOP>(m, x, y, s, plan, 0, nullptr, xop);
}

int check_desc(const llvq_matrix_desc& d) {
    if (d.d_out <= 0 || d.d_in <= 0) return fail(LLVQ_ERR_INVALID, "matrix: d_out %d, d_in %d", d.d_out, d.d_in);
    if (d.shell_cap != 12)
        return fail(LLVQ_ERR_UNSUPPORTED, "matrix: shell cap %d; only the 47-bit cap-12 ball is served", d.shell_cap);
    if (d.tail_mode != LLVQ_TAIL_F32 && d.tail_mode != LLVQ_TAIL_F16) return fail(LLVQ_ERR_INVALID, "matrix: tail_mode %d", d.tail_mode);
    if (!d.centroids || !d.row_scales) return fail(LLVQ_ERR_INVALID, "matrix: null centroids or row scales");
    if (d.d_in / kDim > 0 && !d.codes) return fail(LLVQ_ERR_INVALID, "matrix: null code stream");
    if (d.d_in % kDim > 0 && !d.tail) return fail(LLVQ_ERR_INVALID, "matrix: null tail with %d tail columns", d.d_in % kDim);
    return LLVQ_OK;
}

void free_matrix_buffers(llvq_matrix* m) {
    cudaFree(m->codes);
    cudaFree(m->cent);
    cudaFree(m->rscale);
    cudaFree(m->tail);
    cudaFree(m->x_stage);
    cudaFree(m->y_stage);
}

int upload_impl(llvq_runtime* rt, const llvq_matrix_desc* descs, int n, llvq_matrix** out) {
    if (!rt || !descs || !out || n <= 0) return fail(LLVQ_ERR_INVALID, "upload: null argument");
    long long d_out = 0;
    for (int i = 0; i < n; ++i) {
        int st = check_desc(descs[i]);
        if (st) return st;
        if (descs[i].d_in != descs[0].d_in || descs[i].tail_mode != descs[0].tail_mode)
            return fail(LLVQ_ERR_INVALID, "upload_group: segment %d differs in d_in or tail_mode", i);
        d_out += descs[i].d_out;
    }
    if (d_out > (1ll << 30)) return fail(LLVQ_ERR_INVALID, "upload: %lld rows", d_out);
    DeviceGuard g(rt->device);
    std::unique_ptr<llvq_matrix> m(new llvq_matrix);
    m->rt = rt;
    m->d_out = (int)d_out;
    m->d_in = descs[0].d_in;
    m->nb = m->d_in / kDim;
    m->tail_w = m->d_in % kDim;
    m->tail_mode = descs[0].tail_mode;
    m->codes_bytes = (size_t)m->d_out * m->nb * 6;

    // Host staging: concatenate the segments row-wise; narrow scales to f32 with one
    // rounding (llvq-llm/src/fused.rs:1210-1212) and the tail to binary16 when asked
    // (fused.rs:655-659).
    std::vector<unsigned char> codes(m->codes_bytes + 64, 0);
    std::vector<float2> cent((size_t)m->d_out);
    std::vector<float> rs((size_t)m->d_out);
    std::vector<float> tail32((size_t)m->d_out * m->tail_w);
    size_t row = 0;
    for (int i = 0; i < n; ++i) {
        const llvq_matrix_desc& d = descs[i];
        std::memcpy(codes.data() + row * m->nb * 6, d.codes ? d.codes : codes.data(), (size_t)d.d_out * m->nb * 6);
        for (int r = 0; r < d.d_out; ++r) {
            cent[row + r] = make_float2((float)d.centroids[0], (float)d.centroids[1]);
            rs[row + r] = (float)d.row_scales[r];
        }
        if (m->tail_w) std::memcpy(tail32.data() + row * m->tail_w, d.tail, (size_t)d.d_out * m->tail_w * sizeof(float));
        row += d.d_out;
    }
    auto bail = [&](int st) {
        free_matrix_buffers(m.get());
        return st;
    };
#define UP_TRY(expr)                                                                                             \
    do {                                                                                                         \
        cudaError_t e_ = (expr);                                                                                 \
        if (e_ != cudaSuccess) return bail(fail(LLVQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_))); \
    } while (0)
    UP_TRY(cudaMalloc(&m->codes, codes.size()));
    UP_TRY(cudaMemcpy(m->codes, codes.data(), codes.size(), cudaMemcpyHostToDevice));
    UP_TRY(cudaMalloc(&m->cent, cent.size() * sizeof(float2)));
    UP_TRY(cudaMemcpy(m->cent, cent.data(), cent.size() * sizeof(float2), cudaMemcpyHostToDevice));
    UP_TRY(cudaMalloc(&m->rscale, rs.size() * sizeof(float)));
    UP_TRY(cudaMemcpy(m->rscale, rs.data(), rs.size() * sizeof(float), cudaMemcpyHostToDevice));
    if (m->tail_w) {
        if (m->tail_mode == LLVQ_TAIL_F16) {
            std::vector<__half> t16(tail32.size());
            for (size_t i = 0; i < tail32.size(); ++i) t16[i] = __float2half_rn(tail32[i]);
            UP_TRY(cudaMalloc(&m->tail, t16.size() * sizeof(__half)));
            UP_TRY(cudaMemcpy(m->tail, t16.data(), t16.size() * sizeof(__half), cudaMemcpyHostToDevice));
        } else {
            UP_TRY(cudaMalloc(&m->tail, tail32.size() * sizeof(float)));
            UP_TRY(cudaMemcpy(m->tail, tail32.data(), tail32.size() * sizeof(float), cudaMemcpyHostToDevice));
        }
    } else {
        UP_TRY(cudaMalloc(&m->tail, 16));  // never read; keeps the pointer valid
    }
    UP_TRY(cudaMalloc(&m->x_stage, (size_t)m->d_in * sizeof(float) + 16));
    UP_TRY(cudaMalloc(&m->y_stage, (size_t)m->d_out * sizeof(float) + 16));
#undef UP_TRY
    *out = m.release();
    return LLVQ_OK;
}

template <typename XT, typename YT>
int gemv_host(llvq_matrix* m, const XT* xh, YT* yh, llvq_stream_t stream) {
    if (!m || !xh || !yh) return fail(LLVQ_ERR_INVALID, "gemv_host: null argument");
    DeviceGuard g(m->rt->device);
    cudaStream_t s = (cudaStream_t)stream;
    CUDA_TRY(cudaMemcpyAsync(m->x_stage, xh, (size_t)m->d_in * sizeof(XT), cudaMemcpyHostToDevice, s));
    int st = launch_gemv<XT, YT>(m, (const XT*)m->x_stage, (YT*)m->y_stage, s);
    if (st) return st;
    CUDA_TRY(cudaMemcpyAsync(yh, m->y_stage, (size_t)m->d_out * sizeof(YT), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    return LLVQ_OK;
}

}  // namespace

struct llvq_archive {
    Archive a;
};

struct llvq_rotation {
    llvq_runtime* rt = nullptr;
    RotationTables t;
    unsigned int* d_signbits = nullptr;
    float* d_small = nullptr;
    size_t smem = 0;
};

struct llvq_tp_ctx {
    int device = 0;
    TpRank r{};
};

template <int HD, int G>
static int launch_attn(const __half* q, const KvCacheView& kc, const KvCacheView& vc, const long long* pos, __half* out,
                       float* scratch, int n_kv, int splits, cudaStream_t s) {
    const int smem = (int)sizeof(AttnSmem<HD, G>);
    {
        int st = ensure_dyn_smem((const void*)attn_splitkv_kernel<HD, G>, (size_t)smem);
        if (st) return st;
    }
    CUDA_TRY(launch_dep(attn_splitkv_kernel<HD, G>, dim3(n_kv, splits), dim3(kAttnThreads), smem, s, q, kc, vc, pos, out, scratch, n_kv));
    if (splits > 1) CUDA_TRY(launch_dep(attn_combine_kernel<HD>, dim3(n_kv * G), dim3(HD), splits * sizeof(float), s, scratch, out, splits));
    g_launches += splits > 1 ? 2 : 1;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

template <int HD>
static int launch_attn_g(int G, const __half* q, const KvCacheView& kc, const KvCacheView& vc, const long long* pos,
                         __half* out, float* scratch, int n_kv, int splits, cudaStream_t s) {
    switch (G) {
        case 1: return launch_attn<HD, 1>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
        case 2: return launch_attn<HD, 2>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
        case 3: return launch_attn<HD, 3>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
        case 4: return launch_attn<HD, 4>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
        case 5: return launch_attn<HD, 5>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
        case 6: return launch_attn<HD, 6>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
        case 7: return launch_attn<HD, 7>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
        case 8: return launch_attn<HD, 8>(q, kc, vc, pos, out, scratch, n_kv, splits, s);
    }
    return fail(LLVQ_ERR_UNSUPPORTED, "op_attn_decode: %d query heads per KV head (1 to %d)", G, kAttnMaxG);
}

extern "C" {

const char* llvq_last_error(void) { return g_error.c_str(); }
const char* llvq_version(void) { return "0.1.0"; }
uint64_t llvq_launch_count(void) { return g_launches.load(); }

void llvq_runtime_destroy(llvq_runtime* rt) {
    if (!rt) return;
    DeviceGuard g(rt->device);
    cudaFree(rt->d_cls);
    cudaFree(rt->d_ends);
    cudaFree(rt->d_lut);
    cudaFree(rt->d_golay);
    cudaFree(rt->d_err);
    cudaFree(rt->gemm_ws);
    cudaFreeHost(rt->many_host);
    cudaFree(rt->many_dev);
    if (rt->many_stream) {
        for (int k = 0; k < kManySegments; ++k) {
            cudaEventDestroy(rt->many_ready[k]);
            cudaEventDestroy(rt->many_in[k]);
            cudaEventDestroy(rt->many_done[k]);
        }
        cudaStreamDestroy(rt->many_stream);
        cudaStreamDestroy(rt->many_up);
    }
    cudaFree(rt->d_tab_blob);
    cudaFree(rt->d_tab_off);
    cudaFree(rt->d_tab_on3);
    delete rt;
}

int llvq_runtime_create(int device, llvq_runtime** out) {
    if (!out) return fail(LLVQ_ERR_INVALID, "runtime_create: null out");
    *out = nullptr;
    int ndev = 0;
    CUDA_TRY(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev) return fail(LLVQ_ERR_INVALID, "runtime_create: device %d of %d", device, ndev);
    DeviceGuard g(device);
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(LLVQ_ERR_UNSUPPORTED, "runtime_create: device %d is sm_%d%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
    std::unique_ptr<llvq_runtime> rt(new llvq_runtime);
    rt->device = device;
    rt->max_smem_optin = (int)prop.sharedMemPerBlockOptin;
    rt->sm_count = prop.multiProcessorCount;
    const Codebook& cb = rt->cb;
    if (cb.classes.size() != (size_t)kMaxClasses || cb.n_classes12 != 301 || cb.total13 != kN13 || cb.total12 != kN12)
        return fail(LLVQ_ERR_CODEBOOK, "class enumeration does not cover the ball: %zu classes, N=%llu", cb.classes.size(),
                    (unsigned long long)cb.total13);
    std::vector<DevClass> dc;
    cb.dev_classes(dc);
    std::vector<uint16_t> lut;
    cb.class_lut(kLutShift, lut);
    auto bail = [&](int st) {
        llvq_runtime_destroy(rt.release());
        return st;
    };
#define RT_TRY(expr)                                                                                             \
    do {                                                                                                         \
        cudaError_t e_ = (expr);                                                                                 \
        if (e_ != cudaSuccess) return bail(fail(LLVQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_))); \
    } while (0)
    RT_TRY(cudaMalloc(&rt->d_cls, dc.size() * sizeof(DevClass)));
    RT_TRY(cudaMemcpy(rt->d_cls, dc.data(), dc.size() * sizeof(DevClass), cudaMemcpyHostToDevice));
    RT_TRY(cudaMalloc(&rt->d_ends, cb.ends.size() * sizeof(uint64_t)));
    RT_TRY(cudaMemcpy(rt->d_ends, cb.ends.data(), cb.ends.size() * sizeof(uint64_t), cudaMemcpyHostToDevice));
    RT_TRY(cudaMalloc(&rt->d_lut, lut.size() * sizeof(uint16_t)));
    RT_TRY(cudaMemcpy(rt->d_lut, lut.data(), lut.size() * sizeof(uint16_t), cudaMemcpyHostToDevice));
    RT_TRY(cudaMalloc(&rt->d_golay, sizeof cb.golay));
    RT_TRY(cudaMemcpy(rt->d_golay, cb.golay, sizeof cb.golay, cudaMemcpyHostToDevice));
    RT_TRY(cudaMalloc((void**)&rt->d_err, sizeof(int)));
    RT_TRY(cudaMemset(rt->d_err, 0, sizeof(int)));
    rt->T.cls = (const DevClass*)rt->d_cls;
    rt->T.ends = (const unsigned long long*)rt->d_ends;
    rt->T.lut = (const unsigned short*)rt->d_lut;
    rt->T.golay = (const unsigned int*)rt->d_golay;
    rt->T.lut_shift = kLutShift;

    {
        TabTablesHost th;
        build_tab_tables(cb, th);
        rt->TL = th.layout;
        RT_TRY(cudaMalloc(&rt->d_tab_blob, th.blob.size()));
        RT_TRY(cudaMemcpy(rt->d_tab_blob, th.blob.data(), th.blob.size(), cudaMemcpyHostToDevice));
        RT_TRY(cudaMalloc(&rt->d_tab_off, th.lut_off.size() * sizeof(OffEntry)));
        RT_TRY(cudaMemcpy(rt->d_tab_off, th.lut_off.data(), th.lut_off.size() * sizeof(OffEntry), cudaMemcpyHostToDevice));
        RT_TRY(cudaMalloc(&rt->d_tab_on3, th.lut_on3.size() * sizeof(unsigned long long)));
        RT_TRY(cudaMemcpy(rt->d_tab_on3, th.lut_on3.data(), th.lut_on3.size() * sizeof(unsigned long long), cudaMemcpyHostToDevice));
        if (th.slow_mass != 0.0) return bail(fail(LLVQ_ERR_CODEBOOK, "decoder tables leave %.3g of the ball unserved", th.slow_mass));
    }

    // The hot kernels must run out of registers only: a spill to local memory is refused, as the reference
    // refuses it when it loads its kernels (llvq-cuda/src/gpu.rs:413-436, llvq-llm/src/fused_cuda.rs:229-239).
    {
        const struct { const char* name; const void* fn; } hot[] = {
            {"llvq_gemv_pipe_kernel<f16,f16>", (const void*)llvq_gemv_pipe_kernel<__half, __half, kXPlain>},
            {"llvq_gemv_pipe_kernel<f16,f16,norm>", (const void*)llvq_gemv_pipe_kernel<__half, __half, kXNorm>},
            {"llvq_gemv_pipe_kernel<f16,f16,silu>", (const void*)llvq_gemv_pipe_kernel<__half, __half, kXSilu>},
            {"llvq_gemv_pipe_kernel<f32,f16>", (const void*)llvq_gemv_pipe_kernel<float, __half, kXPlain>},
            {"llvq_gemv_pipe_kernel<f32,f32>", (const void*)llvq_gemv_pipe_kernel<float, float, kXPlain>},
            {"llvq_decode_tab_kernel", (const void*)llvq_decode_tab_kernel},
            {"llvq_gemm_tab_kernel", (const void*)llvq_gemm_tab_kernel},
        };
        for (const auto& k : hot) {
            cudaFuncAttributes fa;
            RT_TRY(cudaFuncGetAttributes(&fa, k.fn));
            rt->kernel_info.push_back({k.name, fa.numRegs, (int)fa.localSizeBytes, (int)fa.sharedSizeBytes, fa.binaryVersion});
            if (fa.localSizeBytes != 0)
                return bail(fail(LLVQ_ERR_UNSUPPORTED, "%s uses %zu bytes of local memory per thread (register spill): refused",
                                 k.name, (size_t)fa.localSizeBytes));
        }
    }

    // Verify the device tables against the published fingerprint: decode the probe
    // indices on the GPU and fold them into the reference's digest.
    std::vector<uint64_t> probes;
    probe_indices(cb, probes);
    const size_t np = probes.size();
    unsigned long long* d_idx = nullptr;
    signed char* d_pts = nullptr;
    unsigned char* d_shell = nullptr;
    RT_TRY(cudaMalloc(&d_idx, np * sizeof(uint64_t)));
    RT_TRY(cudaMalloc(&d_pts, np * kDim));
    RT_TRY(cudaMalloc(&d_shell, np));
    RT_TRY(cudaMemcpy(d_idx, probes.data(), np * sizeof(uint64_t), cudaMemcpyHostToDevice));
    decode_indices_kernel<<<(unsigned)((np + 127) / 128), 128>>>(rt->T, d_idx, np, d_pts, d_shell, kN13);
    g_launches++;
    RT_TRY(cudaGetLastError());
    std::vector<int8_t> pts(np * kDim);
    std::vector<uint8_t> shell(np), ok(np);
    RT_TRY(cudaMemcpy(pts.data(), d_pts, np * kDim, cudaMemcpyDeviceToHost));
    RT_TRY(cudaMemcpy(shell.data(), d_shell, np, cudaMemcpyDeviceToHost));
    cudaFree(d_idx);
    cudaFree(d_pts);
    cudaFree(d_shell);
#undef RT_TRY
    for (size_t i = 0; i < np; ++i) ok[i] = shell[i] != 255;
    rt->fingerprint = fingerprint_from_points(cb, probes, pts.data(), ok.data());
    if (rt->fingerprint != LLVQ_PUBLISHED_FINGERPRINT)
        return bail(fail(LLVQ_ERR_CODEBOOK, "device codebook fingerprint %016llx differs from the published %016llx",
                         (unsigned long long)rt->fingerprint, (unsigned long long)LLVQ_PUBLISHED_FINGERPRINT));
    *out = rt.release();
    return LLVQ_OK;
}

int llvq_codebook_fingerprint(llvq_runtime* rt, uint64_t* out) {
    if (!rt || !out) return fail(LLVQ_ERR_INVALID, "codebook_fingerprint: null argument");
    *out = rt->fingerprint;
    return LLVQ_OK;
}

int llvq_codebook_info(llvq_runtime* rt, int shell_cap, int32_t* n_classes, uint64_t* ball_size) {
    if (!rt) return fail(LLVQ_ERR_INVALID, "codebook_info: null runtime");
    if (shell_cap != 12 && shell_cap != 13) return fail(LLVQ_ERR_INVALID, "codebook_info: shell cap %d", shell_cap);
    if (n_classes) *n_classes = shell_cap == 12 ? rt->cb.n_classes12 : (int)rt->cb.classes.size();
    if (ball_size) *ball_size = shell_cap == 12 ? rt->cb.total12 : rt->cb.total13;
    return LLVQ_OK;
}

int llvq_codebook_class_record(int32_t ci, void* out) {
    static const Codebook cb;
    static const std::vector<DevClass> dc = [] {
        std::vector<DevClass> v;
        cb.dev_classes(v);
        return v;
    }();
    if (!out || ci < 0 || ci >= (int)dc.size()) return fail(LLVQ_ERR_INVALID, "class_record: class %d", ci);
    std::memcpy(out, &dc[ci], sizeof(DevClass));
    return LLVQ_OK;
}

int llvq_codebook_golay(uint32_t* out) {
    static const Codebook cb;
    if (!out) return fail(LLVQ_ERR_INVALID, "codebook_golay: null out");
    std::memcpy(out, cb.golay, sizeof cb.golay);
    return LLVQ_OK;
}

int llvq_runtime_set_overlap(llvq_runtime* rt, int32_t on) {
    if (!rt) return fail(LLVQ_ERR_INVALID, "set_overlap: null runtime");
    rt->overlap_launches = on ? 1 : 0;
    g_overlap_ops.store(on ? 1 : 0);  // the decode-step kernels take no runtime: one switch for the process
    return LLVQ_OK;
}

int llvq_runtime_kernel_info(llvq_runtime* rt, int32_t index, const char** name, int32_t* regs, int32_t* local_bytes,
                             int32_t* static_smem_bytes, int32_t* binary_version) {
    if (!rt) return fail(LLVQ_ERR_INVALID, "kernel_info: null runtime");
    if (index < 0 || index >= (int)rt->kernel_info.size()) return fail(LLVQ_ERR_INVALID, "kernel_info: index %d of %zu", index, rt->kernel_info.size());
    const auto& k = rt->kernel_info[index];
    if (name) *name = k.name;
    if (regs) *regs = k.regs;
    if (local_bytes) *local_bytes = k.local_bytes;
    if (static_smem_bytes) *static_smem_bytes = k.static_smem;
    if (binary_version) *binary_version = k.binary_version;
    return LLVQ_OK;
}

int llvq_runtime_poll_error(llvq_runtime* rt, int32_t* flag) {
    if (!rt || !flag) return fail(LLVQ_ERR_INVALID, "poll_error: null argument");
    DeviceGuard g(rt->device);
    CUDA_TRY(cudaDeviceSynchronize());
    int v = 0;
    CUDA_TRY(cudaMemcpy(&v, rt->d_err, sizeof v, cudaMemcpyDeviceToHost));
    CUDA_TRY(cudaMemset(rt->d_err, 0, sizeof v));
    *flag = v;
    return LLVQ_OK;
}

int llvq_matrix_upload(llvq_runtime* rt, const llvq_matrix_desc* desc, llvq_matrix** out) {
    return upload_impl(rt, desc, 1, out);
}

int llvq_matrix_upload_group(llvq_runtime* rt, const llvq_matrix_desc* descs, int32_t n, llvq_matrix** out) {
    return upload_impl(rt, descs, n, out);
}

void llvq_matrix_free(llvq_matrix* m) {
    if (!m) return;
    DeviceGuard g(m->rt->device);
    free_matrix_buffers(m);
    delete m;
}

int llvq_matrix_dims(const llvq_matrix* m, int32_t* d_out, int32_t* d_in) {
    if (!m) return fail(LLVQ_ERR_INVALID, "matrix_dims: null matrix");
    if (d_out) *d_out = m->d_out;
    if (d_in) *d_in = m->d_in;
    return LLVQ_OK;
}

int llvq_matrix_algorithmic_bytes(const llvq_matrix* m, int32_t x_elem_bytes, int32_t y_elem_bytes, uint64_t* out) {
    if (!m || !out) return fail(LLVQ_ERR_INVALID, "algorithmic_bytes: null argument");
    *out = (uint64_t)m->codes_bytes + (uint64_t)m->d_out * m->tail_w * 4 + (uint64_t)m->d_out * 8 +
           (uint64_t)m->d_in * x_elem_bytes + (uint64_t)m->d_out * y_elem_bytes;
    return LLVQ_OK;
}

int llvq_gemv_f32(llvq_matrix* m, const float* x, float* y, llvq_stream_t s) { return gemv_entry<float, float>(m, x, y, s); }
int llvq_gemv_h(llvq_matrix* m, const uint16_t* x, uint16_t* y, llvq_stream_t s) {
    return gemv_entry<__half, __half>(m, (const __half*)x, (__half*)y, s);
}
int llvq_gemv_f32x_h(llvq_matrix* m, const float* x, uint16_t* y, llvq_stream_t s) {
    return gemv_entry<float, __half>(m, x, (__half*)y, s);
}

int llvq_gemv_norm_h(llvq_matrix* m, const uint16_t* resid, const uint16_t* delta, const uint16_t* norm_w, float eps,
                     uint16_t* resid_out, uint16_t* y, llvq_stream_t s) {
    if (!m || !resid || !norm_w || !resid_out || !y) return fail(LLVQ_ERR_INVALID, "gemv_norm: null argument");
    if (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)norm_w | (uintptr_t)resid_out) & 15u)
        return fail(LLVQ_ERR_INVALID, "gemv_norm: the vectors must be 16-byte aligned");
    if ((uintptr_t)y & 1u) return fail(LLVQ_ERR_INVALID, "gemv_norm: misaligned result");
    if (resid_out == resid) return fail(LLVQ_ERR_INVALID, "gemv_norm: the updated stream must not alias the stream read");
    if ((m->d_in & 1) || m->d_in > 16384) return fail(LLVQ_ERR_UNSUPPORTED, "gemv_norm: width %d (even, up to 16384)", m->d_in);
    PipeXOp xop{};
    xop.delta = (const __half*)delta;
    xop.w = (const __half*)norm_w;
    xop.x_out = (__half*)resid_out;
    xop.eps = eps;
    xop.n = m->d_in;
    return gemv_xop_entry<kXNorm>(m, (const __half*)resid, (__half*)y, xop, (cudaStream_t)s, "gemv_norm");
}

int llvq_gemv_silu_h(llvq_matrix* m, const uint16_t* gate_up, uint16_t* y, llvq_stream_t s) {
    if (!m || !gate_up || !y) return fail(LLVQ_ERR_INVALID, "gemv_silu: null argument");
    if (((uintptr_t)gate_up & 15u) || (m->d_in & 7))
        return fail(LLVQ_ERR_INVALID, "gemv_silu: gate and up must both start on 16 bytes (width a multiple of 8)");
    if ((uintptr_t)y & 1u) return fail(LLVQ_ERR_INVALID, "gemv_silu: misaligned result");
    PipeXOp xop{};
    xop.n = m->d_in;
    return gemv_xop_entry<kXSilu>(m, (const __half*)gate_up, (__half*)y, xop, (cudaStream_t)s, "gemv_silu");
}

int llvq_gemv_probe_h(llvq_matrix* m, const uint16_t* x, uint16_t* y, int32_t mode, llvq_stream_t s) {
    if (!m || !x || !y) return fail(LLVQ_ERR_INVALID, "gemv_probe: null argument");
    if (mode < 0 || mode > 7) return fail(LLVQ_ERR_INVALID, "gemv_probe: mode %d (0 to 7)", mode);
    if (((uintptr_t)x & 15u) || ((uintptr_t)y & 1u)) return fail(LLVQ_ERR_INVALID, "gemv_probe: x must be 16-byte aligned");
    llvq_runtime* rt = m->rt;
    DeviceGuard g(rt->device);
    const PipePlan plan = pipe_plan<__half>(rt->TL, rt->max_smem_optin, m->d_out, m->nb, rt->sm_count);
    if (m->nb == 0 || plan.tile_max == 0) return fail(LLVQ_ERR_UNSUPPORTED, "gemv_probe: matrix not served by the pipelined kernel");
    return launch_pipe<__half, __half>(m, (const __half*)x, (__half*)y, (cudaStream_t)s, plan, mode);
}

int llvq_gemv_trace_h(llvq_matrix* m, const uint16_t* x, uint16_t* y, int32_t mode, uint64_t* trace_host, int32_t max_ctas,
                      int32_t* n_ctas, llvq_stream_t s) {
    if (!m || !x || !y || !trace_host || !n_ctas || max_ctas <= 0) return fail(LLVQ_ERR_INVALID, "gemv_trace: bad argument");
    if (mode < 0 || mode > 7) return fail(LLVQ_ERR_INVALID, "gemv_trace: mode %d (0 to 7)", mode);
    if (((uintptr_t)x & 15u) || ((uintptr_t)y & 1u)) return fail(LLVQ_ERR_INVALID, "gemv_trace: x must be 16-byte aligned");
    llvq_runtime* rt = m->rt;
    DeviceGuard g(rt->device);
    const PipePlan plan = pipe_plan<__half>(rt->TL, rt->max_smem_optin, m->d_out, m->nb, rt->sm_count);
    if (m->nb == 0 || plan.tile_max == 0) return fail(LLVQ_ERR_UNSUPPORTED, "gemv_trace: matrix not served by the pipelined kernel");
    const int grid = (m->d_out + plan.rows_per_cta - 1) / plan.rows_per_cta;
    unsigned long long* d_trace = nullptr;
    const size_t bytes = (size_t)grid * kTraceEvents * sizeof(unsigned long long);
    CUDA_TRY(cudaMalloc((void**)&d_trace, bytes));
    cudaMemsetAsync(d_trace, 0, bytes, (cudaStream_t)s);
    int st = launch_pipe<__half, __half>(m, (const __half*)x, (__half*)y, (cudaStream_t)s, plan, mode, d_trace);
    if (!st) {
        cudaError_t e = cudaStreamSynchronize((cudaStream_t)s);
        const int n = grid < max_ctas ? grid : max_ctas;
        if (e == cudaSuccess) e = cudaMemcpy(trace_host, d_trace, (size_t)n * kTraceEvents * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) st = fail(LLVQ_ERR_CUDA, "gemv_trace: %s", cudaGetErrorString(e));
        *n_ctas = n;
    }
    cudaFree(d_trace);
    return st;
}

int llvq_gemm_h(llvq_matrix* m, const uint16_t* x, uint16_t* y, int32_t batch, llvq_stream_t stream) {
    if (!m || !x || !y || batch <= 0) return fail(LLVQ_ERR_INVALID, "gemm_h: bad argument");
    if (((uintptr_t)x & 1u) || ((uintptr_t)y & 1u)) return fail(LLVQ_ERR_INVALID, "gemm_h: misaligned buffer");
    llvq_runtime* rt = m->rt;
    DeviceGuard g(rt->device);
    cudaStream_t s = (cudaStream_t)stream;
    if (batch < 16) {
        // below 16 rows the contraction is too thin for the tensor cores: one fused GEMV per row,
        // as the reference's drive_rows does (llvq-llm/src/model.rs:497-536)
        for (int b = 0; b < batch; ++b) {
            int st = launch_gemv<__half, __half>(m, (const __half*)x + (size_t)b * m->d_in,
                                                 (__half*)y + (size_t)b * m->d_out, s);
            if (st) return st;
        }
        return LLVQ_OK;
    }
    // one persistent CTA per SM walks (row tile, column split) units; the plan picks the split
    const GemmTabPlan plan = gemm_tab_plan(rt->TL, m->d_out, m->nb, rt->sm_count);
    const int splits = plan.splits;
    if ((int)plan.total > rt->max_smem_optin) return fail(LLVQ_ERR_UNSUPPORTED, "gemm_h: %u bytes of shared memory", plan.total);
    const size_t need = (size_t)(splits > 0 ? splits : 1) * kGMaxN * m->d_out * sizeof(float);
    if (need > rt->gemm_ws_bytes) {  // first use or a larger matrix: (re)allocate the workspace
        CUDA_TRY(cudaStreamSynchronize(s));
        CUDA_TRY(cudaFree(rt->gemm_ws));
        rt->gemm_ws = nullptr;
        rt->gemm_ws_bytes = 0;
        CUDA_TRY(cudaMalloc((void**)&rt->gemm_ws, need));
        rt->gemm_ws_bytes = need;
    }
    {
        int st = ensure_dyn_smem((const void*)llvq_gemm_tab_kernel, plan.total);
        if (st) return st;
    }
    const MatrixView mv = m->view();
    const int want_ctas = (plan.units + kTGHalves - 1) / kTGHalves;  // every CTA runs two unit streams
    const int grid = want_ctas < rt->sm_count ? want_ctas : rt->sm_count;
    for (int b0 = 0; b0 < batch; b0 += kGMaxN) {
        const int nb_rows = batch - b0 < kGMaxN ? batch - b0 : kGMaxN;
        GemmArgs ga;
        ga.x = (const __half*)x + (size_t)b0 * m->d_in;
        ga.ws = rt->gemm_ws;
        ga.batch = nb_rows;
        ga.n_pad = (nb_rows + 15) & ~15;
        ga.x_vec_ok = ((m->d_in & 7) == 0 && ((uintptr_t)ga.x & 15u) == 0) ? 1 : 0;
        if (splits > 0) {
            CUDA_TRY(launch_dep(llvq_gemm_tab_kernel, dim3(grid), dim3(kTGThreads), plan.total, s, (const unsigned char*)rt->d_tab_blob,
                                (const OffEntry*)rt->d_tab_off, (const unsigned long long*)rt->d_tab_on3, rt->TL, mv, ga, plan,
                                rt->d_err));
            g_launches++;
            CUDA_TRY(cudaGetLastError());
        }
        CUDA_TRY(launch_dep(gemm_reduce_kernel, dim3((m->d_out + 127) / 128, nb_rows), dim3(128), 0, s, mv, ga.x, rt->gemm_ws,
                            (__half*)y + (size_t)b0 * m->d_out, nb_rows, ga.n_pad, splits));
        g_launches++;
        CUDA_TRY(cudaGetLastError());
    }
    return LLVQ_OK;
}

int llvq_gemv_f32_host(llvq_matrix* m, const float* x, float* y, llvq_stream_t s) { return gemv_host<float, float>(m, x, y, s); }
int llvq_gemv_h_host(llvq_matrix* m, const uint16_t* x, uint16_t* y, llvq_stream_t s) {
    return gemv_host<__half, __half>(m, (const __half*)x, (__half*)y, s);
}

int llvq_op_add_rmsnorm_h(uint16_t* x, const uint16_t* delta, const uint16_t* w, uint16_t* y, int32_t n, float eps,
                          llvq_stream_t stream) {
    if (!x || !w || !y || n <= 0 || (n & 1) || n > 16384) return fail(LLVQ_ERR_INVALID, "op_add_rmsnorm: bad argument (n even, <= 16384)");
    CUDA_TRY(launch_dep(add_rmsnorm_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, (__half*)x, (const __half*)delta, (const __half*)w, (__half*)y, n,
                                                            eps));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_op_qkv_rope_cache_h(const uint16_t* qkv, const uint16_t* q_norm, const uint16_t* k_norm, const float* cos_t,
                             const float* sin_t, const int64_t* pos, uint16_t* q_out, uint8_t* kq, uint16_t* ks,
                             uint16_t* kb, uint8_t* vq, uint16_t* vs, uint16_t* vb, int32_t n_heads, int32_t n_kv,
                             int32_t head_dim, float eps, llvq_stream_t stream) {
    if (!qkv || !q_norm || !k_norm || !cos_t || !sin_t || !pos || !q_out || !kq || !ks || !kb || !vq || !vs || !vb)
        return fail(LLVQ_ERR_INVALID, "op_qkv_rope_cache: null argument");
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv) return fail(LLVQ_ERR_INVALID, "op_qkv_rope_cache: %d heads over %d", n_heads, n_kv);
    const KvCacheView kc{kq, (__half*)ks, (__half*)kb}, vc{vq, (__half*)vs, (__half*)vb};
    const int grid = n_heads + 2 * n_kv;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 128)
        CUDA_TRY(launch_dep(qkv_rope_cache_kernel<128>, dim3(grid), dim3(32), 0, s, (const __half*)qkv, (const __half*)q_norm, (const __half*)k_norm, cos_t,
                                                       sin_t, (const long long*)pos, (__half*)q_out, kc, vc, n_heads, n_kv, eps));
    else if (head_dim == 64)
        CUDA_TRY(launch_dep(qkv_rope_cache_kernel<64>, dim3(grid), dim3(32), 0, s, (const __half*)qkv, (const __half*)q_norm, (const __half*)k_norm, cos_t,
                                                      sin_t, (const long long*)pos, (__half*)q_out, kc, vc, n_heads, n_kv, eps));
    else
        return fail(LLVQ_ERR_UNSUPPORTED, "op_qkv_rope_cache: head_dim %d (64 or 128)", head_dim);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_op_attn_decode_int8_h(const uint16_t* q, const uint8_t* kq, const uint16_t* ks, const uint16_t* kb,
                               const uint8_t* vq, const uint16_t* vs, const uint16_t* vb, const int64_t* pos, uint16_t* out,
                               int32_t n_heads, int32_t n_kv, int32_t head_dim, int32_t splits, float* scratch,
                               llvq_stream_t stream) {
    if (!q || !kq || !ks || !kb || !vq || !vs || !vb || !pos || !out) return fail(LLVQ_ERR_INVALID, "op_attn_decode: null argument");
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv) return fail(LLVQ_ERR_INVALID, "op_attn_decode: %d heads over %d", n_heads, n_kv);
    if (splits < 1 || splits > 4096 || (splits > 1 && !scratch))
        return fail(LLVQ_ERR_INVALID, "op_attn_decode: %d splits need a scratch buffer", splits);
    if (((uintptr_t)kq & 15u) || ((uintptr_t)vq & 15u)) return fail(LLVQ_ERR_INVALID, "op_attn_decode: cache codes must be 16-byte aligned");
    const KvCacheView kc{(unsigned char*)kq, (__half*)ks, (__half*)kb}, vc{(unsigned char*)vq, (__half*)vs, (__half*)vb};
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 128)
        return launch_attn_g<128>(n_heads / n_kv, (const __half*)q, kc, vc, (const long long*)pos, (__half*)out, scratch, n_kv, splits, s);
    if (head_dim == 64)
        return launch_attn_g<64>(n_heads / n_kv, (const __half*)q, kc, vc, (const long long*)pos, (__half*)out, scratch, n_kv, splits, s);
    return fail(LLVQ_ERR_UNSUPPORTED, "op_attn_decode: head_dim %d (64 or 128)", head_dim);
}

int llvq_op_silu_mul_h(const uint16_t* gu, uint16_t* y, int32_t inter, llvq_stream_t stream) {
    if (!gu || !y || inter <= 0) return fail(LLVQ_ERR_INVALID, "op_silu_mul: bad argument");
    CUDA_TRY(launch_dep(silu_mul_kernel, dim3((inter + 255) / 256), dim3(256), 0, (cudaStream_t)stream, (const __half*)gu, (__half*)y, inter));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_op_lm_head_argmax_h(const uint16_t* embed, const uint16_t* h, int32_t rows, int32_t hidden, int64_t row_offset,
                             void* scratch, float* val_out, int64_t* idx_out, llvq_stream_t stream) {
    if (!embed || !h || !scratch || !val_out || !idx_out || rows <= 0) return fail(LLVQ_ERR_INVALID, "op_lm_head_argmax: bad argument");
    if (hidden <= 0 || hidden % 8 || hidden > kHeadMaxHidden)
        return fail(LLVQ_ERR_UNSUPPORTED, "op_lm_head_argmax: hidden %d (a multiple of 8 up to %d)", hidden, kHeadMaxHidden);
    if (((uintptr_t)embed & 15u) || ((uintptr_t)h & 15u)) return fail(LLVQ_ERR_INVALID, "op_lm_head_argmax: buffers must be 16-byte aligned");
    int sms = 0, dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int grid = sms * 4;  // 32 warps per SM, each streaming one row at a time
    const int want = (rows + kHeadThreads / 32 - 1) / (kHeadThreads / 32);
    if (grid > want) grid = want;
    if (grid > kHeadMaxGrid) grid = kHeadMaxGrid;
    cudaStream_t s = (cudaStream_t)stream;
    CUDA_TRY(launch_dep(lm_head_argmax_kernel, dim3(grid), dim3(kHeadThreads), 0, s, (const __half*)embed, (const __half*)h, rows, hidden, (HeadBest*)scratch));
    CUDA_TRY(launch_dep(lm_head_pick_kernel, dim3(1), dim3(kHeadMaxGrid), 0, s, (const HeadBest*)scratch, grid, (long long)row_offset, val_out, (long long*)idx_out));
    g_launches += 2;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_op_lm_head_argmax_q8_h(const uint8_t* wq, const uint16_t* scales, const uint16_t* biases, const uint16_t* h, int32_t rows,
                                int32_t hidden, int64_t row_offset, void* scratch, float* val_out, int64_t* idx_out,
                                llvq_stream_t stream) {
    if (!wq || !scales || !biases || !h || !scratch || !val_out || !idx_out || rows <= 0)
        return fail(LLVQ_ERR_INVALID, "op_lm_head_argmax_q8: bad argument");
    if (hidden <= 0 || hidden % 64 || hidden > kHeadMaxHidden)
        return fail(LLVQ_ERR_UNSUPPORTED, "op_lm_head_argmax_q8: hidden %d (a multiple of 64 up to %d)", hidden, kHeadMaxHidden);
    if ((uintptr_t)wq & 15u) return fail(LLVQ_ERR_INVALID, "op_lm_head_argmax_q8: the codes must be 16-byte aligned");
    int sms = 0, dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int grid = sms * 4;
    const int want = (rows + kHeadThreads / 32 - 1) / (kHeadThreads / 32);
    if (grid > want) grid = want;
    if (grid > kHeadMaxGrid) grid = kHeadMaxGrid;
    cudaStream_t s = (cudaStream_t)stream;
    CUDA_TRY(launch_dep(lm_head_argmax_q8_kernel, dim3(grid), dim3(kHeadThreads), 0, s, wq, (const __half*)scales, (const __half*)biases, (const __half*)h, rows,
                                                           hidden, (HeadBest*)scratch));
    CUDA_TRY(launch_dep(lm_head_pick_kernel, dim3(1), dim3(kHeadMaxGrid), 0, s, (const HeadBest*)scratch, grid, (long long)row_offset, val_out, (long long*)idx_out));
    g_launches += 2;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_op_embed_gather_q8_h(const uint8_t* wq, const uint16_t* scales, const uint16_t* biases, const int64_t* ids, int32_t n_tokens,
                              int32_t rows, int32_t hidden, uint16_t* y, llvq_stream_t stream) {
    if (!wq || !scales || !biases || !ids || !y || n_tokens < 0 || rows <= 0 || hidden <= 0)
        return fail(LLVQ_ERR_INVALID, "op_embed_gather_q8: bad argument");
    if (n_tokens == 0) return LLVQ_OK;
    CUDA_TRY(launch_dep(embed_gather_q8_kernel, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, wq, (const __half*)scales, (const __half*)biases,
                                                                     (const long long*)ids, (__half*)y, hidden, rows));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_matrix_dequant_h(llvq_matrix* m, uint16_t* out, llvq_stream_t stream) {
    if (!m || !out) return fail(LLVQ_ERR_INVALID, "matrix_dequant_h: null argument");
    llvq_runtime* rt = m->rt;
    DeviceGuard g(rt->device);
    const MatrixView mv = m->view();
    const size_t items = (size_t)mv.d_out * (mv.nb + (mv.tail_w ? 1 : 0));
    if (items == 0) return LLVQ_OK;
    {
        int st = ensure_dyn_smem((const void*)dequant_dense_kernel, rt->TL.total_bytes);
        if (st) return st;
    }
    const size_t want = (items + kDenseThreads - 1) / kDenseThreads;
    const unsigned int grid = (unsigned int)(want < (size_t)(2 * rt->sm_count) ? want : (size_t)(2 * rt->sm_count));  // two CTAs per SM
    dequant_dense_kernel<<<grid, kDenseThreads, rt->TL.total_bytes, (cudaStream_t)stream>>>(
        (const unsigned char*)rt->d_tab_blob, (const OffEntry*)rt->d_tab_off, (const unsigned long long*)rt->d_tab_on3, rt->TL, mv,
        (__half*)out, rt->d_err);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

// ---- model container ------------------------------------------------------------------

namespace {
// points of the ball of shells 2..cap, from the class enumeration (built once, on the host)
const uint64_t* ball_sizes() {
    static uint64_t ball[16] = {0};
    static bool ready = false;
    if (!ready) {
        Codebook cb;
        for (const ClassInfo& c : cb.classes)
            for (int cap = c.shell; cap <= 13; ++cap) ball[cap] += c.card;
        ready = true;
    }
    return ball;
}

int archive_finish(std::unique_ptr<llvq_archive>& h, const std::string& err, llvq_archive** out) {
    if (!err.empty()) return fail(LLVQ_ERR_INVALID, "archive: %s", err.c_str());
    *out = h.release();
    return LLVQ_OK;
}
}  // namespace

int llvq_archive_open(const char* path, llvq_archive** out) {
    if (!path || !out) return fail(LLVQ_ERR_INVALID, "archive_open: null argument");
    std::unique_ptr<llvq_archive> h(new llvq_archive);
    const std::string err = open_archive(path, LLVQ_PUBLISHED_FINGERPRINT, ball_sizes(), h->a);
    return archive_finish(h, err, out);
}

int llvq_archive_open_memory(const void* data, size_t bytes, llvq_archive** out) {
    if (!data || !out) return fail(LLVQ_ERR_INVALID, "archive_open_memory: null argument");
    std::unique_ptr<llvq_archive> h(new llvq_archive);
    const std::string err = parse_archive((const unsigned char*)data, bytes, LLVQ_PUBLISHED_FINGERPRINT, ball_sizes(), h->a);
    return archive_finish(h, err, out);
}

void llvq_archive_close(llvq_archive* a) { delete a; }

int llvq_archive_counts(const llvq_archive* a, int32_t* version, int32_t* n_matrices, int32_t* n_raw, int32_t* n_blobs,
                        int32_t* has_fingerprint, uint64_t* fingerprint) {
    if (!a) return fail(LLVQ_ERR_INVALID, "archive_counts: null archive");
    if (version) *version = a->a.version;
    if (n_matrices) *n_matrices = (int32_t)a->a.matrices.size();
    if (n_raw) *n_raw = (int32_t)a->a.raws.size();
    if (n_blobs) *n_blobs = (int32_t)a->a.blobs.size();
    if (has_fingerprint) *has_fingerprint = a->a.has_fingerprint ? 1 : 0;
    if (fingerprint) *fingerprint = a->a.fingerprint;
    return LLVQ_OK;
}

int llvq_archive_matrix(const llvq_archive* a, int32_t i, llvq_archive_matrix_info* out) {
    if (!a || !out) return fail(LLVQ_ERR_INVALID, "archive_matrix: null argument");
    if (i < 0 || (size_t)i >= a->a.matrices.size()) return fail(LLVQ_ERR_INVALID, "archive_matrix: no matrix %d", i);
    const ArchiveMatrix& m = a->a.matrices[i];
    out->name = m.name.c_str();
    out->d_out = m.d_out;
    out->d_in = m.d_in;
    out->shell_cap = m.shell_cap;
    out->n_centroids = m.n_centroids;
    out->index_bits = m.index_bits;
    out->gain_bits = m.gain_bits;
    out->has_rotation = m.has_rotation ? 1 : 0;
    out->rotation_seed = m.rotation_seed;
    out->centroids = m.centroids.data();
    out->row_scales = m.row_scales.data();
    out->tail = m.tail.data();
    out->stream = m.stream;
    out->stream_bytes = m.stream_bytes;
    return LLVQ_OK;
}

int llvq_archive_matrix_desc(const llvq_archive* a, int32_t i, int32_t tail_mode, llvq_matrix_desc* out) {
    if (!a || !out) return fail(LLVQ_ERR_INVALID, "archive_matrix_desc: null argument");
    if (i < 0 || (size_t)i >= a->a.matrices.size()) return fail(LLVQ_ERR_INVALID, "archive_matrix_desc: no matrix %d", i);
    const ArchiveMatrix& m = a->a.matrices[i];
    // what the kernels read in place: 47-bit index + 1 gain bit = 6 bytes per block
    if (m.shell_cap != 12 || m.n_centroids != 2)
        return fail(LLVQ_ERR_UNSUPPORTED, "%s: shell cap %d with %d gain centroids; the kernels serve cap 12 with 2 (48-bit records)",
                    m.name.c_str(), m.shell_cap, m.n_centroids);
    out->d_out = m.d_out;
    out->d_in = m.d_in;
    out->shell_cap = m.shell_cap;
    out->tail_mode = tail_mode;
    out->codes = m.stream;
    out->centroids = m.centroids.data();
    out->row_scales = m.row_scales.data();
    out->tail = m.tail.data();
    return LLVQ_OK;
}

int llvq_archive_raw(const llvq_archive* a, int32_t i, llvq_archive_raw_info* out) {
    if (!a || !out) return fail(LLVQ_ERR_INVALID, "archive_raw: null argument");
    if (i < 0 || (size_t)i >= a->a.raws.size()) return fail(LLVQ_ERR_INVALID, "archive_raw: no raw tensor %d", i);
    const ArchiveRaw& t = a->a.raws[i];
    out->name = t.name.c_str();
    out->tag = t.tag;
    out->rank = (int32_t)t.dims.size();
    out->bits = t.bits;
    out->group = t.group;
    out->dims = t.dims.data();
    out->data = t.data;
    out->data_bytes = t.data_bytes;
    out->scales = t.scales;
    out->biases = t.biases;
    out->groups = t.groups;
    return LLVQ_OK;
}

int llvq_archive_blob(const llvq_archive* a, int32_t i, const char** name, const uint8_t** data, uint64_t* bytes) {
    if (!a) return fail(LLVQ_ERR_INVALID, "archive_blob: null archive");
    if (i < 0 || (size_t)i >= a->a.blobs.size()) return fail(LLVQ_ERR_INVALID, "archive_blob: no blob %d", i);
    const ArchiveBlob& b = a->a.blobs[i];
    if (name) *name = b.name.c_str();
    if (data) *data = b.data;
    if (bytes) *bytes = b.bytes;
    return LLVQ_OK;
}

// ---- activation rotation ------------------------------------------------------------

static int rotation_upload(llvq_runtime* rt, RotationTables&& t, llvq_rotation** out) {
    if (t.k > kRotMaxOdd)
        return fail(LLVQ_ERR_UNSUPPORTED, "rotation: width %d has the odd factor %d, beyond %d", t.n, t.k, kRotMaxOdd);
    const size_t smem = rot_smem_floats(t.n, t.k) * sizeof(float);
    if (smem > (size_t)rt->max_smem_optin)
        return fail(LLVQ_ERR_UNSUPPORTED, "rotation: width %d needs %zu bytes of shared memory, the device gives %d", t.n, smem,
                    rt->max_smem_optin);
    DeviceGuard g(rt->device);
    std::unique_ptr<llvq_rotation> r(new llvq_rotation);
    r->rt = rt;
    r->smem = smem;
    r->t = std::move(t);
    cudaError_t e = cudaMalloc((void**)&r->d_signbits, r->t.signbits.size() * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc((void**)&r->d_small, r->t.small.size() * sizeof(float));
    if (e == cudaSuccess)
        e = cudaMemcpy(r->d_signbits, r->t.signbits.data(), r->t.signbits.size() * sizeof(unsigned int), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(r->d_small, r->t.small.data(), r->t.small.size() * sizeof(float), cudaMemcpyHostToDevice);
    if (e == cudaSuccess && ensure_dyn_smem((const void*)rot_apply_kernel, smem) != LLVQ_OK) e = cudaErrorInvalidValue;
    if (e != cudaSuccess) {
        cudaFree(r->d_signbits);
        cudaFree(r->d_small);
        return fail(LLVQ_ERR_CUDA, "rotation upload: %s", cudaGetErrorString(e));
    }
    *out = r.release();
    return LLVQ_OK;
}

int llvq_rotation_create(llvq_runtime* rt, int32_t n, uint64_t seed, llvq_rotation** out) {
    if (!rt || !out || n <= 0) return fail(LLVQ_ERR_INVALID, "rotation_create: bad argument");
    return rotation_upload(rt, build_rotation(n, seed), out);
}

int llvq_rotation_create_from_tables(llvq_runtime* rt, int32_t n, const uint32_t* signbits, const float* small, llvq_rotation** out) {
    if (!rt || !out || n <= 0 || !signbits) return fail(LLVQ_ERR_INVALID, "rotation_create_from_tables: bad argument");
    RotationTables t;
    t.n = n;
    t.m = n & -n;
    t.k = n / t.m;
    if (t.k > 1 && !small) return fail(LLVQ_ERR_INVALID, "rotation_create_from_tables: width %d needs a %d x %d mix", n, t.k, t.k);
    if (t.k > kRotMaxOdd)
        return fail(LLVQ_ERR_UNSUPPORTED, "rotation: width %d has the odd factor %d, beyond %d", n, t.k, kRotMaxOdd);
    t.signbits.assign(signbits, signbits + ((size_t)n + 31) / 32);
    if (t.k > 1) t.small.assign(small, small + (size_t)t.k * t.k);
    else t.small.assign(1, 1.0f);
    t.inv = (float)(1.0 / std::sqrt((double)t.m));
    return rotation_upload(rt, std::move(t), out);
}

int llvq_rotation_build_tables(int32_t n, uint64_t seed, uint32_t* signbits, float* small, float* inv) {
    if (n <= 0) return fail(LLVQ_ERR_INVALID, "rotation_build_tables: width %d", n);
    const RotationTables t = build_rotation(n, seed);
    if (signbits) std::memcpy(signbits, t.signbits.data(), t.signbits.size() * sizeof(uint32_t));
    if (small) std::memcpy(small, t.small.data(), t.small.size() * sizeof(float));
    if (inv) *inv = t.inv;
    return LLVQ_OK;
}

void llvq_rotation_free(llvq_rotation* r) {
    if (!r) return;
    DeviceGuard g(r->rt->device);
    cudaFree(r->d_signbits);
    cudaFree(r->d_small);
    delete r;
}

int llvq_rotation_info(const llvq_rotation* r, int32_t* n, int32_t* m, int32_t* k, float* inv) {
    if (!r) return fail(LLVQ_ERR_INVALID, "rotation_info: null rotation");
    if (n) *n = r->t.n;
    if (m) *m = r->t.m;
    if (k) *k = r->t.k;
    if (inv) *inv = r->t.inv;
    return LLVQ_OK;
}

int llvq_rotation_tables(const llvq_rotation* r, uint32_t* signbits, float* small) {
    if (!r) return fail(LLVQ_ERR_INVALID, "rotation_tables: null rotation");
    if (signbits) std::memcpy(signbits, r->t.signbits.data(), r->t.signbits.size() * sizeof(uint32_t));
    if (small) std::memcpy(small, r->t.small.data(), r->t.small.size() * sizeof(float));
    return LLVQ_OK;
}

int llvq_rotate_h(llvq_rotation* r, const uint16_t* x, float* xr, int32_t batch, llvq_stream_t stream) {
    if (!r || !x || !xr || batch < 0) return fail(LLVQ_ERR_INVALID, "rotate_h: bad argument");
    if (batch == 0) return LLVQ_OK;
    if (((uintptr_t)x & 1u) || ((uintptr_t)xr & 3u)) return fail(LLVQ_ERR_INVALID, "rotate_h: misaligned buffer");
    DeviceGuard g(r->rt->device);
    CUDA_TRY(launch_dep(rot_apply_kernel, dim3(batch), dim3(kRotThreads), r->smem, (cudaStream_t)stream, (const __half*)x, r->d_signbits, r->d_small, xr, r->t.n,
                                                                        r->t.m, r->t.k, r->t.inv));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

static int rot_fused_prepare(llvq_rotation* r, int n, const char* who) {
    if (r->t.n != n) return fail(LLVQ_ERR_INVALID, "%s: the rotation is %d wide, the activation %d", who, r->t.n, n);
    int st = ensure_dyn_smem((const void*)add_rmsnorm_rotate_kernel, r->smem);
    if (!st) st = ensure_dyn_smem((const void*)silu_mul_rotate_kernel, r->smem);
    return st;
}

int llvq_op_add_rmsnorm_rotate_h(uint16_t* x, const uint16_t* delta, const uint16_t* w, llvq_rotation* r, float* xr, int32_t n,
                                 float eps, llvq_stream_t stream) {
    if (!x || !w || !r || !xr || n <= 0 || (n & 1) || n > 16384)
        return fail(LLVQ_ERR_INVALID, "op_add_rmsnorm_rotate: bad argument (n even, <= 16384)");
    DeviceGuard g(r->rt->device);
    int st = rot_fused_prepare(r, n, "op_add_rmsnorm_rotate");
    if (st) return st;
    CUDA_TRY(launch_dep(add_rmsnorm_rotate_kernel, dim3(1), dim3(kRotThreads), r->smem, (cudaStream_t)stream, 
        (__half*)x, (const __half*)delta, (const __half*)w, r->d_signbits, r->d_small, xr, n, r->t.m, r->t.k, r->t.inv, eps));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_op_silu_mul_rotate_h(const uint16_t* gu, llvq_rotation* r, float* xr, int32_t inter, llvq_stream_t stream) {
    if (!gu || !r || !xr || inter <= 0) return fail(LLVQ_ERR_INVALID, "op_silu_mul_rotate: bad argument");
    DeviceGuard g(r->rt->device);
    int st = rot_fused_prepare(r, inter, "op_silu_mul_rotate");
    if (st) return st;
    CUDA_TRY(launch_dep(silu_mul_rotate_kernel, dim3(1), dim3(kRotThreads), r->smem, (cudaStream_t)stream, (const __half*)gu, r->d_signbits, r->d_small, xr,
                                                                              inter, r->t.m, r->t.k, r->t.inv));
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

// ---- peer-memory all-gather of row shards (tensor-parallel token step) ----------------

int llvq_tp_region_create(int32_t device, size_t data_bytes, void** region, uint8_t* ipc_handle) {
    if (!region || !ipc_handle) return fail(LLVQ_ERR_INVALID, "tp_region_create: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == LLVQ_TP_HANDLE_BYTES, "IPC handle size");
    static_assert(kTpFlagBytes == LLVQ_TP_FLAG_BYTES, "flag area size");
    DeviceGuard g(device);
    void* p = nullptr;
    const size_t bytes = (size_t)kTpFlagBytes + data_bytes;
    CUDA_TRY(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(LLVQ_ERR_CUDA, "tp_region_create: %s", cudaGetErrorString(e));
    }
    std::memcpy(ipc_handle, &h, sizeof(h));
    *region = p;
    return LLVQ_OK;
}

int llvq_tp_region_open(int32_t device, const uint8_t* ipc_handle, void** region) {
    if (!region || !ipc_handle) return fail(LLVQ_ERR_INVALID, "tp_region_open: null argument");
    DeviceGuard g(device);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, ipc_handle, sizeof(h));
    CUDA_TRY(cudaIpcOpenMemHandle(region, h, cudaIpcMemLazyEnablePeerAccess));
    return LLVQ_OK;
}

int llvq_tp_region_close(int32_t device, void* region) {
    if (!region) return LLVQ_OK;
    DeviceGuard g(device);
    CUDA_TRY(cudaIpcCloseMemHandle(region));
    return LLVQ_OK;
}

int llvq_tp_region_free(int32_t device, void* region) {
    if (!region) return LLVQ_OK;
    DeviceGuard g(device);
    CUDA_TRY(cudaFree(region));
    return LLVQ_OK;
}

int llvq_tp_ctx_create(int32_t device, int32_t rank, int32_t world, void* const* regions, uint32_t spin_limit,
                       llvq_tp_ctx** out) {
    if (!regions || !out) return fail(LLVQ_ERR_INVALID, "tp_ctx_create: null argument");
    if (world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world)
        return fail(LLVQ_ERR_INVALID, "tp_ctx_create: rank %d of %d (at most %d ranks)", rank, world, kTpMaxWorld);
    for (int p = 0; p < world; ++p)
        if (!regions[p]) return fail(LLVQ_ERR_INVALID, "tp_ctx_create: region of rank %d is null", p);
    DeviceGuard g(device);
    std::unique_ptr<llvq_tp_ctx> c(new llvq_tp_ctx);
    c->device = device;
    c->r.rank = rank;
    c->r.world = world;
    c->r.spin_limit = spin_limit ? spin_limit : 4000000u;  // about a second of polling
    for (int p = 0; p < world; ++p) c->r.region[p] = (unsigned char*)regions[p];
    unsigned int* words = nullptr;
    CUDA_TRY(cudaMalloc((void**)&words, 2 * sizeof(unsigned int)));
    cudaError_t e = cudaMemset(words, 0, 2 * sizeof(unsigned int));
    if (e != cudaSuccess) {
        cudaFree(words);
        return fail(LLVQ_ERR_CUDA, "tp_ctx_create: %s", cudaGetErrorString(e));
    }
    c->r.seq = words;
    c->r.err = (int*)(words + 1);
    *out = c.release();
    return LLVQ_OK;
}

void llvq_tp_ctx_destroy(llvq_tp_ctx* c) {
    if (!c) return;
    DeviceGuard g(c->device);
    cudaFree(c->r.seq);
    delete c;
}

static int tp_fill_call(TpCall& call, const llvq_tp_ctx* c, int32_t site, size_t buf_offset, const void* src, uint32_t shard_bytes) {
    if (!c || !src) return fail(LLVQ_ERR_INVALID, "tp_exchange: null argument");
    if (site < 0 || site >= kTpMaxSites) return fail(LLVQ_ERR_INVALID, "tp_exchange: site %d (0..%d)", site, kTpMaxSites - 1);
    if (buf_offset < (size_t)kTpFlagBytes || buf_offset > 0xffffffffull)
        return fail(LLVQ_ERR_INVALID, "tp_exchange: buffer offset %zu lies inside the flag area or beyond 4 GiB", buf_offset);
    call.r = c->r;
    call.src = (const unsigned char*)src;
    call.shard_bytes = shard_bytes;
    call.buf_offset = (unsigned int)buf_offset;
    call.site = site;
    return LLVQ_OK;
}

int llvq_tp_exchange(llvq_tp_ctx* c, int32_t site, size_t buf_offset, const void* src, uint32_t shard_bytes,
                     llvq_stream_t stream) {
    TpCalls calls{};
    int st = tp_fill_call(calls.c[0], c, site, buf_offset, src, shard_bytes);
    if (st) return st;
    DeviceGuard g(c->device);
    CUDA_TRY(launch_dep(tp_exchange_kernel, dim3(1), dim3(32 * kTpMaxWorld), 0, (cudaStream_t)stream, calls));
    g_launches++;
    return LLVQ_OK;
}

int llvq_tp_exchange_emulated(llvq_tp_ctx* const* ctxs, int32_t n, int32_t site, size_t buf_offset, const void* const* srcs,
                              uint32_t shard_bytes, llvq_stream_t stream) {
    if (!ctxs || !srcs || n < 1 || n > kTpMaxWorld) return fail(LLVQ_ERR_INVALID, "tp_exchange_emulated: bad argument");
    TpCalls calls{};
    for (int i = 0; i < n; ++i) {
        int st = tp_fill_call(calls.c[i], ctxs[i], site, buf_offset, srcs[i], shard_bytes);
        if (st) return st;
        if (ctxs[i]->device != ctxs[0]->device) return fail(LLVQ_ERR_INVALID, "tp_exchange_emulated: ranks on several devices");
    }
    DeviceGuard g(ctxs[0]->device);
    // the CTAs wait on one another: a cooperative launch guarantees that all of them are resident
    void* args[] = {&calls};
    CUDA_TRY(cudaLaunchCooperativeKernel((const void*)tp_exchange_kernel, dim3(n), dim3(32 * kTpMaxWorld), args, 0,
                                         (cudaStream_t)stream));
    g_launches++;
    return LLVQ_OK;
}

int llvq_tp_poll_error(llvq_tp_ctx* c, int32_t* out) {
    if (!c || !out) return fail(LLVQ_ERR_INVALID, "tp_poll_error: null argument");
    DeviceGuard g(c->device);
    int v = 0;
    CUDA_TRY(cudaMemcpy(&v, c->r.err, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) CUDA_TRY(cudaMemset(c->r.err, 0, sizeof(int)));
    *out = v;
    return LLVQ_OK;
}

int llvq_gemv_h_host_many(const llvq_host_call* calls, int32_t n, llvq_stream_t stream) {
    if (!calls || n < 0) return fail(LLVQ_ERR_INVALID, "gemv_h_host_many: bad argument");
    if (n == 0) return LLVQ_OK;
    for (int i = 0; i < n; ++i)
        if (!calls[i].m || !calls[i].x_host || !calls[i].y_host || calls[i].m->rt != calls[0].m->rt)
            return fail(LLVQ_ERR_INVALID, "gemv_h_host_many: call %d has a null field or another runtime", i);
    DeviceGuard g(calls[0].m->rt->device);
    cudaStream_t s = (cudaStream_t)stream;
    // One pinned host buffer and one device buffer of the runtime carry the whole list. The list is cut into a few
    // segments: a segment's activations are packed on the host and go up in one copy on an upload stream while the
    // segment before it computes, its GEMVs run launch behind launch (each one's prologue overlapping the previous
    // one's tail), its results come back in one copy on a second copy stream while the next segment computes, and the
    // host scatters them as soon as they have landed. (A copy per call costs about 2 us of stream time each way; a
    // 252-projection token would spend more time in copies than in a fifth of its kernels.) The buffers grow on
    // demand; calls on one runtime take turns.
    llvq_runtime* rt = calls[0].m->rt;
    std::lock_guard<std::mutex> lock(rt->many_mu);
    std::vector<size_t> xo(n), yo(n);
    size_t at = 0;
    for (int i = 0; i < n; ++i) {
        xo[i] = at;
        at += ((size_t)calls[i].m->d_in * sizeof(__half) + 15) & ~(size_t)15;  // the kernels read x with 16-byte loads
    }
    const size_t x_bytes = at;
    for (int i = 0; i < n; ++i) {
        yo[i] = at;
        at += ((size_t)calls[i].m->d_out * sizeof(__half) + 15) & ~(size_t)15;
    }
    if (at > rt->many_bytes) {
        CUDA_TRY(cudaStreamSynchronize(s));
        cudaFreeHost(rt->many_host);
        cudaFree(rt->many_dev);
        rt->many_host = nullptr;
        rt->many_dev = nullptr;
        rt->many_bytes = 0;
        CUDA_TRY(cudaMallocHost((void**)&rt->many_host, at));
        CUDA_TRY(cudaMalloc((void**)&rt->many_dev, at));
        rt->many_bytes = at;
    }
    if (!rt->many_stream) {
        CUDA_TRY(cudaStreamCreateWithFlags(&rt->many_stream, cudaStreamNonBlocking));
        CUDA_TRY(cudaStreamCreateWithFlags(&rt->many_up, cudaStreamNonBlocking));
        for (int k = 0; k < kManySegments; ++k) {
            CUDA_TRY(cudaEventCreateWithFlags(&rt->many_ready[k], cudaEventDisableTiming));
            CUDA_TRY(cudaEventCreateWithFlags(&rt->many_in[k], cudaEventDisableTiming));
            CUDA_TRY(cudaEventCreateWithFlags(&rt->many_done[k], cudaEventDisableTiming));
        }
    }
    const int segs = n < kManySegments ? n : kManySegments;
    int first[kManySegments + 1];
    // short segments at both ends: what stands before the first kernel (one pack and copy) and behind the last one
    // (one copy and scatter) is a thirty-second of the list
    static const int kCut32[kManySegments + 1] = {0, 1, 4, 8, 16, 24, 28, 31, 32};
    for (int k = 0; k <= segs; ++k)  // both forms increase strictly: no empty segment
        first[k] = n >= 64 ? (int)((long long)n * kCut32[k] / 32) : (int)((long long)n * k / segs);
    // the staging buffers may still be read or written by what the caller's stream holds (an earlier call's kernels)
    CUDA_TRY(cudaEventRecord(rt->many_ready[0], s));
    CUDA_TRY(cudaStreamWaitEvent(rt->many_up, rt->many_ready[0], 0));
    for (int k = 0; k < segs; ++k) {
        // only the first segment's pack and copy stand before the first kernel
        for (int i = first[k]; i < first[k + 1]; ++i)
            std::memcpy(rt->many_host + xo[i], calls[i].x_host, (size_t)calls[i].m->d_in * sizeof(__half));
        const size_t xlo = xo[first[k]], xhi = first[k + 1] < n ? xo[first[k + 1]] : x_bytes;
        CUDA_TRY(cudaMemcpyAsync(rt->many_dev + xlo, rt->many_host + xlo, xhi - xlo, cudaMemcpyHostToDevice, rt->many_up));
        CUDA_TRY(cudaEventRecord(rt->many_in[k], rt->many_up));
        CUDA_TRY(cudaStreamWaitEvent(s, rt->many_in[k], 0));
        for (int i = first[k]; i < first[k + 1]; ++i) {
            int st = launch_gemv<__half, __half>(calls[i].m, (const __half*)(rt->many_dev + xo[i]), (__half*)(rt->many_dev + yo[i]), s);
            if (st) return st;
        }
        const size_t lo = yo[first[k]], hi = first[k + 1] < n ? yo[first[k + 1]] : at;
        CUDA_TRY(cudaEventRecord(rt->many_ready[k], s));
        CUDA_TRY(cudaStreamWaitEvent(rt->many_stream, rt->many_ready[k], 0));
        CUDA_TRY(cudaMemcpyAsync(rt->many_host + lo, rt->many_dev + lo, hi - lo, cudaMemcpyDeviceToHost, rt->many_stream));
        CUDA_TRY(cudaEventRecord(rt->many_done[k], rt->many_stream));
    }
    for (int k = 0; k < segs; ++k) {
        CUDA_TRY(cudaEventSynchronize(rt->many_done[k]));
        for (int i = first[k]; i < first[k + 1]; ++i)
            std::memcpy(calls[i].y_host, rt->many_host + yo[i], (size_t)calls[i].m->d_out * sizeof(__half));
    }
    // the caller's stream has nothing pending from this call; later work on it must also see the copy stream done
    CUDA_TRY(cudaStreamWaitEvent(s, rt->many_done[segs - 1], 0));
    return LLVQ_OK;
}

// ---- host-buffer GEMV that never allocates ---------------------------------
//
// Device staging for llvq_gemv_f32_host_static. The array lives in the module
// image, so every GPU that loads this library holds these bytes until the
// process exits; nothing is ever cudaMalloc'd for it. Layout: the activation
// first, then the result.
static __device__ __align__(256) float g_static_stage[LLVQ_STATIC_MAX_D_IN + LLVQ_STATIC_MAX_D_OUT];

namespace {
// In host code `g_static_stage` is only a handle; the device address has to be
// asked for, once per device, while that device is current.
// The slots are written without a lock: two threads making the first call on one device both
// store the same address, so the race is benign.
constexpr int kMaxDevices = 64;
float* g_static_ptr[kMaxDevices] = {nullptr};
}  // namespace

int llvq_gemv_f32_host_static(llvq_matrix* m, const float* x_host, float* y_host, llvq_stream_t stream) {
    if (!m || !x_host || !y_host) return fail(LLVQ_ERR_INVALID, "gemv_f32_host_static: null argument");
    if (m->d_in > LLVQ_STATIC_MAX_D_IN || m->d_out > LLVQ_STATIC_MAX_D_OUT)
        return fail(LLVQ_ERR_INVALID,
                    "gemv_f32_host_static: %d x %d exceeds the built-in staging area (d_out <= %d, d_in <= %d); use "
                    "llvq_gemv_f32_host",
                    m->d_out, m->d_in, LLVQ_STATIC_MAX_D_OUT, LLVQ_STATIC_MAX_D_IN);
    const int dev = m->rt->device;
    if (dev < 0 || dev >= kMaxDevices) return fail(LLVQ_ERR_INVALID, "gemv_f32_host_static: device %d", dev);
    DeviceGuard g(dev);
    if (!g_static_ptr[dev]) {  // first call on this device: resolve the symbol (do this before any stream capture)
        void* p = nullptr;
        CUDA_TRY(cudaGetSymbolAddress(&p, g_static_stage));
        g_static_ptr[dev] = static_cast<float*>(p);
    }
    float* xs = g_static_ptr[dev];
    float* ys = xs + LLVQ_STATIC_MAX_D_IN;
    cudaStream_t s = (cudaStream_t)stream;
    // Nothing in the staging area has to start at zero: x is copied in full and the kernel
    // stores every row of y. What the previous call left behind is simply overwritten.
    CUDA_TRY(cudaMemcpyAsync(xs, x_host, (size_t)m->d_in * sizeof(float), cudaMemcpyHostToDevice, s));
    int st = launch_gemv<float, float>(m, xs, ys, s);
    if (st) return st;
    CUDA_TRY(cudaMemcpyAsync(y_host, ys, (size_t)m->d_out * sizeof(float), cudaMemcpyDeviceToHost, s));
    CUDA_TRY(cudaStreamSynchronize(s));
    return LLVQ_OK;
}

int llvq_decode_blocks(llvq_runtime* rt, const uint8_t* codes, size_t n, int8_t* points, uint8_t* shell, uint8_t* gain,
                       llvq_stream_t stream) {
    if (!rt) return fail(LLVQ_ERR_INVALID, "decode_blocks: null runtime");
    if (n == 0) return LLVQ_OK;
    if (!codes || !points || !shell) return fail(LLVQ_ERR_INVALID, "decode_blocks: null argument");
    if (n > (size_t)1 << 36) return fail(LLVQ_ERR_INVALID, "decode_blocks: n too large");
    DeviceGuard g(rt->device);
    decode_blocks_kernel<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
        rt->T, codes, n, (signed char*)points, shell, gain, kN12);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_decode_blocks_fast(llvq_runtime* rt, const uint8_t* codes, size_t n, int8_t* points, uint8_t* shell, uint8_t* gain,
                            llvq_stream_t stream) {
    if (!rt) return fail(LLVQ_ERR_INVALID, "decode_blocks_fast: null runtime");
    if (n == 0) return LLVQ_OK;
    if (!codes || !points || !shell) return fail(LLVQ_ERR_INVALID, "decode_blocks_fast: null argument");
    if (n > (size_t)1 << 36) return fail(LLVQ_ERR_INVALID, "decode_blocks_fast: n too large");
    if ((uintptr_t)points & 7u) return fail(LLVQ_ERR_INVALID, "decode_blocks_fast: points must be 8-byte aligned");
    DeviceGuard g(rt->device);
    const size_t smem = rt->TL.total_bytes;
    int st = ensure_dyn_smem((const void*)llvq_decode_tab_kernel, smem);
    if (st) return st;
    // two CTAs per SM hold the tables; each walks a stride of the blocks
    const size_t want = (n + kProbeThreads - 1) / kProbeThreads;
    const unsigned grid = (unsigned)(want < (size_t)2 * rt->sm_count ? want : (size_t)2 * rt->sm_count);
    llvq_decode_tab_kernel<<<grid, kProbeThreads, smem, (cudaStream_t)stream>>>(
        (const unsigned char*)rt->d_tab_blob, (const OffEntry*)rt->d_tab_off, (const unsigned long long*)rt->d_tab_on3, rt->TL,
        codes, n, (signed char*)points, shell, gain);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

int llvq_decode_indices(llvq_runtime* rt, const uint64_t* idx, size_t n, int8_t* points, uint8_t* shell, llvq_stream_t stream) {
    if (!rt) return fail(LLVQ_ERR_INVALID, "decode_indices: null runtime");
    if (n == 0) return LLVQ_OK;
    if (!idx || !points || !shell) return fail(LLVQ_ERR_INVALID, "decode_indices: null argument");
    if (n > (size_t)1 << 36) return fail(LLVQ_ERR_INVALID, "decode_indices: n too large");
    DeviceGuard g(rt->device);
    decode_indices_kernel<<<(unsigned)((n + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
        rt->T, (const unsigned long long*)idx, n, (signed char*)points, shell, kN13);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return LLVQ_OK;
}

}  // extern "C"
