// Host shim: compiles the library's scalar decoders (the very source the CUDA
// kernels include) as plain C++ so the test-suite can run them without a GPU and
// diff them against the CPU oracle. The reference tests its kernels the same way
// (llvq-cuda/tests/host_shim.h, decoder_matches_rust.rs). Test-only.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../llvq_b200/csrc/codebook.cpp"
#include "../../llvq_b200/csrc/decode_generic.cuh"
#include "../../llvq_b200/csrc/tab_tables.cpp"
#include "../../llvq_b200/csrc/decode_tab.cuh"

using namespace llvq;

namespace {
struct HostTables {
    Codebook cb;
    std::vector<DevClass> cls;
    std::vector<uint16_t> lut;
    DevTables T;
    HostTables() {
        cb.dev_classes(cls);
        cb.class_lut(35, lut);
        T.cls = cls.data();
        T.ends = (const unsigned long long*)cb.ends.data();
        T.lut = lut.data();
        T.golay = cb.golay;
        T.lut_shift = 35;
    }
};
HostTables& tables() {
    static HostTables t;
    return t;
}
}  // namespace

extern "C" {

void shim_decode_indices(const uint64_t* idx, int64_t n, int8_t* points, uint8_t* shell, int cap) {
    const DevTables& T = tables().T;
    const unsigned long long limit = cap == 13 ? kN13 : kN12;
    for (int64_t b = 0; b < n; ++b) {
        int8_t* out = points + b * kDim;
        float scale;
        shell[b] = (uint8_t)decode_generic(T, idx[b], limit, [&](int pos, int val) { out[pos] = (int8_t)val; }, &scale);
    }
}

uint64_t shim_fingerprint(void) {
    HostTables& t = tables();
    std::vector<uint64_t> probes;
    probe_indices(t.cb, probes);
    std::vector<int8_t> pts(probes.size() * kDim);
    std::vector<uint8_t> shell(probes.size()), ok(probes.size());
    shim_decode_indices(probes.data(), (int64_t)probes.size(), pts.data(), shell.data(), 13);
    for (size_t i = 0; i < probes.size(); ++i) ok[i] = shell[i] != 255;
    return fingerprint_from_points(t.cb, probes, pts.data(), ok.data());
}

// The state-table decoders the fused GEMV and GEMM run: per index the 24 coordinates and the family
// (0 rare classes, 1 odd/state table, 2 odd/four kinds, 3 even; -1 origin, -2 refused).
void shim_decode_tab(const uint64_t* idx, int64_t n, int8_t* points, int8_t* fam, float* scale) {
    static TabTablesHost th;
    static TabView V;
    static bool ready = false;
    HostTables& t = tables();
    if (!ready) {
        build_tab_tables(t.cb, th);
        V.base = th.blob.data();
        V.lut_off = th.lut_off.data();
        V.lut_on3 = th.lut_on3.data();
        V.L = th.layout;
        ready = true;
    }
    for (int64_t b = 0; b < n; ++b) {
        unsigned int v[6];
        float s;
        fam[b] = (int8_t)tab_decode_any(V, idx[b], v, &s);
        std::memcpy(points + b * kDim, v, kDim);
        if (scale) scale[b] = s;
    }
}

// out: blob bytes, bytes classification needs, off-support entries, mass of the four families * 1e12,
// mass no decoder serves * 1e15, entries of the three-kind on-support table
void shim_tab_table_sizes(int64_t* out) {
    TabTablesHost th;
    build_tab_tables(tables().cb, th);
    out[0] = (int64_t)th.layout.total_bytes;
    out[1] = (int64_t)th.layout.classify_bytes;
    out[2] = (int64_t)th.lut_off.size();
    for (int f = 0; f < 4; ++f) out[3 + f] = (int64_t)(th.family_mass[f] * 1e12);
    out[7] = (int64_t)(th.slow_mass * 1e15);
    out[8] = (int64_t)th.lut_on3.size();
}

}  // extern "C"
