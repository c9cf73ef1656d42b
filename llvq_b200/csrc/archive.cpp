#include "archive.h"

#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace llvq {
namespace {

constexpr int kMaxShell = 13;  // llvq_search::classes::MAX_SHELL

// Cursor over the mapped bytes; every read says what it was reading when the bytes run out.
struct Cursor {
    const unsigned char* p;
    size_t left;
    std::string err;

    bool take(size_t n, const char* what, const unsigned char** out) {
        if (!err.empty()) return false;
        if (n > left) {
            err = std::string("truncated while reading ") + what;
            return false;
        }
        *out = p;
        p += n;
        left -= n;
        return true;
    }
    bool u32(const char* what, uint32_t* v) {
        const unsigned char* b;
        if (!take(4, what, &b)) return false;
        *v = (uint32_t)b[0] | (uint32_t)b[1] << 8 | (uint32_t)b[2] << 16 | (uint32_t)b[3] << 24;
        return true;
    }
    bool u64(const char* what, uint64_t* v) {
        const unsigned char* b;
        if (!take(8, what, &b)) return false;
        uint64_t x = 0;
        for (int i = 7; i >= 0; --i) x = x << 8 | b[i];
        *v = x;
        return true;
    }
    bool str(const char* what, std::string* s) {
        uint32_t n;
        const unsigned char* b;
        if (!u32(what, &n) || !take(n, what, &b)) return false;
        s->assign(reinterpret_cast<const char*>(b), n);
        return true;
    }
};

// ceil(log2(N(cap) + 1)), N(cap) = points of the ball of shells 2..cap (llvq-quant/src/quantizer.rs:572-576)
int index_bits_of(const uint64_t* ball, int shell_cap) {
    if (shell_cap < 2 || shell_cap > kMaxShell) return 0;
    int bits = 0;
    while ((1ull << bits) < ball[shell_cap] + 1) ++bits;
    return bits;
}

int gain_bits_of(uint32_t n_centroids) {
    int b = 0;
    while ((1u << b) < n_centroids) ++b;  // next_power_of_two().trailing_zeros()
    return b;
}

bool read_matrix(Cursor& c, const uint64_t* ball, ArchiveMatrix& m) {
    uint32_t d_out, d_in, cap, n_cent, has_rot;
    uint64_t seed;
    if (!c.str("name", &m.name) || !c.u32("d_out", &d_out) || !c.u32("d_in", &d_in) || !c.u32("shell cap", &cap)) return false;
    if (cap > (uint32_t)kMaxShell) {
        c.err = "inconsistent: " + m.name + ": shell cap " + std::to_string(cap) + " exceeds the supported ball (m <= 13)";
        return false;
    }
    if (!c.u32("centroid count", &n_cent) || !c.u64("rotation seed", &seed) || !c.u32("rotation flag", &has_rot)) return false;
    if (d_out > 0x7fffffffu || d_in > 0x7fffffffu) {
        c.err = "inconsistent: " + m.name + ": dimensions beyond 2^31";
        return false;
    }
    m.d_out = (int)d_out;
    m.d_in = (int)d_in;
    m.shell_cap = (int)cap;
    m.n_centroids = (int)n_cent;
    m.has_rotation = has_rot != 0;
    m.rotation_seed = seed;
    const unsigned char* b;
    if (!c.take((size_t)n_cent * 8, "centroids", &b)) return false;
    m.centroids.resize(n_cent);
    std::memcpy(m.centroids.data(), b, (size_t)n_cent * 8);  // little-endian f64 bits, as this host's
    if (!c.take((size_t)d_out * 8, "row scales", &b)) return false;
    m.row_scales.resize(d_out);
    std::memcpy(m.row_scales.data(), b, (size_t)d_out * 8);
    const uint64_t tail_n = (uint64_t)d_out * (d_in % 24);
    if (!c.take((size_t)tail_n * 4, "tail", &b)) return false;
    m.tail.resize((size_t)tail_n);
    std::memcpy(m.tail.data(), b, (size_t)tail_n * 4);
    uint64_t nbytes;
    if (!c.u64("code length", &nbytes) || !c.take((size_t)nbytes, "code stream", &m.stream)) return false;
    m.stream_bytes = nbytes;
    m.index_bits = index_bits_of(ball, (int)cap);
    m.gain_bits = gain_bits_of(n_cent);
    // the stream must hold every block the dimensions promise (format.rs:343-360)
    const unsigned __int128 need = (unsigned __int128)d_out * (d_in / 24) * (unsigned)(m.index_bits + m.gain_bits);
    if (need > (unsigned __int128)nbytes * 8) {
        c.err = "truncated while reading code stream";
        return false;
    }
    return true;
}

bool read_raw(Cursor& c, int version, ArchiveRaw& t) {
    uint32_t tag = 0, rank;
    if (version >= 3 && !c.u32("raw tensor tag", &tag)) return false;
    if (tag > 1) {
        c.err = "bad raw encoding: tag " + std::to_string(tag);
        return false;
    }
    t.tag = (int)tag;
    if (!c.str("raw tensor name", &t.name) || !c.u32("raw tensor rank", &rank)) return false;
    if (rank > 64) {
        c.err = "inconsistent: " + t.name + ": rank " + std::to_string(rank);
        return false;
    }
    t.dims.resize(rank);
    for (uint32_t i = 0; i < rank; ++i)
        if (!c.u64("raw tensor dims", &t.dims[i])) return false;
    if (tag == 0) {
        uint64_t n;
        if (!c.u64("raw tensor length", &n)) return false;
        if (n > (~0ull) / 2) {
            c.err = "truncated while reading raw tensor data";
            return false;
        }
        t.data_bytes = n * 2;
        return c.take((size_t)t.data_bytes, "raw tensor data", &t.data);
    }
    uint32_t bits, group;
    uint64_t nbytes, groups;
    if (!c.u32("quant width", &bits) || !c.u32("quant group", &group) || !c.u64("quant packed length", &nbytes)) return false;
    if (!c.take((size_t)nbytes, "quant packed data", &t.data) || !c.u64("quant group count", &groups)) return false;
    if (groups > (~0ull) / 2) {
        c.err = "truncated while reading quant scales";
        return false;
    }
    t.data_bytes = nbytes;
    t.bits = (int)bits;
    t.group = (int)group;
    t.groups = groups;
    return c.take((size_t)groups * 2, "quant scales", &t.scales) && c.take((size_t)groups * 2, "quant biases", &t.biases);
}

}  // namespace

Archive::~Archive() {
    if (map) munmap(map, map_bytes);
}

std::string parse_archive(const unsigned char* data, size_t bytes, uint64_t expected_fingerprint, const uint64_t* ball,
                          Archive& out) {
    Cursor c{data, bytes, {}};
    const unsigned char* magic;
    if (!c.take(4, "magic", &magic)) return c.err;
    if (magic[0] != 'L' || magic[1] != 'V' || magic[2] != 'Q' || magic[3] < '1' || magic[3] > '4')
        return "not an artifact: the file does not start with LVQ1..LVQ4";
    out.version = magic[3] - '0';
    uint32_t n_mat;
    if (!c.u32("matrix count", &n_mat)) return c.err;
    if (out.version >= 4) {
        if (!c.u64("codebook fingerprint", &out.fingerprint)) return c.err;
        out.has_fingerprint = true;
        if (out.fingerprint != expected_fingerprint) {
            char buf[128];
            std::snprintf(buf, sizeof buf, "codebook mismatch: the file was written with %016llx, this build decodes %016llx",
                          (unsigned long long)out.fingerprint, (unsigned long long)expected_fingerprint);
            return buf;
        }
    }
    for (uint32_t i = 0; i < n_mat; ++i) {
        out.matrices.emplace_back();
        if (!read_matrix(c, ball, out.matrices.back())) return c.err;
    }
    // a projections-only stream may simply end here (LVQ1); sealed files carry two more sections
    if (out.version == 1 && c.left == 0) return {};
    uint32_t n_raw, n_blob;
    if (!c.u32("raw tensor count", &n_raw)) return c.err;
    for (uint32_t i = 0; i < n_raw; ++i) {
        out.raws.emplace_back();
        if (!read_raw(c, out.version, out.raws.back())) return c.err;
    }
    if (!c.u32("blob count", &n_blob)) return c.err;
    for (uint32_t i = 0; i < n_blob; ++i) {
        out.blobs.emplace_back();
        ArchiveBlob& b = out.blobs.back();
        if (!c.str("blob name", &b.name) || !c.u64("blob length", &b.bytes) || !c.take((size_t)b.bytes, "blob", &b.data)) return c.err;
    }
    return {};
}

std::string open_archive(const char* path, uint64_t expected_fingerprint, const uint64_t* ball, Archive& out) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return std::string("cannot open ") + path;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        close(fd);
        return std::string("cannot stat ") + path + " (or it is empty)";
    }
    void* p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return std::string("cannot map ") + path;
    out.map = p;
    out.map_bytes = (size_t)st.st_size;
    return parse_archive(static_cast<const unsigned char*>(p), out.map_bytes, expected_fingerprint, ball, out);
}

}  // namespace llvq
