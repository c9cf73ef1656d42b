// Reader of the reference's model container ("LVQ1".."LVQ4", llvq-artifact/src/format.rs and
// sealed.rs): header, the quantised matrices as undecoded records (read_matrix_raw,
// format.rs:301-382), then the raw tensors (embedding, norms; f16 or group-affine quantised) and the
// blobs (config.json, tokenizer.json). The file is mapped once; the code streams are used where
// they lie (a record's stream of 47-bit index + 1 gain bit per block IS the 6-byte-per-block layout
// the kernels read), the small f64/f32 side arrays are copied out because the file gives them no
// alignment. Every length field is checked against the bytes that are really there before it is used.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

namespace llvq {

struct ArchiveMatrix {
    std::string name;
    int d_out = 0, d_in = 0, shell_cap = 0, n_centroids = 0;
    bool has_rotation = false;
    uint64_t rotation_seed = 0;
    std::vector<double> centroids, row_scales;
    std::vector<float> tail;          // d_out * (d_in % 24), as stored (f32)
    const unsigned char* stream = nullptr;  // inside the mapped file
    uint64_t stream_bytes = 0;
    int index_bits = 0, gain_bits = 0;
};

struct ArchiveRaw {
    std::string name;
    std::vector<uint64_t> dims;
    int tag = 0;  // 0: f16 values; 1: group-affine quantised
    // f16: `data` = 2 * count bytes. quantised: `data` = packed values, then scales/biases (f16 each)
    const unsigned char* data = nullptr;
    uint64_t data_bytes = 0;
    int bits = 0, group = 0;
    const unsigned char* scales = nullptr;
    const unsigned char* biases = nullptr;
    uint64_t groups = 0;
};

struct ArchiveBlob {
    std::string name;
    const unsigned char* data = nullptr;
    uint64_t bytes = 0;
};

struct Archive {
    int version = 0;
    bool has_fingerprint = false;
    uint64_t fingerprint = 0;
    std::vector<ArchiveMatrix> matrices;
    std::vector<ArchiveRaw> raws;
    std::vector<ArchiveBlob> blobs;
    // the mapping (or nothing, for a caller-owned buffer)
    void* map = nullptr;
    size_t map_bytes = 0;
    ~Archive();
};

// Parses `bytes` bytes at `data` into `out`. Returns an empty string on success, else what was wrong
// (the reference's error kinds: not an artifact, truncated while reading X, inconsistent, bad raw
// encoding, unknown shell cap). `expected_fingerprint` is this build's codebook fingerprint: a file
// that carries another one is refused (read_header, format.rs:588-619). ball[cap] = points of the ball of
// shells 2..cap, cap = 2..13 (it sets the index width of a record).
std::string parse_archive(const unsigned char* data, size_t bytes, uint64_t expected_fingerprint, const uint64_t* ball,
                          Archive& out);

// Maps the file read-only and parses it.
std::string open_archive(const char* path, uint64_t expected_fingerprint, const uint64_t* ball, Archive& out);

}  // namespace llvq
