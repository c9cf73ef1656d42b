/*
 * llvq_b200 — C ABI of the B200 (sm_100a) fused Leech-lattice dequant-GEMV.
 *
 * A projection stays in HBM exactly as the `.llvq` archive stores it: one 48-bit
 * big-endian record per 24-weight block (47-bit index into the ball
 * Lambda24(12) u {0}, then 1 gain bit), row-major d_out x (d_in / 24), plus one
 * row scale per row, two gain centroids and d_in % 24 un-quantised tail columns.
 * The kernels decode every index in registers, bit-exactly as the reference's CPU
 * decoder does, and never materialise dense weights.
 *
 * Conventions shared by every entry point
 *   - returns LLVQ_OK (0) or a negative llvq_status; the message of the last
 *     failure on the calling thread is llvq_last_error(). Nothing aborts.
 *   - "dev" pointers are device memory of the runtime's GPU, "host" pointers are
 *     ordinary host memory. Output buffers are caller-allocated and may be
 *     uninitialised: every element is stored, never accumulated into.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream). Calls only enqueue work; they do not synchronise unless stated.
 *   - one host thread drives one runtime at a time (the reference launches from
 *     a single thread on a single stream, llvq-cuda/src/gpu.rs:243-272).
 *
 * Each declaration names the reference interface it stands in for (path:line in
 * pjmalandrino/llvq).
 */
#ifndef LLVQ_B200_H
#define LLVQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum llvq_status {
    LLVQ_OK = 0,
    LLVQ_ERR_INVALID = -1,     /* bad argument: null pointer, size, alignment, shell cap */
    LLVQ_ERR_CUDA = -2,        /* a CUDA runtime call failed; see llvq_last_error() */
    LLVQ_ERR_CODEBOOK = -3,    /* device tables do not reproduce the published codebook */
    LLVQ_ERR_RANGE = -4,       /* an index in the code stream lies outside the ball */
    LLVQ_ERR_UNSUPPORTED = -5  /* valid request this build does not serve */
} llvq_status;

typedef struct llvq_runtime llvq_runtime; /* per-GPU tables; FusedRuntime, llvq-llm/src/fused_cuda.rs:145 */
typedef struct llvq_matrix llvq_matrix;   /* one resident projection; FusedProj, llvq-llm/src/fused_cuda.rs:119 */
typedef void* llvq_stream_t;              /* cudaStream_t */

/* Published fingerprint of the v1 index map
 * (llvq-artifact/tests/codebook_fingerprint.rs:58). */
#define LLVQ_PUBLISHED_FINGERPRINT 0x338f420f11866319ull

/* Tail storage on the device. The reference's inference path narrows the tail
 * to binary16 once on the host (llvq-llm/src/fused.rs:655-659); its bench path
 * keeps f32 (llvq-cuda/kernels/matvec.cu:139-142). */
enum { LLVQ_TAIL_F32 = 0, LLVQ_TAIL_F16 = 1 };

/* One quantised matrix as the archive holds it: RawMatrix,
 * llvq-artifact/src/format.rs:215-229 (record layout format.rs:148-205). All
 * pointers are host memory and are copied; the caller keeps ownership. */
typedef struct llvq_matrix_desc {
    int32_t d_out;            /* rows */
    int32_t d_in;             /* columns; d_in / 24 blocks + d_in % 24 tail columns */
    int32_t shell_cap;        /* must be 12 (47-bit index); anything else is LLVQ_ERR_UNSUPPORTED */
    int32_t tail_mode;        /* LLVQ_TAIL_F32 or LLVQ_TAIL_F16 */
    const uint8_t* codes;     /* d_out * (d_in / 24) * 6 bytes, archive order, MSB-first */
    const double* centroids;  /* exactly 2 (one gain bit), ascending */
    const double* row_scales; /* d_out */
    const float* tail;        /* d_out * (d_in % 24), row-major; may be NULL when d_in % 24 == 0 */
} llvq_matrix_desc;

/* Message of the last failure on this thread ("" when none). Mirrors the
 * Result<_, String> every reference entry returns (llvq-llm/src/fused_cuda.rs:770-787). */
const char* llvq_last_error(void);

/* Library version, "major.minor.patch". */
const char* llvq_version(void);

/* ---- runtime ------------------------------------------------------------- */

/* Build the Golay, class and unranking tables on `device` and verify them
 * against LLVQ_PUBLISHED_FINGERPRINT by decoding the fingerprint's probe indices
 * on the GPU. Replaces FusedRuntime::new (llvq-llm/src/fused_cuda.rs:182-347)
 * minus its NVRTC step, and the header check of read_header
 * (llvq-artifact/src/format.rs:588-619). Synchronises. */
int llvq_runtime_create(int device, llvq_runtime** out);
void llvq_runtime_destroy(llvq_runtime* rt);

/* Fingerprint of the index map the device tables implement
 * (codebook_fingerprint, llvq-artifact/src/codebook.rs:129-185). */
int llvq_codebook_fingerprint(llvq_runtime* rt, uint64_t* out);

/* Class count and ball size of the cap-`shell_cap` codebook (12 or 13):
 * enumerate_classes / index_bits, llvq-search/src/classes.rs:144,
 * llvq-quant/src/quantizer.rs:572-576. */
int llvq_codebook_info(llvq_runtime* rt, int shell_cap, int32_t* n_classes, uint64_t* ball_size);

/* Host-only views of the index map, usable without a GPU. `ci` runs over the 383
 * classes in format order (the first 301 make the cap-12 ball); `out` receives
 * the 64-byte record the device decoders read (struct DevClass of
 * llvq_b200/csrc/codebook.h), the counterpart of CascadeClass,
 * llvq-search/src/fastdec.rs:89-133. llvq_codebook_golay copies the 4096
 * codewords in format order (Golay::codewords, llvq-core/src/golay.rs:99). */
int llvq_codebook_class_record(int32_t ci, void* out);
int llvq_codebook_golay(uint32_t* out);

/* Reads and clears the runtime's sticky range flag: *flag is 1 when any kernel
 * since the last poll met an index outside the ball (the reference surfaces this
 * as Error::IndexOutOfRange at load, llvq-artifact/src/format.rs:389-392).
 * Synchronises the device. */
/* Registers per thread, local-memory bytes per thread (0: no spill), static shared memory and binary
 * version of hot kernel `index` (0 .. until LLVQ_ERR_INVALID), read back with cudaFuncGetAttributes when
 * the runtime was created. llvq_runtime_create refuses to start if one of them spills, as the reference
 * does when it loads its kernels (llvq-cuda/src/gpu.rs:413-436, llvq-llm/src/fused_cuda.rs:229-239). */
int llvq_runtime_kernel_info(llvq_runtime* rt, int32_t index, const char** name, int32_t* regs, int32_t* local_bytes,
                             int32_t* static_smem_bytes, int32_t* binary_version);

/* Overlap of consecutive GEMV launches (on by default). The fused GEMV is launched with programmatic stream
 * serialisation: when the kernel before it in the stream is another fused GEMV, its CTAs take each SM as the
 * previous launch leaves it and bring the decoder tables and their first codes into shared memory before the
 * previous launch has finished; they wait for its completion before reading x or writing y. The code stream
 * and the tables of a matrix must therefore not be written by a kernel still running when a GEMV on it is
 * launched (llvq_matrix_upload and llvq_runtime_create synchronise, so this holds for everything this library
 * uploads). on = 0 gives ordinary launches. The reference has no counterpart: it pays 3.6 us per launch
 * (docs/mesures/a3-graph-2026-08-06.txt:6) or captures the token in a CUDA graph. */
int llvq_runtime_set_overlap(llvq_runtime* rt, int32_t on);

int llvq_runtime_poll_error(llvq_runtime* rt, int32_t* flag);

/* ---- matrices ------------------------------------------------------------ */

/* Copy one matrix to the GPU as stored (no transcode): upload_matrix,
 * llvq-llm/src/fused_cuda.rs:1058-1144. Synchronises. */
int llvq_matrix_upload(llvq_runtime* rt, const llvq_matrix_desc* desc, llvq_matrix** out);

/* Row-concatenate `n` matrices that share d_in (q|k|v or gate|up) into one
 * resident object served by one launch; every segment keeps its own centroid
 * pair. Same idea as tv_planes_seg, llvq-cuda/kernels/planes_seg.cu:65-133. */
int llvq_matrix_upload_group(llvq_runtime* rt, const llvq_matrix_desc* descs, int32_t n, llvq_matrix** out);

void llvq_matrix_free(llvq_matrix* m);
int llvq_matrix_dims(const llvq_matrix* m, int32_t* d_out, int32_t* d_in);


/* Bytes one GEMV must move at minimum: codes + tail + row scales (as stored in
 * the archive: f64) + x + y. Used by the benchmark's roofline. */
int llvq_matrix_algorithmic_bytes(const llvq_matrix* m, int32_t x_elem_bytes, int32_t y_elem_bytes, uint64_t* out);

/* ---- fused dequant-GEMV, device buffers ----------------------------------- */

/* y[d_out] = W x, f32 activation, f32 result: tv_slot / tv_planes,
 * llvq-cuda/kernels/matvec.cu:102, llvq-cuda/kernels/planes.cu:27. */
int llvq_gemv_f32(llvq_matrix* m, const float* x_dev, float* y_dev, llvq_stream_t stream);

/* f16 activation, f16 result (activations of the f16 model path). x_dev and
 * y_dev are IEEE binary16 passed as uint16_t. */
int llvq_gemv_h(llvq_matrix* m, const uint16_t* x_dev, uint16_t* y_dev, llvq_stream_t stream);

/* llvq_gemv_h with the activation produced inside the kernel, for the two places of a decode step where
 * a projection follows an elementwise step (Block::forward_cached, llvq-llm/src/model.rs:778-834):
 *   llvq_gemv_norm_h  y = W (RMSNorm(resid + delta) * norm_w); resid_out = resid + delta (delta may be
 *                     NULL; resid_out must not alias resid). Bit-identical to llvq_op_add_rmsnorm_h
 *                     followed by llvq_gemv_h. All vectors 16-byte aligned, d_in even, up to 16384.
 *   llvq_gemv_silu_h  y = W (silu(gate) * up), gate_up = [gate | up], d_in values each, d_in a
 *                     multiple of 8. Bit-identical to llvq_op_silu_mul_h followed by llvq_gemv_h.
 * LLVQ_ERR_UNSUPPORTED for a matrix the pipelined kernel does not serve (no whole block of 24 columns). */
int llvq_gemv_norm_h(llvq_matrix* m, const uint16_t* resid_dev, const uint16_t* delta_dev, const uint16_t* norm_w_dev, float eps,
                     uint16_t* resid_out_dev, uint16_t* y_dev, llvq_stream_t stream);
int llvq_gemv_silu_h(llvq_matrix* m, const uint16_t* gate_up_dev, uint16_t* y_dev, llvq_stream_t stream);

/* f32 (rotated) activation, f16 result: the exact signature of tv_planes_h,
 * llvq-llm/kernels/tv_planes_h.cu:38-72, which FusedRuntime::forward_rotated
 * launches (llvq-llm/src/fused_cuda.rs:384-402). */
int llvq_gemv_f32x_h(llvq_matrix* m, const float* x_dev, uint16_t* y_dev, llvq_stream_t stream);

/* ---- batched dequant-GEMM -------------------------------------------------- */

/* Y[B, d_out] = X[B, d_in] W^T for a batch of B activations (row-major, f16 in,
 * f16 out). The reference serves a batch as B serial matvec launches
 * (group_forward / drive_rows, llvq-llm/src/model.rs:497-536); here every code
 * is decoded once per batch. */
int llvq_gemm_h(llvq_matrix* m, const uint16_t* x_dev, uint16_t* y_dev, int32_t batch, llvq_stream_t stream);

/* ---- host-buffer convenience (what a plugin holding host tensors calls) ---- */

/* Same as llvq_gemv_f32 / llvq_gemv_h but x and y are host memory: the call
 * copies x in, launches, copies y out and synchronises the stream. */
int llvq_gemv_f32_host(llvq_matrix* m, const float* x_host, float* y_host, llvq_stream_t stream);
int llvq_gemv_h_host(llvq_matrix* m, const uint16_t* x_host, uint16_t* y_host, llvq_stream_t stream);

/* A whole list of host-buffer GEMVs (f16 in, f16 out) enqueued back to back with ONE
 * synchronisation at the end: what a layer or a token is for a plugin that holds host
 * tensors. The reference's loop also issues every launch of a token and synchronises once,
 * at the argmax read-back (llvq-llm/src/model.rs:1058-1072). The list is served in up to eight
 * segments (short ones at both ends): a segment's activations are packed into a pinned buffer
 * of the runtime and go up in one copy on an upload stream while the segment before computes,
 * its GEMVs run launch behind launch, and its results come back in one copy on a second copy
 * stream and are scattered into y_host while the next segment computes, before the call returns
 * (the buffers are sized by the first call and grow on demand; calls on one runtime take turns).
 * The calls of a list are independent: no call reads another call's result. */
typedef struct llvq_host_call {
    llvq_matrix* m;
    const uint16_t* x_host; /* d_in halves */
    uint16_t* y_host;       /* d_out halves */
} llvq_host_call;
int llvq_gemv_h_host_many(const llvq_host_call* calls, int32_t n, llvq_stream_t stream);

/* No counterpart in the reference. Same contract as llvq_gemv_f32_host, for
 * callers that must not cause a device allocation: code that runs while another
 * part of the process is capturing a CUDA graph (cudaMalloc is illegal there), or a
 * plugin hosted by a server whose device memory is handed out once at start-up and
 * audited afterwards. The device staging of x and y is a fixed array inside the
 * library image (LLVQ_STATIC_MAX_D_IN + LLVQ_STATIC_MAX_D_OUT floats, about 1.3 MB,
 * held by every GPU that loads the library until the process exits), so the call
 * performs no cudaMalloc/cudaFree, directly or through any library.
 *   - matrices larger than the two limits are refused with LLVQ_ERR_INVALID;
 *   - the first call on a device looks the array's address up; make that call
 *     before any stream capture begins;
 *   - all calls on one device share the array: two calls whose GPU work overlaps
 *     (different streams or threads) race on it. The array keeps whatever the last
 *     call left; nothing in it needs clearing because x is copied in whole and
 *     every row of y is stored before it is copied out.
 * Synchronises the stream, like llvq_gemv_f32_host. */
#define LLVQ_STATIC_MAX_D_IN 65536
#define LLVQ_STATIC_MAX_D_OUT 262144
int llvq_gemv_f32_host_static(llvq_matrix* m, const float* x_host, float* y_host, llvq_stream_t stream);

/* ---- the rest of a batch-1 decode step ------------------------------------- */

/* The non-projection steps of one Qwen3 block at batch 1, fused into four kernels; all tensors are
 * device memory, f16 passed as uint16_t, arithmetic in f32. The reference runs these steps as stock
 * candle ops (Block::forward_cached, llvq-llm/src/model.rs:778-834) and only simulates the int8 KV
 * cache (quantize_dequantize, llvq-llm/src/kvq.rs:110-165); here the cache stores the u8 codes with
 * an f16 scale and bias per group of 64 along head_dim ([capacity, n_kv, head_dim] codes,
 * [capacity, n_kv, head_dim / 64] scales and biases). `pos_dev` points at the int64 position of the
 * token in device memory, so a captured CUDA graph can be replayed for every token.
 * head_dim must be 64 or 128. */

/* x += delta (skipped when delta is NULL); y = x / rms(x) * w   (ln1 / ln2 / final norm + residual add) */
int llvq_op_add_rmsnorm_h(uint16_t* x_dev, const uint16_t* delta_dev, const uint16_t* w_dev, uint16_t* y_dev, int32_t n,
                          float eps, llvq_stream_t stream);
/* qkv = [q | k | v] of one token: per-head RMSNorm of q and k, RoPE (rotate-half; cos/sin tables
 * f32 [capacity, head_dim / 2]) at *pos_dev, q out; k and v quantised into the cache at *pos_dev. */
int llvq_op_qkv_rope_cache_h(const uint16_t* qkv_dev, const uint16_t* q_norm_dev, const uint16_t* k_norm_dev,
                             const float* cos_dev, const float* sin_dev, const int64_t* pos_dev, uint16_t* q_out_dev,
                             uint8_t* kq_dev, uint16_t* ks_dev, uint16_t* kb_dev, uint8_t* vq_dev, uint16_t* vs_dev,
                             uint16_t* vb_dev, int32_t n_heads, int32_t n_kv, int32_t head_dim, float eps,
                             llvq_stream_t stream);
/* softmax(q k^T / sqrt(head_dim)) v over positions 0..*pos_dev of the int8 cache, grouped-query heads.
 * Split-KV: the positions are cut into `splits` equal slices handled by separate CTAs and merged by a
 * second kernel (splits = 1: single pass, scratch may be NULL). scratch_dev: n_heads * splits *
 * (head_dim + 2) floats, caller-owned. */
int llvq_op_attn_decode_int8_h(const uint16_t* q_dev, const uint8_t* kq_dev, const uint16_t* ks_dev, const uint16_t* kb_dev,
                               const uint8_t* vq_dev, const uint16_t* vs_dev, const uint16_t* vb_dev,
                               const int64_t* pos_dev, uint16_t* out_dev, int32_t n_heads, int32_t n_kv, int32_t head_dim,
                               int32_t splits, float* scratch_dev, llvq_stream_t stream);
/* y[i] = silu(gate_up[i]) * gate_up[inter + i] */
int llvq_op_silu_mul_h(const uint16_t* gate_up_dev, uint16_t* y_dev, int32_t inter, llvq_stream_t stream);

/* Greedy head over a tied f16 embedding shard: logits = E[rows, hidden] h in f32, argmax with the
 * lowest row on ties; writes the best logit and row_offset + its row. The reference reads the
 * logits back and takes the argmax on the host (llvq-llm/src/model.rs:1041-1073). scratch_dev:
 * LLVQ_LM_HEAD_SCRATCH_BYTES of device memory, caller-owned. hidden: a multiple of 8 up to 8192. */
#define LLVQ_LM_HEAD_SCRATCH_BYTES 8192
int llvq_op_lm_head_argmax_h(const uint16_t* embed_dev, const uint16_t* h_dev, int32_t rows, int32_t hidden,
                             int64_t row_offset, void* scratch_dev, float* val_out_dev, int64_t* idx_out_dev,
                             llvq_stream_t stream);

/* The same head over an embedding carried as int8 g64 (w = scale * q + bias per group of 64 along the row,
 * f16 scale and bias, f32 multiply then add, not contracted): tv_q8_h of llvq-llm/kernels/emb_q8.cu:80-106,
 * with the argmax taken on the device. hidden: a multiple of 64 up to 8192; scales/biases [rows, hidden / 64]. */
int llvq_op_lm_head_argmax_q8_h(const uint8_t* wq_dev, const uint16_t* scales_dev, const uint16_t* biases_dev,
                                const uint16_t* h_dev, int32_t rows, int32_t hidden, int64_t row_offset, void* scratch_dev,
                                float* val_out_dev, int64_t* idx_out_dev, llvq_stream_t stream);
/* Token ids (int64, device) -> dequantised f16 rows [n_tokens, hidden]: emb_q8_gather (emb_q8.cu:53-66). */
int llvq_op_embed_gather_q8_h(const uint8_t* wq_dev, const uint16_t* scales_dev, const uint16_t* biases_dev,
                              const int64_t* ids_dev, int32_t n_tokens, int32_t rows, int32_t hidden, uint16_t* y_dev,
                              llvq_stream_t stream);

/* Write the matrix as dense f16 [d_out, d_in] (row-major, out_dev caller-owned): what the
 * reference's dense-decoded run keeps resident (llvq-llm/src/bin/fusedrun.rs:263-278), here a
 * transient operand for long-prompt GEMMs. An index outside the ball raises the runtime's range flag. */
int llvq_matrix_dequant_h(llvq_matrix* m, uint16_t* out_dev, llvq_stream_t stream);

/* ---- model container ----------------------------------------------------------
 * Reader of the reference's file format, "LVQ1".."LVQ4" (llvq-artifact/src/format.rs:301-382 for a
 * matrix record, :588-619 for the header, src/sealed.rs:224-343 for raw tensors and blobs). The file is
 * mapped read-only; a matrix's code stream is used where it lies (47-bit index + 1 gain bit per block
 * is the 6-byte record the kernels read), so llvq_archive_matrix_desc + llvq_matrix_upload load a
 * projection without decoding or re-packing anything. Needs no GPU. A version-4 file whose codebook
 * fingerprint is not 0x338f420f11866319 is refused; every length field is checked against the bytes
 * present. Pointers handed out stay valid until llvq_archive_close. */
typedef struct llvq_archive llvq_archive;
typedef struct {
    const char* name;
    int32_t d_out, d_in, shell_cap, n_centroids, index_bits, gain_bits, has_rotation;
    uint64_t rotation_seed;
    const double* centroids;  /* n_centroids */
    const double* row_scales; /* d_out */
    const float* tail;        /* d_out * (d_in % 24), as stored */
    const uint8_t* stream;    /* (index_bits + gain_bits) bits per block, MSB first, row-major blocks */
    uint64_t stream_bytes;
} llvq_archive_matrix_info;
typedef struct {
    const char* name;
    int32_t tag; /* 0: f16 values (data = 2 bytes each); 1: group-affine quantised (w = scale q + bias) */
    int32_t rank, bits, group;
    const uint64_t* dims;
    const uint8_t* data; /* unaligned: copy before reinterpreting */
    uint64_t data_bytes;
    const uint8_t* scales; /* tag 1: `groups` f16 values each */
    const uint8_t* biases;
    uint64_t groups;
} llvq_archive_raw_info;

int llvq_archive_open(const char* path, llvq_archive** out);
/* The same over bytes the caller keeps alive until close. */
int llvq_archive_open_memory(const void* data, size_t bytes, llvq_archive** out);
void llvq_archive_close(llvq_archive* a);
int llvq_archive_counts(const llvq_archive* a, int32_t* version, int32_t* n_matrices, int32_t* n_raw, int32_t* n_blobs,
                        int32_t* has_fingerprint, uint64_t* fingerprint);
int llvq_archive_matrix(const llvq_archive* a, int32_t i, llvq_archive_matrix_info* out);
/* Fill an upload descriptor that points into the archive; refuses records the kernels do not serve
 * (shell cap other than 12, other than 2 gain centroids) with LLVQ_ERR_UNSUPPORTED. */
int llvq_archive_matrix_desc(const llvq_archive* a, int32_t i, int32_t tail_mode, llvq_matrix_desc* out);
int llvq_archive_raw(const llvq_archive* a, int32_t i, llvq_archive_raw_info* out);
int llvq_archive_blob(const llvq_archive* a, int32_t i, const char** name, const uint8_t** data, uint64_t* bytes);

/* ---- activation rotation ------------------------------------------------------
 * Every sealed matrix was quantised in a rotated basis, Q = (Q_odd (x) H_m) D built from its
 * rotation seed (llvq-quant/src/rotation.rs:51-68); the runtime rotates the activation once per
 * shared input and feeds the f32 result to llvq_gemv_f32x_h. This replaces FusedRuntime::rotate /
 * the rot_apply kernel (llvq-llm/src/fused_cuda.rs:362-379, llvq-cuda/kernels/rotate.cu:38-67) and
 * RotationTables::build (llvq-llm/src/fused.rs:678-725). Odd factors up to 32, as the reference. */
typedef struct llvq_rotation llvq_rotation;
/* Build the tables from (width, seed) on the host and upload them. */
int llvq_rotation_create(llvq_runtime* rt, int32_t n, uint64_t seed, llvq_rotation** out);
/* The same from tables the caller already holds: signbits = ceil(n / 32) words, bit i & 31 of word
 * i >> 5 set = negative; small = Q_odd, k x k row-major f32 (k = n / largest power of two in n; may be
 * NULL when k = 1). */
int llvq_rotation_create_from_tables(llvq_runtime* rt, int32_t n, const uint32_t* signbits, const float* small,
                                     llvq_rotation** out);
/* Host only (no GPU needed): the tables of (width, seed) into caller buffers of ceil(n / 32) words and
 * k * k floats (either may be NULL), and 1 / sqrt(m). */
int llvq_rotation_build_tables(int32_t n, uint64_t seed, uint32_t* signbits_out, float* small_out, float* inv_sqrt_m_out);
void llvq_rotation_free(llvq_rotation* rot);
int llvq_rotation_info(const llvq_rotation* rot, int32_t* n, int32_t* m, int32_t* k, float* inv_sqrt_m);
/* Copy the host tables out (either pointer may be NULL): ceil(n / 32) words, k * k floats. */
int llvq_rotation_tables(const llvq_rotation* rot, uint32_t* signbits_out, float* small_out);
/* x' = Q x for `batch` activations: f16 [batch, n] in, f32 [batch, n] out, both device memory, one
 * launch (one CTA per activation). */
int llvq_rotate_h(llvq_rotation* rot, const uint16_t* x_dev, float* xr_dev, int32_t batch, llvq_stream_t stream);

/* The two decode-step kernels that feed a rotated projection group, with the rotation folded in (the
 * normalised / gated activation keeps its f16 rounding, so the f32 result equals the two-kernel
 * sequence bit for bit): x += delta; xr = Q f16(x / rms(x) * w), and xr = Q f16(silu(gate) * up). */
int llvq_op_add_rmsnorm_rotate_h(uint16_t* x_dev, const uint16_t* delta_dev, const uint16_t* w_dev, llvq_rotation* rot,
                                 float* xr_dev, int32_t n, float eps, llvq_stream_t stream);
int llvq_op_silu_mul_rotate_h(const uint16_t* gate_up_dev, llvq_rotation* rot, float* xr_dev, int32_t inter,
                              llvq_stream_t stream);

/* ---- peer-memory all-gather of row shards (tensor-parallel token step) -------
 * No counterpart in the reference, which is single-GPU. A rank owns one region =
 * LLVQ_TP_FLAG_BYTES of flags followed by its gather buffers, maps the regions of its peers
 * through CUDA IPC, and llvq_tp_exchange copies its shard into every rank's buffer with peer
 * stores, releases a flag on each peer and waits (bounded) for the peers' flags in its own
 * region. All ranks must issue the same sequence of exchanges. */
#define LLVQ_TP_FLAG_BYTES 512
#define LLVQ_TP_HANDLE_BYTES 64
#define LLVQ_TP_ERR_PEER_TIMEOUT 4 /* bit of the error word: a peer's flag did not arrive in time */
typedef struct llvq_tp_ctx llvq_tp_ctx;

/* cudaMalloc + zero a region of LLVQ_TP_FLAG_BYTES + data_bytes; ipc_handle_out: LLVQ_TP_HANDLE_BYTES
 * to hand to the peers (any transport). */
int llvq_tp_region_create(int32_t device, size_t data_bytes, void** region_out, uint8_t* ipc_handle_out);
int llvq_tp_region_open(int32_t device, const uint8_t* ipc_handle, void** region_out); /* a peer's region */
int llvq_tp_region_close(int32_t device, void* peer_region);
int llvq_tp_region_free(int32_t device, void* own_region);
/* regions[p]: the region of rank p as mapped in this process (own region at index rank).
 * spin_limit: polls before a wait gives up (0 = default, about a second). */
int llvq_tp_ctx_create(int32_t device, int32_t rank, int32_t world, void* const* regions, uint32_t spin_limit,
                       llvq_tp_ctx** out);
void llvq_tp_ctx_destroy(llvq_tp_ctx* ctx);
/* Gather: afterwards the buffer at region + buf_offset holds world shards of shard_bytes in rank
 * order. site (0..15) names the flag row; reuse a site only for exchanges at least two apart. */
int llvq_tp_exchange(llvq_tp_ctx* ctx, int32_t site, size_t buf_offset, const void* src_dev, uint32_t shard_bytes,
                     llvq_stream_t stream);
/* The same exchange for n ranks whose regions all live on one GPU, as ONE cooperative launch
 * (ranks that wait on one another must not be separate launches on one GPU). For tests. */
int llvq_tp_exchange_emulated(llvq_tp_ctx* const* ctxs, int32_t n, int32_t site, size_t buf_offset,
                              const void* const* srcs_dev, uint32_t shard_bytes, llvq_stream_t stream);
/* Read and clear the error word (synchronises the device). */
int llvq_tp_poll_error(llvq_tp_ctx* ctx, int32_t* out);

/* ---- attribution probes ---------------------------------------------------- */

/* llvq_gemv_h with parts of the kernel left out, for timing what the rest costs: the reference's
 * "floor" kernels (llvq-cuda/kernels/nullk.cu:61: same grid, staging and reduction, no weights;
 * llvq-cuda/kernels/llvq_floor.cuh:133-135: stream only / + table / + shared-memory reads).
 * mode is a bit set: 0 = the full kernel; bit 0 = no decoders (records are read and classified,
 * activations staged, rows summed and stored); bit 1 = no class search (records are only read);
 * bit 2 = no decode batches at all (0 to 7). y is NOT the product for mode > 0. */
int llvq_gemv_probe_h(llvq_matrix* m, const uint16_t* x_dev, uint16_t* y_dev, int32_t mode, llvq_stream_t stream);

/* One launch of the f16 GEMV kernel (mode as in llvq_gemv_probe_h) with time stamps: for each of
 * the first max_ctas CTAs, 64 uint64 nanosecond readings of the GPU's global timer taken by thread 0
 * (first warp group): [0] kernel entry, [1] classification tables landed and first tile staged, then
 * three readings per tile of that group: [2 + 3 i] end of its classification phase, [3 + 3 i] end of
 * its decode phase, [4 + 3 i] end of its row sums; 0 where an event did not occur. The per-phase timing
 * the reference prints for a token (generate_phased, llvq-llm/src/model.rs:1116-1163), at the scale
 * of one kernel. Allocates and frees a device buffer; synchronises the stream. */
#define LLVQ_TRACE_EVENTS 64
int llvq_gemv_trace_h(llvq_matrix* m, const uint16_t* x_dev, uint16_t* y_dev, int32_t mode, uint64_t* trace_host,
                      int32_t max_ctas, int32_t* n_ctas, llvq_stream_t stream);

/* ---- decode probes --------------------------------------------------------- */

/* Decode n packed 6-byte records on the GPU to their lattice points: 24 int8
 * per block, the shell m (||p||^2 = 16 m; 0 for the origin, 255 for an index
 * outside the ball) and the gain bit. The integer dump the reference's
 * preflight uses to diff a kernel against the Rust decoder
 * (llvq-cuda/kernels/preflight.cu:28-60). All pointers are device memory. */
int llvq_decode_blocks(llvq_runtime* rt, const uint8_t* codes_dev, size_t n, int8_t* points_dev,
                       uint8_t* shell_dev, uint8_t* gain_dev, llvq_stream_t stream);

/* The same dump through the decoders the fused GEMV and GEMM kernels run (class search and
 * the state-table / arrangement-table family decoders, tables in shared memory), so that
 * their integer output can be diffed block by block on the device
 * (llvq-cuda/kernels/preflight.cu:39-60, decode_probe). Cap-12 ball only; points_dev
 * must be 8-byte aligned. */
int llvq_decode_blocks_fast(llvq_runtime* rt, const uint8_t* codes_dev, size_t n, int8_t* points_dev,
                            uint8_t* shell_dev, uint8_t* gain_dev, llvq_stream_t stream);

/* Decode n raw indices (up to the cap-13 ball, 48 bits) on the GPU:
 * Indexer::decode, llvq-search/src/index.rs:334-435. shell_dev as above. */
int llvq_decode_indices(llvq_runtime* rt, const uint64_t* idx_dev, size_t n, int8_t* points_dev,
                        uint8_t* shell_dev, llvq_stream_t stream);

/* Number of kernels this library has launched on the calling process so far
 * (all runtimes). The benchmark reports the difference across its timed region. */
uint64_t llvq_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* LLVQ_B200_H */
