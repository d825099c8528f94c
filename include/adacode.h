/*
 * adacode.h — C ABI of the B200 (sm_100a) float11 KV-cache codec.
 *
 * float11 stores a bf16 tensor losslessly as
 *   - one sign/mantissa byte per element,
 *   - an n-bit exponent code per element (n in 1..4) against a window
 *     (left, right], left = right - 2**n + 1, eight codes forming one big-endian
 *     n-byte word with element 0 in the most significant bits,
 *   - an escape list holding the raw exponent of every element whose exponent
 *     is outside the window (code 0), in flat [b][h][s][d] order,
 *   - per (b,h) tile the inclusive running escape count ("tile base").
 * A "tile" is seq_tile consecutive tokens of one (batch, kv head): seq_tile*D
 * elements.  A "segment" is all B*H tiles of one seq_tile-token block.
 *
 * Conventions: every function returns 0 (ADACODE_OK) or a negative code, never
 * throws, never synchronises the device and never allocates device memory
 * unless stated.  All buffers belong to the caller.  `stream` is a
 * cudaStream_t passed as void*.  Device-side problems (escape capacity
 * exceeded, escape list too short) are reported by OR-ing bits into
 * *status (a device int32 the caller zeroes and reads when it wishes).
 *
 * Each entry point names the interface of the reference implementation
 * (lichangshiwhu/Adacode, paths relative to that project) that it replaces.
 */
#ifndef ADACODE_H_
#define ADACODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ADACODE_OK 0
#define ADACODE_ERR_INVALID_ARG (-1)
#define ADACODE_ERR_CUDA (-2)
#define ADACODE_ERR_WORKSPACE (-3)
#define ADACODE_ERR_NO_CANDIDATE (-4) /* adjuster: nothing beats 8 bits per exponent */
#define ADACODE_ERR_TOO_LARGE (-5)

/* bits OR-ed into the device status word */
#define ADACODE_STATUS_ESCAPE_OVERFLOW 1 /* pack: escapes_capacity too small, stream truncated */
#define ADACODE_STATUS_ESCAPE_UNDERRUN 2 /* unpack: a tile wanted an escape beyond n_escapes */
#define ADACODE_STATUS_TIMEOUT 4         /* a bounded on-chip wait gave up; results are invalid */
#define ADACODE_STATUS_MISALIGNED 8      /* a plane pointer inside a segment record is not 16-byte aligned */

/* Library version, major*10000 + minor*100 + patch. */
int adacode_version(void);

/* Text for a return code of this library. */
const char *adacode_strerror(int code);

/* Last CUDA runtime error string seen by this library on the calling thread
 * (valid after a call returned ADACODE_ERR_CUDA). */
const char *adacode_last_cuda_error(void);

/*
 * Bytes of scratch `adacode_pack_tiles` needs for a call that packs
 * n_tiles = B*H*n_blocks tiles of tile_elems = seq_tile*D elements.
 * The scratch must be zero-filled once when it is allocated; the library
 * leaves it ready for the next call.  Calls sharing one scratch buffer must
 * be ordered on one stream.
 */
size_t adacode_pack_workspace_bytes(int64_t n_tiles, int64_t tile_elems);

/*
 * Pack n_blocks consecutive seq_tile-token blocks of a bf16 tensor
 * src[B][H][n_blocks*seq_tile][D] (element strides stride_b/h/s, unit stride
 * along D) with one window.
 * Replaces: compress_tiled_tensor / _build_tiled_tensor
 *   (compress_tiled_kv.py:591-630, :524-588), which run
 *   CompressorBitMap.compress (compress_bitmap_merge.py:768-822):
 *   get_exp_mask_count_fused_kernel (:179-208), the boolean-mask gather and
 *   cumsum of get_invalid_index_values (:210-254) and compress{1,2,3,4}bit_vector
 *   (:256-420) once per block; and the pure-torch equivalent
 *   compress_open_tiled_rows + seal_open_tiled_rows (compress_tiled_kv.py:721-751,
 *   :633-718).
 *
 * Outputs are segment-major, i.e. block j owns
 *   sign_mant [j*B*H*tile_elems, (j+1)*B*H*tile_elems)            (sign_mass_data)
 *   codes     [j*B*H*tile_elems*nbits/8, ...)                     (exp_data)
 *   tile_base [j*B*H, (j+1)*B*H)   inclusive, restarting at every block (tile_invalid_base)
 *   escapes   [seg_escape_offsets[j], seg_escape_offsets[j+1])    (invalid_exp)
 * seg_escape_offsets has n_blocks+1 int64 entries, entry 0 is 0.
 * hist256 (nullable) receives += the 256-bin histogram of all exponents.
 * Requirements: D % 8 == 0, 1 <= nbits <= 4, 16-byte aligned src/sign_mant/codes,
 * strides multiples of 8, B*H*n_blocks*seq_tile*D < 2**31.
 */
int adacode_pack_tiles(const void *src_bf16, int64_t stride_b, int64_t stride_h, int64_t stride_s,
                       int B, int H, int n_blocks, int seq_tile, int D, int right, int nbits,
                       uint8_t *sign_mant, uint8_t *codes, uint8_t *escapes, int64_t escapes_capacity,
                       int32_t *tile_base, int64_t *seg_escape_offsets, int32_t *hist256,
                       void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * One tensor of a multi-tensor pack launch (adacode_pack_jobs): the arguments of
 * adacode_pack_tiles that may differ between the tensors of one call.
 */
typedef struct adacode_pack_job {
    const void *src_bf16;        /* [B][H][n_blocks*seq_tile][D], element strides below */
    int64_t stride_b, stride_h, stride_s;
    int32_t n_blocks;
    int32_t right;               /* window (right - 2**nbits + 1, right] */
    uint8_t *sign_mant;
    uint8_t *codes;
    uint8_t *escapes;
    int64_t escapes_capacity;
    int32_t *tile_base;
    int64_t *seg_escape_offsets; /* n_blocks + 1 entries */
    int32_t *hist256;            /* nullable */
} adacode_pack_job;

/* Largest n_jobs adacode_pack_jobs / adacode_unpack_jobs accept. */
int adacode_max_jobs(void);

/*
 * adacode_pack_tiles for up to adacode_max_jobs() tensors of one shape and code length in ONE
 * pack launch (plus one compaction launch): e.g. the keys and the values of a layer, each
 * with its own window, outputs and histogram.  `jobs` is host memory, read before the call
 * returns.  Every job's outputs are exactly what adacode_pack_tiles would write for it.
 * Replaces: the pair of compress_tiled_tensor calls per flushed block in
 *   float11Layer._compress_span (float_cache_utils.py:993-1011), i.e. two passes of
 *   CompressorBitMap.compress per 128 tokens, by one launch per prefill span.
 * The scratch must hold adacode_pack_workspace_bytes(total tiles of all jobs, seq_tile*D);
 * the elements of all jobs together must stay below 2**31.
 */
int adacode_pack_jobs(const adacode_pack_job *jobs, int n_jobs, int B, int H, int seq_tile, int D, int nbits,
                      void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * Maximum size of the library-owned scratch used by adacode_pack_tiles_static, in bytes.
 * A call fits when adacode_pack_workspace_bytes(n_tiles, tile_elems) is not larger (roughly
 * 4 Mi bf16 elements per call, e.g. thirty-two 128-token blocks of an [8, 128]-shaped head set).
 */
#define ADACODE_STATIC_SCRATCH_BYTES (4u * 1024u * 1024u + 512u * 1024u)

/*
 * adacode_pack_tiles for callers that cannot allocate device memory.
 * This entry point has no counterpart in the reference implementation.
 *
 * Some hosts of this library own no allocator at the moment they need to pack: a serving
 * process that carved up the whole GPU at start-up and treats every later cudaMalloc as a
 * fault (it stalls all streams of the device), or a plain C program that binds this library
 * without a tensor framework behind it.  For them the pack scratch (escape slots, per-tile
 * counts and the completion counter that the caller of adacode_pack_tiles must provide) lives
 * in a file-scope __device__ array of ADACODE_STATIC_SCRATCH_BYTES inside the library; every
 * GPU that loads the library holds that array until the process exits.  Inputs and outputs
 * are still the caller's.  Nothing is allocated or freed by this call.
 *
 * Limits and rules:
 *   - a call whose scratch need exceeds ADACODE_STATIC_SCRATCH_BYTES is rejected with
 *     ADACODE_ERR_WORKSPACE and does nothing; split the span into fewer blocks per call;
 *   - the first call on each device looks up the array's device address (with that device
 *     current); make that first call before any stream capture begins;
 *   - all calls on a device share the one array, which keeps what the previous call left:
 *     the call clears the part that must start at zero itself, on `stream`, but two calls
 *     whose kernels overlap on the GPU (different streams, no ordering) race on it.
 * Arguments and results are those of adacode_pack_tiles without workspace/workspace_bytes.
 */
int adacode_pack_tiles_static(const void *src_bf16, int64_t stride_b, int64_t stride_h, int64_t stride_s,
                              int B, int H, int n_blocks, int seq_tile, int D, int right, int nbits,
                              uint8_t *sign_mant, uint8_t *codes, uint8_t *escapes, int64_t escapes_capacity,
                              int32_t *tile_base, int64_t *seg_escape_offsets, int32_t *hist256,
                              int32_t *status, void *stream);

/*
 * Inverse of adacode_pack_tiles for planes laid out as that call writes them.
 * Replaces: TiledCompressedTensor.materialize / materialize_tiled_state /
 *   _decode_tiled_bf16_kernel (compress_tiled_kv.py:313-337, :754-791, :33-93),
 *   one launch for n_blocks segments instead of one per segment plus torch.cat.
 * Block j is written to dst[b][h][j*seq_tile + r][d] using the dst element strides.
 * seg_escape_offsets may be NULL when n_blocks == 1.  escapes_len bounds the reads.
 */
int adacode_unpack_tiles(const uint8_t *sign_mant, const uint8_t *codes, const uint8_t *escapes,
                         int64_t escapes_len, const int32_t *tile_base, const int64_t *seg_escape_offsets,
                         int B, int H, int n_blocks, int seq_tile, int D, int left, int nbits,
                         void *dst_bf16, int64_t dstride_b, int64_t dstride_h, int64_t dstride_s,
                         int32_t *status, void *stream);

/*
 * One packed segment as the cache stores it; an array of these in DEVICE memory
 * describes a whole layer (segments may differ in window and code length).
 */
typedef struct adacode_segment {
    const uint8_t *sign_mant; /* B*H*tile_elems bytes */
    const uint8_t *codes;     /* B*H*tile_elems*nbits/8 bytes */
    const uint8_t *escapes;   /* escapes_len bytes */
    const int32_t *tile_base; /* B*H inclusive counts */
    int64_t escapes_len;
    int64_t dst_seq_offset;   /* first token of this segment in dst */
    int32_t left;
    int32_t nbits;
} adacode_segment;

/*
 * Unpack n_segments segments described by a device array in one launch.
 * Replaces: float11Layer._materialize_prefix_segmented_tiled / _materialize_segments
 *   (float_cache_utils.py:1245-1264, :940-949): a Python loop of one decode launch
 *   per segment followed by torch.cat.
 */
int adacode_unpack_segments(const adacode_segment *segments_dev, int n_segments, int B, int H,
                            int seq_tile, int D, void *dst_bf16, int64_t dstride_b, int64_t dstride_h,
                            int64_t dstride_s, int32_t *status, void *stream);

/*
 * Testing aid for the failure path of the pipelined kernels; not needed in normal use.
 * Every on-chip wait of those kernels is bounded: after `polls` failed polls (0 restores the
 * default, 2**22) the waiter ORs ADACODE_STATUS_TIMEOUT into *status and carries on, so a launch
 * always ends.  With withhold_unit >= 0 the next adacode_unpack_* launches never signal that unit
 * (counted per CTA, CTA 0 only) as loaded and give it nothing to do, so that its wait runs out:
 * the call still returns, the status word says TIMEOUT, no memory outside the call's buffers is
 * touched.  -1 switches this off.  Process-wide, not thread-safe.
 * The reference implementation has no counterpart (its kernels never wait on one another).
 */
int adacode_debug_set_wait_limit(unsigned int polls, int withhold_unit);

/* One destination of a multi-tensor unpack launch (adacode_unpack_jobs). */
typedef struct adacode_unpack_job {
    const adacode_segment *segments_dev; /* device array, n_segments records */
    int32_t n_segments;
    int32_t reserved;
    void *dst_bf16;
    int64_t dstride_b, dstride_h, dstride_s;
} adacode_unpack_job;

/*
 * adacode_unpack_segments for up to adacode_max_jobs() destinations of one shape in one launch
 * (the keys and the values of a layer).  `jobs` is host memory, read before the call returns.
 * Replaces: the two _materialize_prefix_segmented_tiled passes (keys, values) of
 *   float11Layer.materialize_dense (float_cache_utils.py:1245-1290).
 */
int adacode_unpack_jobs(const adacode_unpack_job *jobs, int n_jobs, int B, int H, int seq_tile, int D,
                        int32_t *status, void *stream);

/* Elements per escape-base block of the flat layout for a code length: 128 * {8, 4, 8, 2}[nbits - 1]
 * (compress_bitmap_merge.py:653-657, invalid_block_size); 0 for an invalid nbits. */
int adacode_flat_block_elems(int nbits);

/*
 * Unpack a FLAT packed tensor: n_elems elements (a multiple of adacode_flat_block_elems(nbits)) with
 * one compact escape list and block_base[i] = number of escapes in blocks 0..i (inclusive).  The planes
 * are those adacode_pack_tiles writes for tiles of one block each, so a flat tensor is packed by calling
 * it with B = 1, H = n_elems / block, n_blocks = 1, seq_tile * D = block (tile_base is block_base).
 * Replaces: CompressorBitMap.uncompress / uncompress_with_weights and the
 *   uncompress{1,2,3,4}bit_vector_merge kernels (compress_bitmap_merge.py:423-597, :829-873), used by
 *   the 'legacy' cache layout (float_cache_utils.py:1219-1243) and by the weight hooks (manager.py:46-72).
 * Most of the tensor is decoded as 16384-element tiles that take their escape offset from every
 * (16384 / block)-th base.  Needs the pipelined kernels (not available with ADACODE_DISABLE_PIPELINE=1).
 */
int adacode_unpack_flat(const uint8_t *sign_mant, const uint8_t *codes, const uint8_t *escapes, int64_t escapes_len,
                        const int32_t *block_base, int64_t n_elems, int left, int nbits, void *dst_bf16,
                        int32_t *status, void *stream);

/*
 * hist256 += 256-bin histogram of the exponent field of src[B][H][S][D].
 * Replaces: float11Layer._extract_exponent_histogram (float_cache_utils.py:883-891)
 *   and the histogram half of get_exp_mask_count_fused_kernel
 *   (compress_bitmap_merge.py:205-208).
 */
int adacode_hist_bf16(const void *src_bf16, int64_t stride_b, int64_t stride_h, int64_t stride_s,
                      int B, int H, int S, int D, int32_t *hist256, void *stream);

/*
 * Code-length adjuster on the device: reads n_hists histograms (int32[256] each)
 * and writes (right, nbits) int32 pairs; nbits == 0 marks "no candidate".
 * Replaces: analysis_best_bits / _compute_adjusted_params
 *   (float_cache_utils.py:373-402), without the histogram .to('cpu') round trip.
 */
int adacode_choose_params(const int32_t *hist256_dev, int n_hists, int32_t *right_nbits_dev, void *stream);

/* The same rule on host memory (int64 histogram).  Returns ADACODE_ERR_NO_CANDIDATE
 * where the reference raises IndexError. */
int adacode_choose_params_host(const int64_t *hist256, int *right, int *nbits);

/*
 * Offline calibration rule on host memory: code lengths 1..8 with 2**n coded bins.
 * Replaces: analysis_best_bits_coo (best_bit_analysis_kv_cache.py:28-59), used by
 *   export_initial_compress_parameters (:191-204).
 */
int adacode_calibrate_host(const int64_t *hist256, int *right, int *nbits);

/*
 * Copy `bytes` (a multiple of 4, at most 1 MiB) from device memory into page-locked host memory
 * with a kernel, in stream order; the caller waits for an event recorded after it and reads the
 * host buffer.  dst must be pinned host memory that the current device can address (cudaHostAlloc /
 * cudaHostRegister under unified addressing): anything else is refused with
 * ADACODE_ERR_INVALID_ARG, nothing is launched.
 * Replaces: the small `.to('cpu')` / `.item()` reads of the reference's cache (escape totals of a
 *   freshly packed block, compress_tiled_kv.py:559-588; adjuster histograms,
 *   float_cache_utils.py:373, :883-891).  Those are cudaMemcpy calls: on a GPU whose copy engine is
 *   busy with bulk transfers (KV offload, prefill upload) each of them queues behind megabytes of
 *   unrelated traffic.  A kernel's stores to mapped memory do not use the copy engine.
 */
int adacode_copy_to_host(const void *src_dev, void *dst_host_pinned, size_t bytes, void *stream);

/*
 * Bytes of scratch adacode_decode_attn needs (split partials, fp32).  n_splits <= 0 sizes for
 * the largest split count the library will pick itself.
 */
size_t adacode_decode_attn_workspace_bytes(int B, int Hq, int D, int n_splits);

/*
 * Single-query ("decode step") attention computed straight from the packed cache:
 *   out[b][hq] = softmax(scale * q[b][hq] . K[b][hq / G]^T) V[b][hq / G],  G = Hq / Hkv,
 * where K and V are n_segments packed 128-token segments each (device arrays of segment
 * records in sequence order; dst_seq_offset is ignored) followed by tail_len dense bf16
 * tokens (the cache's not-yet-packed residual, element strides tail_stride_b/h/s, unit
 * stride along D).  Every cached token is visible to the query (no mask).  The planes are
 * decoded tile by tile in shared memory, so HBM sees the packed bytes only; the work is
 * split along the sequence into n_splits parts (<= 0: chosen by the library; at most 128)
 * whose partial results a second kernel merges.  A CTA serves up to eight query heads of a group;
 * larger groups (G > 8) are served by ceil(G / 8) CTAs that each decode the tiles again.
 * The reference implementation has no counterpart: its caches report
 *   decode_impl 'materialize_dense' (float_cache_utils.py:1342) and always rebuild dense K/V
 *   (float11Layer.update, :1278-1316) before the model's own attention runs; the module its
 *   validation script imports for a fused path (ops/kv_attention.py) is not in its tree.
 * Arithmetic: products and sums in fp32 (head_dim 128: bf16 x bf16 tensor-core products with
 * fp32 accumulation, probabilities rounded to bf16 for the weighted sum and its denominator
 * alike; head_dim 64: fp32 throughout), output rounded to bf16 (nearest even).  Requirements: seq_tile == 128, D in {64, 128}, q with unit stride
 * along D and element strides q_stride_b/h, out contiguous [B][Hq][D].
 */
int adacode_decode_attn(const void *q_bf16, int64_t q_stride_b, int64_t q_stride_h,
                        const adacode_segment *k_segments_dev, const adacode_segment *v_segments_dev, int n_segments,
                        const void *k_tail_bf16, const void *v_tail_bf16, int tail_len, int64_t tail_stride_b,
                        int64_t tail_stride_h, int64_t tail_stride_s, int B, int Hq, int Hkv, int seq_tile, int D,
                        float scale, void *out_bf16, void *workspace, size_t workspace_bytes, int n_splits,
                        int32_t *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ADACODE_H_ */
