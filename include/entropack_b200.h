/*
 * entropack_b200 -- C ABI of the B200 (sm_100a) kernels behind the entropack compression hot path.
 *
 * One shared object, plain pointers and sizes, no framework types. Every entry point is what a
 * backend "lane" module of the reference would bind (the reference launches its kernels from Python
 * through raw device pointers, entropack/backends/cuda/kernels.py:31-62); each declaration names the
 * reference interface it stands in for.
 *
 * Conventions
 *  - Pointers named *_dev are device pointers on the current CUDA device; *_host are host pointers.
 *    Device buffers need the 16-byte alignment the container format guarantees
 *    (entropack/compression/compressed_tensor.py:13-14) unless a comment asks for less.
 *  - The caller owns every allocation. Nothing here allocates device memory.
 *  - Calls are asynchronous on `stream` (a cudaStream_t passed as void*) unless stated otherwise.
 *  - Return value: EP_OK or a negative EP_ERR_* code; ep_status_string() names it. Kernels never
 *    trap: a malformed bitstream is reported through the optional `error_dev` word (device int32,
 *    zero-initialised by the caller, first non-zero code wins) and the offending tile is skipped.
 */
#ifndef ENTROPACK_B200_H
#define ENTROPACK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define EP_OK 0
#define EP_ERR_INVALID_ARGUMENT (-1)
#define EP_ERR_UNSUPPORTED (-2)
#define EP_ERR_CUDA (-3)
#define EP_ERR_NORMALIZE (-4)
#define EP_ERR_ALPHABET (-5)
#define EP_ERR_TOO_LARGE (-6)
/* not an error: the call stopped because a caller-sized buffer is too small; the size it needs is in an output argument */
#define EP_MORE_BINS 1

/* codes written to error_dev by decode kernels */
#define EP_STREAM_BAD_OFFSETS 1
#define EP_STREAM_UNDERRUN 2
#define EP_STREAM_NOT_CONSUMED 3
#define EP_STREAM_BAD_RAW_LENGTH 4
#define EP_STREAM_BAD_SYMBOL 5   /* a decoded symbol that selects a table lies outside the tables (lossy: a coset above 1) */
#define EP_KERNEL_TIMEOUT 9      /* a bounded wait inside a tensor-core product ran out; its output is incomplete */

typedef void* ep_stream_t;

const char* ep_status_string(int status);
/* ABI version of this header; bumped on any signature change. */
int ep_abi_version(void);
/* Last CUDA runtime error text seen by this library on the calling thread (for EP_ERR_CUDA). */
const char* ep_last_cuda_error(void);
/* How many SMs the calling thread's next launches of ep_lattice_decode (decode_sms) and of the tensor-core products
 * ep_linear_forward / _fp8 / _int8 (product_sms) may fill; 0 lifts a limit. Both kernels are persistent, one block (or
 * block pair) to an SM, and each needs most of an SM's shared memory, so two of them share the GPU only side by side:
 * a caller that decodes the next layer's weight on a second stream while the current layer's product runs gives the
 * decode 52 SMs and the product 96 (what entropack_b200.linear.DecodeAhead does). No reference counterpart: the
 * reference decodes and multiplies one after the other (entropack/linear/linear.py:163-165). */
int ep_set_sm_limits(int decode_sms, int product_sms);

/* ---------------------------------------------------------------------------------------------
 * Tile-ANS (lossless, byte-lane rANS).  Buffer schema: entropack/schemes/tile_ans/format.py:58-64.
 * ------------------------------------------------------------------------------------------- */

/* Decode a Tile-ANS container into `output_dev` (num_elements * num_lanes bytes, whole elements are
 * written with one store each). Stands in for decode() of entropack/schemes/tile_ans/cuda.py:122-170
 * and the four kernels it picks from (tile_ans.cu:175-469). `lane_modes_host` is the container's
 * lane_modes buffer copied to the host (0 = ANS, 1 = raw), as the reference caches it.
 * `payload_words` is the length of `payload_dev` and bounds every read. */
int ep_tile_ans_decode(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                       const uint32_t* states_dev, const uint32_t* decode_tables_dev, const uint8_t* lane_modes_host,
                       void* output_dev, int64_t num_elements, int64_t tile_elements, int prob_bits, int num_lanes,
                       int* error_dev, ep_stream_t stream);

/* The same decode for tiles [first_tile, first_tile + tile_count) only: it reads those tiles' streams
 * (stream = lane * tiles + tile, as in tile_ans.cu:175-469) and writes their elements at their places in
 * `output_dev`, which is still the whole tensor's buffer. Tiles are independent given the tables, so a
 * caller that streams a container in from the host can decode and send back each range as soon as its
 * payload bytes have arrived; offsets, states and tables must be resident in full. No reference
 * counterpart (its decode() always launches over every tile). */
int ep_tile_ans_decode_tiles(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                             const uint32_t* states_dev, const uint32_t* decode_tables_dev, const uint8_t* lane_modes_host,
                             void* output_dev, int64_t num_elements, int64_t tile_elements, int prob_bits, int num_lanes,
                             int64_t first_tile, int64_t tile_count, int* error_dev, ep_stream_t stream);

/* Per-byte-lane 256-bin histogram of the tensor's bytes into histograms_dev[num_lanes][256] (u64,
 * cleared by the call). Stands in for _lane_histogram, entropack/schemes/tile_ans/cuda.py:31-47 /
 * tile_ans_histogram_kernel, tile_ans.cu:27-65. */
int ep_tile_ans_histogram(const void* input_dev, int64_t num_elements, int num_lanes, uint64_t* histograms_dev,
                          ep_stream_t stream);

/* Host-only: choose probability_bits (0 = automatic) and lane modes and build the coding tables from
 * the histograms. Stands in for _lane_tables, entropack/schemes/tile_ans/cuda.py:50-61, i.e.
 * select_coding_options / build_tables_from_counts / lane_modes_from_counts of
 * entropack/schemes/tile_ans/eager.py:16-145. Outputs: frequencies[num_lanes][256],
 * cdfs[num_lanes][256], decode_tables[num_lanes][1 << *prob_bits_out] (room for 4096 entries per
 * lane), lane_modes[num_lanes]. */
int ep_tile_ans_plan(const uint64_t* histograms_host, int num_lanes, int64_t tile_elements, double raw_lane_threshold,
                     int prob_bits_in, int* prob_bits_out, uint16_t* frequencies_host, uint16_t* cdfs_host,
                     uint32_t* decode_tables_host, uint8_t* lane_modes_host);

/* Encode every (byte lane, tile) stream into its own slot of scratch_dev
 * (num_lanes * tiles * tile_elements u16 words), writing word_counts_dev[streams] and
 * states_dev[ans_lanes * tiles][32]. Stands in for tile_ans_encode_kernel, tile_ans.cu:67-155
 * (launch at entropack/schemes/tile_ans/cuda.py:64-98). */
int ep_tile_ans_encode(const void* input_dev, int64_t num_elements, int num_lanes, int64_t tile_elements, int prob_bits,
                       const uint16_t* frequencies_dev, const uint16_t* cdfs_dev, const uint8_t* lane_modes_host,
                       uint16_t* scratch_dev, uint32_t* word_counts_dev, uint32_t* states_dev, ep_stream_t stream);

/* Exclusive prefix sum of u32 counts into offsets_dev[count + 1] (u32) with the u64 grand total in
 * total_dev[0]; the device-side stand-in for the cupy.cumsum calls of the reference's encoders
 * (tile_ans/cuda.py:99-104, lattice_rans/cuda.py:543-551). `count` up to 2^31-1. */
int ep_exclusive_scan_u32(const uint32_t* counts_dev, int64_t count, uint32_t* offsets_dev, uint64_t* total_dev,
                          ep_stream_t stream);

/* Gather per-stream scratch slots (stride `slot_words`) into the contiguous payload. Stands in for
 * tile_ans_compact_kernel (tile_ans.cu:157-173) and e8_compact_kernel (lattice_rans.cu:467-481). */
int ep_compact_streams(const uint16_t* scratch_dev, const uint32_t* offsets_dev, uint16_t* payload_dev, int64_t slot_words,
                       int64_t streams, ep_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * EntroPack-Lossy (E8 lattice + coset-conditioned rANS).
 * Buffer schema: entropack/schemes/lattice_rans/format.py:91-98.
 * ------------------------------------------------------------------------------------------- */

/* element type written by ep_lattice_decode (the reference's store kinds, lattice_rans/cuda.py:65-69) */
#define EP_STORE_BF16 0
#define EP_STORE_F16 1
#define EP_STORE_F32 2
#define EP_STORE_F8_E4M3 3
#define EP_STORE_F8_E5M2 4
#define EP_STORE_I8 5
#define EP_STORE_U8 6
#define EP_STORE_I16 7
#define EP_STORE_U16 8
#define EP_STORE_I32 9
#define EP_STORE_U32 10
#define EP_STORE_I64 11
#define EP_STORE_U64 12
#define EP_STORE_BOOL 13

/* Bytes of table scratch ep_lattice_decode needs for a container when it builds the slot tables itself
 * (tables_ready = 0): 0 when they fit in shared memory (prob_bits <= 11, whatever the alphabets), else
 * 17 * 2^prob_bits * 8. */
int64_t ep_lattice_decode_scratch_bytes(int prob_bits, int max_alphabet);

/* A container's slot tables, built once and kept by the caller for every later decode of that container
 * -- the decode plan that the reference caches per container (entropack/schemes/lattice_rans/cuda.py:697-741).
 * ep_lattice_slot_tables_bytes gives the size (17 * 2^prob_bits entries of 4, 5 or 8 bytes, by table
 * layout), ep_lattice_build_slot_tables fills a 16-byte aligned device buffer of that size from the
 * container's stream_meta and freq_tables (one small launch). Passing the buffer to ep_lattice_decode /
 * ep_lattice_linear_forward as table_scratch_dev with tables_ready = 1 replaces the table build at the head
 * of every decode (13 us at 4 bpp, 30 us with alphabets beyond 512) by a copy into shared memory. */
int64_t ep_lattice_slot_tables_bytes(int prob_bits, int max_alphabet);
int ep_lattice_build_slot_tables(const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev, int64_t freq_entries,
                                 int prob_bits, int max_alphabet, void* slot_tables_dev, int64_t slot_tables_bytes,
                                 ep_stream_t stream);

/* Decode + reconstruct + container cast into output_dev[rows][cols] (cols = the padded column count
 * stored in the layout, a multiple of 8). Stands in for decode() of
 * entropack/schemes/lattice_rans/cuda.py:781-805 together with its host-side _decode_plan (:697-741)
 * and the e8_decode_vector_* kernels (lattice_rans.cu:732-1141). With tables_ready = 0 the slot tables
 * are rebuilt on the device from freq_tables inside the call (table_scratch_dev is plain scratch, see
 * ep_lattice_decode_scratch_bytes); with tables_ready = 1 table_scratch_dev holds tables that
 * ep_lattice_build_slot_tables made for this container. `max_alphabet` is the largest alphabet in
 * stream_meta (the caller reads that 17x4 buffer once); `freq_entries` is the length of freq_tables_dev
 * and bounds every read of it, whatever the table records claim. bf16 output saturates at the largest
 * finite value, as the reference's eager lane does. A coset symbol above 1 (only a corrupt coset table
 * yields one) is decoded as 1 and reported as EP_STREAM_BAD_SYMBOL. */
int ep_lattice_decode(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                      const uint32_t* states_dev, const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev,
                      int64_t freq_entries, const float* scales_dev, void* output_dev, int store_kind, int64_t rows,
                      int64_t cols, int prob_bits, int64_t tile_elements, int max_alphabet, void* table_scratch_dev,
                      int64_t table_scratch_bytes, int tables_ready, int* error_dev, ep_stream_t stream);

/* Fused forward of a lossy-coded bf16 layer for 1..4 tokens: y[t][r] = bf16(sum_c x[t][c] * W[r][c] + bias[r]) with
 * W the decoded weight rounded to bf16, which is never written out: the decode kernel multiplies every
 * reconstructed vector into the tokens' dot products and adds them per weight row into products_dev
 * (fp32, tokens * rows + 1 words, cleared by the call; the last word counts finished blocks, and the block
 * that finishes last writes y). x_dev bf16 [tokens][cols], bias_dev bf16 [rows] or null, y_dev bf16
 * [tokens][rows]. Decode arguments as for ep_lattice_decode. Sums are added with atomics, so the last bits of a
 * result can differ between runs. Stands in for decode + F.linear of CompressedLinear.forward
 * (entropack/linear/linear.py:125-130, 163-165) at decode-time batch sizes. */
int ep_lattice_linear_forward(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                              const uint32_t* states_dev, const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev,
                              int64_t freq_entries, const float* scales_dev, int64_t rows, int64_t cols, int prob_bits,
                              int64_t tile_elements,
                              int max_alphabet, void* table_scratch_dev, int64_t table_scratch_bytes, int tables_ready,
                              const void* x_dev, const void* bias_dev, int tokens, float* products_dev, void* y_dev,
                              int* error_dev, ep_stream_t stream);

/* Same decode for callers that cannot allocate device memory when they need it -- for example a
 * serving process that has given all of HBM to its own pool, or code running inside an allocator
 * callback. This entry point has no counterpart in the reference. The slot tables of the global-table
 * path are kept in a fixed 1.06 MB array inside the library (resident on every GPU that loads it, for
 * the life of the process), so no scratch is passed and nothing is allocated. Limits and rules:
 *   - a container that needs the global-table path must have prob_bits <= 13
 *     (ep_lattice_decode_static_max_prob_bits()); larger ones return EP_ERR_TOO_LARGE. Containers whose
 *     tables fit in shared memory (prob_bits <= 11) are always accepted;
 *   - the first call on each device looks up the array's device address (a runtime query), and if the
 *     library's code has not been loaded onto that device yet, that first call is also when the CUDA
 *     runtime loads it together with the fixed array: make that first call outside any stream capture
 *     and before the host's own pool takes the rest of the device's memory;
 *   - every call on a device shares the one array. It is rewritten in full by each call that uses it,
 *     so stale contents never matter, but two such calls in flight at once on the same device
 *     (different streams or threads) race; serialise them. */
int ep_lattice_decode_static_max_prob_bits(void);
int ep_lattice_decode_static(const uint16_t* payload_dev, int64_t payload_words, const uint32_t* offsets_dev,
                             const uint32_t* states_dev, const int32_t* stream_meta_dev, const uint16_t* freq_tables_dev,
                             int64_t freq_entries, const float* scales_dev, void* output_dev, int store_kind, int64_t rows,
                             int64_t cols, int prob_bits, int64_t tile_elements, int max_alphabet, int* error_dev,
                             ep_stream_t stream);

/* --- encode. Work tensors are bf16 or fp32 [rows][cols], cols a multiple of 8 (is_bf16 selects);
 * quantised symbols travel as fields_dev int16[vectors][8] (z0..z6, m) and cosets_dev u8[vectors].
 * Replaces the kernels and host glue of entropack/schemes/lattice_rans/cuda.py:115-597. --- */

/* rms_dev[row] = max(sqrt(mean(x^2)), 1e-12) in fp32 with a fixed summation order
 * (the torch reduction at lattice_rans/cuda.py:580). */
int ep_lattice_row_rms(const void* weight_dev, int is_bf16, int64_t rows, int64_t cols, float* rms_dev, ep_stream_t stream);

/* Nearest-E8 quantisation of (x / rms_row) / scale, plus per-stream min/max into minmax_dev[34]
 * (16 x (min, max), max coset, int16-overflow flag; initialised by the call). Stands in for
 * e8_quantize_fields_kernel, lattice_rans.cu:149-241 (call site cuda.py:115-139). */
int ep_lattice_quantize(const void* weight_dev, int is_bf16, const float* rms_dev, int64_t rows, int64_t cols, float scale,
                        int16_t* fields_dev, uint8_t* cosets_dev, int32_t* minmax_dev, ep_stream_t stream);

/* The rate search as one call: `iterations` steps of geometric bisection of the global scale between `low` and `high`
 * on the (sub-sampled) operand, each step = ep_lattice_quantize + ep_lattice_histogram into `stats_dev`
 * (int32[36 + bins_capacity]: min/max record[34], bins used, pad, bins), the statistics read back and priced with
 * ep_lattice_coded_bytes + rows * 4 + fixed_bytes against target_bpp. Writes sqrt(low * high) after the last step
 * to *scale_host. Returns EP_MORE_BINS with the needed capacity in *bins_needed_host when a step's alphabets do
 * not fit `bins_capacity` (call again with a larger buffer). Stands in for _bisect_scale_cuda / _SearchState.total_at,
 * entropack/schemes/lattice_rans/cuda.py:315-478; synchronises `stream` once or twice per step. */
int ep_lattice_search_scale(const void* weight_dev, int is_bf16, const float* rms_dev, int64_t rows, int64_t cols,
                            int16_t* fields_dev, uint8_t* cosets_dev, int32_t* stats_dev, int64_t bins_capacity,
                            double target_bpp, int prob_bits, int64_t tile_elements, int iterations, double low, double high,
                            double fixed_bytes, double* scale_host, int64_t* bins_needed_host, ep_stream_t stream);

/* Exact per-stream symbol counts into compact bins (2 coset bins, then max - min + 1 bins per live
 * stream, in table order); bins_used_dev[0] receives the number of bins the min/max record implies and
 * nothing is counted when that exceeds bins_capacity. Stands in for e8_histogram_kernel,
 * lattice_rans.cu:376-396 (call site cuda.py:181-220). */
int ep_lattice_histogram(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t vectors, const int32_t* minmax_dev,
                         int32_t* bins_dev, int64_t bins_capacity, int32_t* bins_used_dev, ep_stream_t stream);

/* Host-only helpers over a min/max record and its bins copied to the host. */
int64_t ep_lattice_bins_needed(const int32_t* minmax_host);
int ep_lattice_max_alphabet(const int32_t* minmax_host);
/* Container-size model of the rate search: rans.coded_bytes, entropack/schemes/lattice_rans/rans.py:224-258. */
int ep_lattice_coded_bytes(const int32_t* minmax_host, const int32_t* bins_host, int64_t vectors, int prob_bits,
                           int64_t tile_elements, double* bytes_out);
/* stream_meta[17][4] and the concatenated normalised frequency tables for the final encode:
 * _build_codec_tables, entropack/schemes/lattice_rans/cuda.py:481-517. */
int ep_lattice_tables(const int32_t* minmax_host, const int32_t* bins_host, int64_t vectors, int prob_bits,
                      int32_t* stream_meta_host, uint16_t* freq_tables_host, int64_t freq_capacity, int64_t* freq_entries_out);

/* Least-squares row scales against the quantised points (fallback scale * rms_row). Stands in for
 * e8_refit_scales_kernel, lattice_rans.cu:243-332. */
int ep_lattice_refit_scales(const void* weight_dev, int is_bf16, const int16_t* fields_dev, const uint8_t* cosets_dev,
                            const float* rms_dev, float scale, int64_t rows, int64_t cols, float* scales_dev, ep_stream_t stream);

/* The same fit, plus row_sse_dev[row] = |x|^2 - (x.p)^2 / |p|^2 clamped at zero (|x|^2 when the row
 * quantised to zero): _refit_row_scales, entropack/schemes/lattice_rans/eager.py:209-224. */
int ep_lattice_refit_rows(const void* weight_dev, int is_bf16, const int16_t* fields_dev, const uint8_t* cosets_dev,
                          const float* rms_dev, float scale, int64_t rows, int64_t cols, float* scales_dev, float* row_sse_dev,
                          ep_stream_t stream);

/* --- per-row rate-distortion refinement (row_rdo_iterations > 0): the device side of
 * entropack/schemes/lattice_rans/rdo.py:70-162. --- */

/* Min/max record (same 34 words as ep_lattice_quantize writes) of symbols that are already quantised. */
int ep_lattice_minmax(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t vectors, int32_t* minmax_dev,
                      ep_stream_t stream);

/* rates_dev[row] = modelled bits of the row's symbols under a 17-table rate model: table t starts at
 * rate_offsets_dev[t] (18 entries) inside rate_values_dev and its first entry prices symbol
 * rate_minima_dev[t]. rdo.row_rates, rdo.py:70-84. */
int ep_lattice_row_rates(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t rows, int64_t cols,
                         const float* rate_values_dev, const int32_t* rate_offsets_dev, const int32_t* rate_minima_dev,
                         float* rates_dev, ep_stream_t stream);

/* Output row r = row r of candidate choice_dev[r]; the two pointer arrays (device memory, `candidates`
 * entries) name each candidate's fields and cosets. rdo.select_candidate_rows, rdo.py:103-120. */
int ep_lattice_select_rows(const int16_t* const* candidate_fields_dev, const uint8_t* const* candidate_cosets_dev, int candidates,
                           const int32_t* choice_dev, int64_t rows, int64_t cols, int16_t* fields_dev, uint8_t* cosets_dev,
                           ep_stream_t stream);

/* u16 words of per-tile scratch ep_lattice_encode writes into (tiles * tile_vectors * 9). */
int64_t ep_lattice_encode_scratch_words(int64_t vectors, int64_t tile_elements);

/* rANS-encode every tile into its scratch slot; word_counts_dev[tiles], states_dev[tiles][32].
 * symbol_scratch_dev: freq_entries * 8 bytes of scratch for the per-symbol encode records.
 * Follow with ep_exclusive_scan_u32 and ep_compact_streams (slot = tile_vectors * 9 words). Stands in
 * for e8_rans_encode_vector_kernel, lattice_rans.cu:400-465 (call site cuda.py:520-558). */
int ep_lattice_encode(const int16_t* fields_dev, const uint8_t* cosets_dev, int64_t vectors, const int32_t* stream_meta_dev,
                      const uint16_t* freq_tables_dev, int64_t freq_entries, int prob_bits, int64_t tile_elements,
                      void* symbol_scratch_dev, uint16_t* scratch_dev, uint32_t* word_counts_dev, uint32_t* states_dev,
                      ep_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * DFloat11 (Huffman-coded bf16 exponents). Buffer schema: entropack/schemes/dfloat11/format.py:32-63.
 * ------------------------------------------------------------------------------------------- */

/* Decode into output_dev (bf16[n_elements]). bytes_per_thread / threads_per_block / max_block_elems are
 * the container's layout values. Stands in for decode(), entropack/schemes/dfloat11/cuda.py:57-101 /
 * dfloat11_decode_kernel, dfloat11.cu:314-522. threads_per_block up to 1024. */
int ep_dfloat11_decode(const uint8_t* luts_dev, int num_luts, const uint8_t* encoded_dev, int64_t n_bytes,
                       const uint8_t* sign_mantissa_dev, const uint32_t* output_positions_dev, const uint16_t* thread_meta_dev,
                       void* output_dev, int64_t n_elements, int bytes_per_thread, int threads_per_block, int max_block_elems,
                       const void* decode_tables_dev, int64_t decode_tables_bytes, int* error_dev, ep_stream_t stream);

/* A container's decode tables, built once and kept by the caller for every later decode of that container: the
 * level tables fused with the length row and an 11-bit multi-symbol table (up to four codewords per look-up). The
 * reference rebuilds nothing per decode either -- its kernel reads luts as stored (dfloat11.cu:314-522); this is the
 * form that kernel's look-ups take here. ep_dfloat11_decode_tables_bytes gives the size, ep_dfloat11_build_decode_tables
 * fills a 16-byte aligned device buffer of that size from luts (one small launch); passed to ep_dfloat11_decode as
 * decode_tables_dev it replaces the table build at the head of every CUDA block by a copy, and, where the layout
 * allows it, selects the faster of the two decode kernels: one warp per run of 32 regions, persistent blocks, inputs
 * brought in by bulk copies ahead of their use. That kernel takes containers whose bytes_per_thread is a multiple of 4,
 * whose encoded / sign_mantissa / output buffers start on 16-byte boundaries and whose stream and element counts fit
 * 32 bits; any other container is decoded by the block-per-format-block kernel with the same tables. A bulk copy that
 * does not complete within its bounded wait ends the decode with EP_KERNEL_TIMEOUT in *error_dev. With a null
 * decode_tables_dev the decode builds a 10-bit table itself (block kernel). */
int64_t ep_dfloat11_decode_tables_bytes(int num_luts);
int ep_dfloat11_build_decode_tables(const uint8_t* luts_dev, int num_luts, void* tables_dev, int64_t tables_bytes,
                                    ep_stream_t stream);

/* 256-bin histogram of the exponent byte (u64, cleared by the call). Stands in for exponent_counter,
 * entropack/schemes/dfloat11/cuda.py:104-122. */
int ep_dfloat11_histogram(const void* bf16_dev, int64_t n_elements, uint64_t* histogram_dev, ep_stream_t stream);

/* Host-only: prefix code for the histogram -- code_len[257] / code_val[257], index 256 = end of stream --
 * and the multi-level LUT rows (levels + 1 rows of 256 bytes; luts_host holds max_rows rows). Stand in for
 * get_32bit_codec / get_luts, entropack/schemes/dfloat11/eager.py:42-116; the reference takes its code
 * from the dahuffman package, this library builds a canonical Huffman code (same lengths as any optimal
 * code up to ties; the bitstream carries its own tables, so either side decodes the other's). */
int ep_dfloat11_build_code(const uint64_t* histogram_host, int32_t* code_len_host, uint32_t* code_val_host);
int ep_dfloat11_build_luts(const int32_t* code_len_host, const uint32_t* code_val_host, uint8_t* luts_host, int max_rows,
                           int* rows_out);

/* Encode, in three calls replacing the five kernels + cumsum of entropack/schemes/dfloat11/cuda.py:136-223:
 * ep_dfloat11_chunk_bits sums code lengths per chunk (ep_dfloat11_chunks(n) chunks), ep_exclusive_scan_u32
 * turns them into bit offsets and the total, ep_dfloat11_pack writes the bitstream (encoded_dev must hold
 * ceil(total_bits / 8) rounded up to 4, plus 4 bytes), sign_mantissa, thread_meta[blocks * threads_per_block]
 * and output_positions[blocks + 1]. region_scratch_dev: 2 * blocks * threads_per_block u32 of scratch.
 * total_bits must be below 2^32. */
int64_t ep_dfloat11_chunks(int64_t n_elements);
int ep_dfloat11_chunk_bits(const void* bf16_dev, int64_t n_elements, const int32_t* code_len_dev, uint32_t* chunk_bits_dev,
                           ep_stream_t stream);
int ep_dfloat11_pack(const void* bf16_dev, int64_t n_elements, const int32_t* code_len_dev, const int32_t* code_val_dev,
                     const uint32_t* chunk_offsets_dev, uint64_t total_bits, int bytes_per_thread, int threads_per_block,
                     int eof_length, uint32_t eof_value, uint8_t* encoded_dev, uint8_t* sign_mantissa_dev,
                     uint16_t* thread_meta_dev, uint32_t* output_positions_dev, uint32_t* region_scratch_dev, ep_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Linear forward on a decoded weight.
 * ------------------------------------------------------------------------------------------- */

/* y[m][n] = x[m][k] . weight[n][k]^T (+ bias[n]), all bf16, fp32 accumulation. k must be a multiple of 8
 * and the three matrices 16-byte aligned. Stands in for the F.linear call of CompressedLinear.forward
 * (entropack/linear/linear.py:163-165): m <= 16 streams the weight straight into m16n8k16 fragments,
 * larger m runs the persistent tcgen05 / TMEM tensor-core kernel fed by TMA. A wait that runs out inside the tensor-core kernel is
 * reported as code 9 in error_dev (optional device int32, zeroed by the caller). */
int ep_linear_forward(const void* x_dev, const void* weight_dev, const void* bias_dev, void* y_dev, int64_t m, int64_t n,
                      int64_t k, int* error_dev, ep_stream_t stream);

/* ep_linear_forward for a column-sharded layer, with the all-gather of the outputs folded into the epilogue: this
 * rank's product is columns [y_col0, y_col0 + n) of output rows that are y_ld elements long, and every finished tile
 * is stored to y_dev and, with ordinary stores through peer mappings, to the same place in each of the `peers`
 * buffers of y_peers_host (a host array of device pointers: the other GPUs' output buffers as mapped on this GPU, at
 * most 7). y_ld and y_col0 must be multiples of 8 for 16-byte stores (else element stores). The two-block tensor-core
 * kernel only: m <= 128 returns EP_ERR_UNSUPPORTED (gather those few rows instead). The reference has no multi-GPU code; this is
 * the NVLink half of CompressedLinear.forward (entropack/linear/linear.py:163-165) on a column shard. */
int ep_linear_forward_scatter(const void* x_dev, const void* weight_dev, const void* bias_dev, void* y_dev,
                              void* const* y_peers_host, int peers, int64_t y_ld, int64_t y_col0, int64_t m, int64_t n, int64_t k,
                              int* error_dev, ep_stream_t stream);

/* Barrier between the `world` GPUs (at most 8) that write into one another's buffers, as one small launch on `stream`:
 * flag_rows_host[r] is rank r's row of `world` uint32 flags as mapped on this GPU (zero before the first use). The
 * kernel stores `epoch` (use 1, 2, 3, ... per barrier) into slot `rank` of every peer's row with a system-scope
 * release and polls slot r of its own row until peer r's epoch shows, for at most timeout_us microseconds; a peer
 * that does not arrive in time sets *error_dev to EP_KERNEL_TIMEOUT and the kernel returns -- no trap, no endless
 * wait. Stream order makes everything this rank launched before the barrier visible to the peers that pass it. */
int ep_peer_barrier(void* const* flag_rows_host, int rank, int world, uint32_t epoch, int64_t timeout_us, int* error_dev,
                    ep_stream_t stream);

/* The 8-bit layer's product: y[m][n] = (x_codes[m][k] . weight_codes[n][k]^T) * x_scale[m] * weight_scale[n]
 * (+ bias[n], fp32), both code matrices fp8 e4m3, accumulation in fp32 on the tcgen05 kernel
 * (kind::f8f6f4), y written as bf16 (y_is_f32 = 0) or fp32. k must be a multiple of 16. Stands in for
 * the torch._scaled_mm call of CompressedFP8Linear (entropack/linear/linear.py:399-418). */
int ep_linear_forward_fp8(const void* x_codes_dev, const void* weight_codes_dev, const float* x_scale_dev,
                          const float* weight_scale_dev, const float* bias_dev, void* y_dev, int y_is_f32, int64_t m, int64_t n,
                          int64_t k, int* error_dev, ep_stream_t stream);

/* Per-row activation quantisation of the FP8 layer: scales_dev[r] = max(absmax(x[r]) / 448, eps32),
 * codes_dev[r][c] = e4m3(clamp(x[r][c] / scale, -448, 448)). x_kind: 0 bf16, 1 fp16, 2 fp32.
 * QuantizedLinear._quantize_rows, entropack/linear/linear.py:286-293. */
int ep_quantize_rows_fp8(const void* x_dev, int x_kind, int64_t rows, int64_t cols, void* codes_dev, float* scales_dev,
                         ep_stream_t stream);

/* The INT8 layer's counterparts: signed 8-bit codes, kind::i8 product with 32-bit integer accumulators, the same scaled
 * epilogue; scales_dev[r] = max(absmax / 127, eps32), codes = clamp(rint(x / scale), -127, 127). Stand in for
 * torch._int_mm plus the scale/bias arithmetic of CompressedINT8Linear (entropack/linear/linear.py:421-490, without the
 * ConvRot rotation) and for its _quantize_rows. */
int ep_linear_forward_int8(const void* x_codes_dev, const void* weight_codes_dev, const float* x_scale_dev,
                           const float* weight_scale_dev, const float* bias_dev, void* y_dev, int y_is_f32, int64_t m, int64_t n,
                           int64_t k, int* error_dev, ep_stream_t stream);
int ep_quantize_rows_int8(const void* x_dev, int x_kind, int64_t rows, int64_t cols, void* codes_dev, float* scales_dev,
                          ep_stream_t stream);

/* y[r] = x[r] . R applied to every group of `group` consecutive features (group a power of four that divides cols), R the
 * ConvRot matrix of entropack/linear/convrot.py:35-45: symmetric and self-inverse, so this one call stands in for
 * rotate_activation and for rotate_weight in both directions (convrot.py:48-61). x_kind: 0 bf16, 1 fp16, 2 fp32; the
 * arithmetic is fp32 with one rounding at the end. */
int ep_convrot_rows(const void* x_dev, int x_kind, int64_t rows, int64_t cols, int group, void* y_dev, ep_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* ENTROPACK_B200_H */
