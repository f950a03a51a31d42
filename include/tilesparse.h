/* tilesparse.h -- C ABI of libtilesparse (NVIDIA B200, sm_100a).
 *
 * A drop-in for the hot path of clevercool/TileSparsity: the Stream Masked GEMM for tile-wise (TW)
 * sparse weights and the TW/TEW mask construction that feeds it.  Each entry point names the
 * reference interface it replaces (paths relative to the reference repository).
 *
 * Conventions
 *  - Every function returns an int status: TS_OK or a TS_ERR_* code; it never aborts the process.
 *    ts_last_error() returns a description of the calling thread's last failure.
 *  - Device pointers are borrowed for the duration of the enqueued work; the caller allocates and
 *    frees them (as in StreamMaskedGEMM/perf/basic_nn.cu:936-984,1107-1129).
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued on it, with no hidden device
 *    synchronisation unless the function's comment says otherwise.
 *  - Matrix layout is the reference's column-major convention (basic_nn.cu:412-426):
 *      At  activations  [K][lda]  batch dimension M contiguous   (column-major M x K)
 *      Ct  outputs      [N][ldc]  batch dimension M contiguous   (column-major M x N)
 *    M, lda and ldc must be multiples of 8 (the reference rounds its sizes up to 8, basic_nn.cu:1157)
 *    and base pointers 16-byte aligned.
 *  - There is no CPU fallback: without a CUDA device every compute call fails with TS_ERR_CUDA.
 */
#ifndef TILESPARSE_H_
#define TILESPARSE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TS_OK 0
#define TS_ERR_INVALID 1     /* bad argument                                                   */
#define TS_ERR_CUDA 2        /* a CUDA runtime / driver call failed                            */
#define TS_ERR_TIMEOUT 3     /* a bounded device-side wait ran out (kernel returned early)     */
#define TS_ERR_UNSUPPORTED 4 /* valid request this build does not implement                    */
#define TS_ERR_NOMEM 5       /* device or host allocation failed                               */

#define TS_DTYPE_F16 0
#define TS_DTYPE_BF16 1
#define TS_DTYPE_F32 2

/* Index-list formats accepted by ts_layer_set_tiles. */
#define TS_INDEX_ABSOLUTE 0 /* list[i] = kept index                                            */
#define TS_INDEX_RELATIVE 1 /* list[i] = kept index - i  (mask_gen, basic_nn.cu:697-718;
                               convert_mask_to_offset, Pruning/BERT/utils/MyHook.py:66-74)      */

/* Activation layouts accepted by ts_masked_gemm. */
#define TS_LAYOUT_K_MAJOR 0 /* [K][M], the reference's layout                                  */

typedef struct ts_layer ts_layer_t;

/* Library version (major*10000 + minor*100 + patch).  No reference counterpart. */
int ts_version(void);

/* Copies a description of the calling thread's last error into buf (NUL terminated, at most n
 * bytes); returns the length written.  Replaces the reference's cudaGetErrorString prints
 * (basic_nn.cu:346-349). */
int ts_last_error(char* buf, int n);

/* ---------------------------------------------------------------------------------------------
 * Layer handle: one tile-wise sparse weight matrix W[K][N] (row-major), G columns per tile.
 * Replaces the per-layer bookkeeping TestCutlassGemm keeps in host arrays N_cal/K_cal/mask_k/
 * mask_n/off_B/off_C (basic_nn.cu:836-903).
 * ------------------------------------------------------------------------------------------- */

/* Creates an empty layer on the current CUDA device.  G is the maximum number of kept columns per
 * tile and must be <= 128 (N_dim, basic_nn.cu:73).  dtype is the 16-bit compute type of
 * activations, packed weights and outputs (accumulation is fp32). */
int ts_layer_create(ts_layer_t** out, int K, int N, int G, int dtype);

/* Frees the layer and every device buffer it owns.  Synchronises the device. */
int ts_layer_destroy(ts_layer_t* layer);

/* Installs the tile structure (host arrays; copied to the device, synchronous).
 *   tile_k_ptr[n_tiles+1], kept_k_idx: CSR of each tile's kept K rows, ascending, in [0, K)
 *   tile_n_ptr[n_tiles+1], kept_n_idx: CSR of each tile's kept columns, in [0, N), at most G each
 * With TS_INDEX_RELATIVE the lists hold `index - position` per tile as the reference stores them.
 * Replaces mask_gen + the cudaMalloc/cudaMemcpy of the lists (basic_nn.cu:697-741,889-903). */
int ts_layer_set_tiles(ts_layer_t* layer, int n_tiles, const int32_t* tile_k_ptr,
                       const int32_t* kept_k_idx, const int32_t* tile_n_ptr,
                       const int32_t* kept_n_idx, int index_format);

/* Packs the kept weights of W_dev ([K][ldw_in] row-major, w_dtype any TS_DTYPE_*) into the
 * layer's per-tile compacted matrix.  Replaces gen_masked_stream_weight (basic_nn.cu:757-769) and
 * the kernel compaction of exportPrunedModel (MyHook.py:76-85). */
int ts_layer_pack_weights(ts_layer_t* layer, const void* W_dev, int64_t ldw_in, int w_dtype,
                          void* stream);

/* Reads back the packed weights as [n_tiles*128][ldw] 16-bit (synchronous).  Pass out == NULL to
 * query: *rows and *ldw receive the packed matrix's shape.  Testing/export aid; mirrors the
 * compacted kernels exportPrunedModel pickles (MyHook.py:84-89). */
int ts_layer_get_packed(const ts_layer_t* layer, void* out_host, int64_t* rows, int64_t* ldw);

/* kept_flops = 2 * sum_t K_t * N_t (per batch row); packed_bytes = bytes of kept weights;
 * index_bytes = bytes of the index lists.  Any pointer may be NULL. */
int ts_layer_stats(const ts_layer_t* layer, int64_t* kept_flops_per_row, int64_t* packed_bytes,
                   int64_t* index_bytes, int* n_tiles, int* max_kept_k);

/* Masked GEMM of the whole layer in one launch:
 *     Ct[n][m] = alpha * sum_k At[k][m] * (W .* mask)[k][n] + beta * Ct[n][m]   for kept columns n
 * Columns that no tile keeps are not written.  Replaces Stream_Gemm_NN (basic_nn.cu:378-445),
 * i.e. params.initialize + Gemm::launch(params, mask_k, mask_n, stream) per tile
 * (StreamMaskedGEMM/cutlass/gemm/gemm.h:317-327). */
int ts_masked_gemm(ts_layer_t* layer, int M, const void* At_dev, int64_t lda, void* Ct_dev,
                   int64_t ldc, float alpha, float beta, void* stream);

/* Same operation on the CUDA cores in fp32 (the twin of the reference's CUDA_MODE build,
 * basic_nn.cu:55-71,239-246).  Cross-check path, not tuned. */
int ts_masked_gemm_simt(ts_layer_t* layer, int M, const void* At_dev, int64_t lda, void* Ct_dev,
                        int64_t ldc, float alpha, float beta, void* stream);

/* Same operation with HOST buffers: copies At (K x M, ld = M) to the device, runs ts_masked_gemm,
 * copies Ct (N x M, ld = M) back and synchronises.  Pinned host memory makes the copies
 * asynchronous; pageable memory works too.  The device staging buffers belong to the layer and
 * grow on demand.  Ct is read from the host only when beta != 0; with beta == 0 the columns that
 * no tile keeps come back as zeros.  This is the whole of TestCutlassGemm's H2D -> Stream_Gemm_NN -> D2H sequence
 * (basic_nn.cu:986-1034) as one call. */
int ts_masked_gemm_host(ts_layer_t* layer, int M, const void* At_host, void* Ct_host, float alpha,
                        float beta, void* stream);

/* Reads and clears the layer's device status word (synchronises `stream`).  Returns TS_OK or the
 * error a kernel recorded (TS_ERR_TIMEOUT when a bounded wait ran out). */
int ts_layer_check(ts_layer_t* layer, void* stream);

/* Per-CTA load of the schedule ts_masked_gemm uses for batch size M: writes the summed cost of
 * every CTA's work units (in 64-row K blocks, epilogue included) to cta_cost[0..*n_ctas).  Pass
 * cta_cost == NULL to query *n_ctas. */
int ts_layer_schedule_stats(ts_layer_t* layer, int M, int* n_ctas, float* cta_cost, int* n_units);

/* ---------------------------------------------------------------------------------------------
 * Reference-signature entry point.
 * ------------------------------------------------------------------------------------------- */

/* Stream_Gemm_NN with the reference's arguments (basic_nn.cu:378-393): A is At [K][M]; B holds the
 * compacted tiles column-major with ldb = K, tile t at B + off_B[t]; C is Ct [N][M], tile t at
 * C + off_C[t]; mask_k[t] / mask_n[t] are DEVICE pointers to K_cal[t] / N_cal[t] relative
 * offsets; N_cal, K_cal, off_B, off_C are HOST arrays of block_num entries (block_num <= 32,
 * N_cal[t] <= 128).  All tiles run in one launch on `stream`.  The call uploads a small tile table
 * (synchronous copy into a cached workspace), then enqueues the kernel. */
int ts_stream_gemm_nn(int M, int N, int K, float alpha, const void* A, const void* B, float beta,
                      void* C, int block_num, const int* N_cal, const int* K_cal,
                      int* const* mask_n, int* const* mask_k, const int* off_B, const int* off_C,
                      int dtype, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Helpers
 * ------------------------------------------------------------------------------------------- */

/* out[c][r] = in[r][c] for 16-bit elements: row-major activations [M][K] -> At [K][M].  The
 * reference does this on the host (transpose_matrix, basic_nn.cu:823). */
int ts_transpose16(const void* in_dev, int64_t ld_in, void* out_dev, int64_t ld_out, int rows,
                   int cols, void* stream);

/* Greedy longest-processing-time assignment of column tiles to n_parts devices by kept work
 * cost[t] (e.g. K_t * N_t); owner_out[t] in [0, n_parts).  Pure host function.  The reference has
 * no multi-device path; its unit of distribution is the same column tile, one per CUDA stream
 * (basic_nn.cu:396-427). */
int ts_shard_plan(int n_tiles, const int64_t* cost, int n_parts, int32_t* owner_out);

#ifdef __cplusplus
}
#endif

#endif /* TILESPARSE_H_ */
