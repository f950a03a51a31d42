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

/* Fused epilogue of ts_masked_gemm_ex:  Ct[n][m] = act(alpha * acc + beta * Ct[n][m] + bias[n]).
 *   bias_dev     fp32 [N] on the device, indexed by the column of W (row of Ct), or NULL
 *   activation   TS_ACT_NONE, TS_ACT_RELU, or TS_ACT_GELU (the tanh form of the reference's BERT,
 *                Pruning/BERT/utils/modeling.py:264-277)
 *   peer_ct      up to 7 further output buffers with the layout of Ct (same ldc, 16-byte aligned): every
 *                kept row is also stored there (a full tile as one TMA tile store per buffer, through
 *                tensor maps the layer encodes once per set of buffers; a ragged tile, or any tile when
 *                beta != 0, as plain 16-byte stores).  Given the peer-mapped Ct buffers of the other GPUs
 *                of a tile-sharded layer, the GEMM's epilogue performs the all-gather over NVLink.
 * This is what the reference's mask_dense does after its matmul (bias add, modeling.py:1003-1007)
 * folded into the GEMM; the reference has no multi-GPU path. */
#define TS_ACT_NONE 0
#define TS_ACT_RELU 1
#define TS_ACT_GELU 2
typedef struct ts_epilogue {
  float alpha;
  float beta;
  const float* bias_dev;
  int activation;
  int n_peers;
  void* peer_ct[7];
  void* multicast_ct; /* NULL, or the NVSwitch multicast address that maps Ct on every GPU of the group
                         (this one included): each kept row is then written once with multimem.st and
                         delivered to all copies by the switch; Ct_dev and peer_ct are not written
                         (beta must be 0).  Stores only: nothing is ever loaded through the mapping. */
} ts_epilogue_t;

int ts_masked_gemm_ex(ts_layer_t* layer, int M, const void* At_dev, int64_t lda, void* Ct_dev,
                      int64_t ldc, const ts_epilogue_t* epilogue, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Convolution as an implicit masked GEMM.  The reference prunes a conv kernel [kh][kw][cin][cout] as the
 * matrix [(kh*kw*cin)][cout] with row k = (r*kw + j)*cin + c (img2col_forward, Pruning/VGG/
 * prune_algo.py:16-24) and leaves the convolution itself to TensorFlow; its GEMM driver has no conv
 * path.  Here a stride-1, same-padded convolution runs on the masked GEMM without an im2col matrix:
 * the NHWC input is stored once per horizontal tap as zero-padded channel-major planes, and the
 * GEMM's row gather reads row k of the virtual im2col matrix as a run of plane (j, c) shifted by r
 * padded image rows.  Pixels live in a padded index space: Hp = H + kh - 1 rows of Wp = W + kw - 1
 * (rounded up to 8) columns per image, m = (b*Hp + y)*Wp + x; outputs at y >= H or x >= W are scratch.
 * ------------------------------------------------------------------------------------------- */

/* Sizes of the padded pixel space (pure host function): *m_padded = B*Hp*Wp is the GEMM's batch
 * dimension, *plane_ld the elements every input plane must hold (m_padded + (kh-1)*Wp). */
int ts_conv_geometry(int B, int H, int W, int kh, int kw, int* Hp, int* Wp, int64_t* m_padded, int64_t* plane_ld);

/* Declares the layer's weights to be a kh x kw conv kernel over cin channels (K = kh*kw*cin; odd
 * kh, kw <= 9), row order as img2col_forward produces it. */
int ts_layer_set_conv(ts_layer_t* layer, int cin, int kh, int kw);

/* planes[j][c][m] = Xpad[b][y][x + j][c] for the NHWC 16-bit input x_nhwc_dev [B][H][W][C]:
 * planes_dev is [kw][C][plane_ld] 16-bit, plane_ld >= the value ts_conv_geometry reports.  C must be a
 * multiple of 8 and both pointers 16-byte aligned. */
int ts_conv_pack_input(const void* x_nhwc_dev, int B, int H, int W, int C, int kh, int kw, void* planes_dev,
                       int64_t plane_ld, void* stream);

/* The padded-space output of one convolution, Ct_dev [C][ldc], as the input planes of the next
 * convolution with the same image size and a kh x kw kernel: planes[j][c][m] = Ct[c][m shifted by the
 * tap], zero where the tap leaves the image (which also clears the scratch positions of Ct).  A chain
 * of convolutions therefore stays in the channel-major padded layout: no NHWC round trip between layers. */
int ts_conv_repack(const void* Ct_dev, int64_t ldc, int B, int H, int W, int C, int kh, int kw, void* planes_dev,
                   int64_t plane_ld, void* stream);

/* Ct[n][m] = act(alpha * conv(X, W .* mask)[m][n] + beta * Ct[n][m] + bias[n]) over the padded pixel
 * space, for the layer's kept output channels n; Ct_dev is [N][ldc], ldc >= m_padded. */
int ts_masked_conv(ts_layer_t* layer, int B, int H, int W, const void* planes_dev, int64_t plane_ld, void* Ct_dev,
                   int64_t ldc, const ts_epilogue_t* epilogue, void* stream);

/* y[b][yy][xx][n] = Ct[n][(b*Hp + yy)*Wp + xx]: the padded-space output back to NHWC [B][H][W][N].
 * N and ldc must be multiples of 8 and both pointers 16-byte aligned. */
int ts_conv_unpack_output(const void* Ct_dev, int64_t ldc, int B, int H, int W, int kh, int kw, int N, void* y_nhwc_dev,
                          void* stream);

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

/* The same in two steps, for callers that keep several of these in flight.  _async queues the work:
 * one contiguous copy in, the GEMM and one contiguous copy out on three streams of the layer's own,
 * ordered after what `stream` holds at the call (calls on different layers overlap: one call's
 * copy-out runs under the next call's copy-in, so both directions of the link stay busy).  _wait makes `stream` wait (on the device, not the host) for the arrival of the last
 * block of the layer's latest call; Ct_host is valid once the caller has then synchronised `stream`.
 * Calls on different layers overlap with each other; calls on one layer run one after the other.
 * No counterpart in the reference (its driver copies, computes and copies back in sequence,
 * basic_nn.cu:986-1034). */
int ts_masked_gemm_host_async(ts_layer_t* layer, int M, const void* At_host, void* Ct_host, float alpha,
                              float beta, void* stream);
int ts_masked_gemm_host_wait(ts_layer_t* layer, void* stream);

/* Reads and clears the layer's device status word (synchronises `stream`).  Returns TS_OK or the
 * error a kernel recorded (TS_ERR_TIMEOUT when a bounded wait ran out). */
int ts_layer_check(ts_layer_t* layer, void* stream);

/* Per-CTA load of the schedule ts_masked_gemm uses for batch size M: writes the summed cost of
 * every CTA's work units to cta_cost[0..*n_ctas).  The cost of a unit is the scheduler's model of it
 * in units of 8 KiB moved between L2 and the SM (packed weights and gathered activations per K block,
 * the output, and a constant per unit).  Pass cta_cost == NULL to query *n_ctas.  This is the
 * CTA-level load balance of the single launch that replaces the reference's stream per tile
 * (basic_nn.cu:396-427). */
int ts_layer_schedule_stats(ts_layer_t* layer, int M, int* n_ctas, float* cta_cost, int* n_units);

/* Pins the kernel variant of the layer: work units of at most 128 or 256 batch rows; 0 returns the
 * choice to the scheduler.  Drops the cached schedules (synchronises the device).  A tuning and
 * testing aid; the reference fixes its CTA tile at compile time (basic_nn.cu:250-259). */
int ts_layer_set_unit_rows(ts_layer_t* layer, int unit_rows);

/* Split-K.  A work unit's K blocks run one after the other on one SM, so a launch cannot be shorter
 * than its longest tile's kept rows / 64 blocks.  Where such a chain is long (>= 32 blocks) and the
 * tile's share of the SMs is at least twice its number of 256-row units (a layer with few tiles and
 * thousands of kept rows, e.g. a conv5 kernel pruned to a handful of column tiles), the scheduler cuts
 * the tile's kept rows into up to four ranges that run as units of their own; they leave fp32 partial sums in scratch memory of the cached schedule
 * and a second kernel adds them up and applies beta, bias and activation.  Deterministic, but not
 * bit-identical to the unsplit schedule (another summation order).  On by default; calls that write
 * peer buffers never split.  ts_layer_set_split_k(layer, 0) turns it off for a layer (no counterpart
 * in the reference, whose tiles each run as one CUTLASS launch, basic_nn.cu:396-427).
 * ts_plan_split returns the number of ranges per tile the scheduler would use (host logic only, no
 * device needed): k_counts / n_counts = kept rows / kept columns per tile, K the rows of the activation
 * matrix, M the batch size, n_ctas the number of SMs. */
int ts_layer_set_split_k(ts_layer_t* layer, int enabled);
int ts_plan_split(int n_tiles, const int32_t* k_counts, const int32_t* n_counts, int64_t K, int M, int n_ctas,
                  int32_t* parts_out);

/* The work distribution ts_masked_gemm would use for tiles with k_counts[t] kept rows and n_counts[t]
 * kept columns, activations of K rows and batch size M, on n_ctas SMs -- without a device (pure host
 * function).  Work units are (tile, run of batch rows); units_out receives one quadruple
 * {cta, tile, m_begin, m_len} per unit, CTA by CTA in processing order (max_units quadruples of room;
 * pass NULL to query *n_units_out first); cta_cost_out[n_ctas] receives the modelled load per CTA.
 * While the activations fit in L2 the schedule is a balanced contiguous partition of the 64-row
 * batch granules; beyond that a list schedule over L2-sized groups of tiles.  Replaces the reference's
 * "tile t runs on stream t" (basic_nn.cu:402-427). */
int ts_plan_schedule(int n_tiles, const int32_t* k_counts, const int32_t* n_counts, int64_t K, int M, int n_ctas,
                     int unit_rows, int* unit_rows_out, int* n_ctas_out, int* n_units_out, int32_t* units_out,
                     int max_units, float* cta_cost_out);

/* Element-wise residual of a TEW mask as a sparse term, applied after ts_masked_gemm:
 *     Ct[n][m] = (col_written[n] ? Ct[n][m] : 0) + alpha * sum_p val[p] * At[row_idx[p]][m]
 * over the non-zeros p in col_ptr[n] .. col_ptr[n+1] of column n (device arrays; val is 16-bit in
 * `dtype`; col_written_dev may be NULL when the tile-wise part wrote every column).  The reference's
 * tw1m / tw2m masks (prune_algo.py:151-191) carry these elements only as extra ones in the dense 0/1
 * mask; its GPU driver has no kernel for them. */
int ts_residual_gemm(int dtype, int M, int N, const int32_t* col_ptr_dev, const int32_t* row_idx_dev,
                     const void* val_dev, const uint8_t* col_written_dev, const void* At_dev, int64_t lda,
                     void* Ct_dev, int64_t ldc, float alpha, void* stream);

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
 * Mask construction
 * ------------------------------------------------------------------------------------------- */

/* Algorithms.  The first four are the reference's pruning_fun names (Pruning/VGG/prune_algo.py:
 * 267-278); the BERT ones are the pruning types of SparseColumnPruningRank.pruning
 * (Pruning/BERT/utils/MyHook.py:216-313). */
#define TS_MASK_TW1 0           /* "tw1"  tiled_wise_1d      prune_algo.py:113-148              */
#define TS_MASK_TW2 1           /* "tw2"  tiled_wise_2d      prune_algo.py:55-111               */
#define TS_MASK_TW1M 2          /* "tw1m" tiled_wise_1d_mix  prune_algo.py:180-184 (TEW)        */
#define TS_MASK_TW2M 3          /* "tw2m" tiled_wise_2d_mix  prune_algo.py:187-191 (TEW)        */
#define TS_MASK_BERT_PER_TILE 4 /* type 2 granularity_pruning, per-tile percentile, MyHook.py:202-214 */
#define TS_MASK_BERT_TW_K 5     /* type 7, tw1 with N divisible by G,          MyHook.py:226-258 */
#define TS_MASK_BERT_TW_KN 6    /* type 8, tw2 without the sparsity remap,     MyHook.py:260-313 */
#define TS_MASK_TOPK_L1 7       /* per-tile top-k by L1 row magnitude, ties to the lower row index;
                                   k = round(K*(1-sparsity/100)); no reference counterpart      */
#define TS_MASK_TW_COLS_ROWS 8  /* the two stages of tiled_wise_2d with percentiles of their own:
                                   columns at `g1percent`, then tile rows at `sparsity` (the
                                   reference ties both to one remapped value, prune_algo.py:61)  */

typedef struct ts_mask_result ts_mask_result_t;

/* Builds tile-wise masks for a group of layers that share one threshold, on the GPU, bit-identical
 * to pruning_fun(name)(scores, sparsity, G[, g1percent]) of the reference with NumPy 2.3.
 *   scores_dev[l]  float32 [Ks[l]][lds[l]] (lds NULL: dense rows), the scores as the reference's hooks
 *                  hand them over (2-D, absolute values; img2col_forward, prune_algo.py:16-24)
 *   sparsity       percent in [0, 100]; sparsity_is_f64 != 0 selects the double-precision percentile
 *                  arithmetic NumPy uses when the caller passes a numpy.float64 instead of a Python
 *                  number (the tw2 variants always switch to it after their remap, prune_algo.py:61)
 *   g1percent      element-wise residual percentage of the TEW variants; the column-stage percentile
 *                  of TS_MASK_TW_COLS_ROWS; ignored otherwise
 *   masks_dev[l]   optional uint8 [Ks[l]][ld_masks[l]] outputs receiving the 0/1 mask (TW part plus,
 *                  for TEW, the residual elements); the array or any entry may be NULL
 *   residual_dev[l] optional uint8 [Ks[l]][Ns[l]] outputs receiving the residual elements only
 *   *out           tile structure of every layer (the TW part): read it with ts_mask_result_*
 * Allocates device scratch (norms, keys, histograms), synchronises `stream` several times and
 * returns when the masks are complete.  Limits (TS_ERR_UNSUPPORTED beyond them): 65535 column tiles
 * and 1048560 rows per layer. */
int ts_build_tw_mask(int mode, int n_layers, const void* const* scores_dev, const int* Ks, const int* Ns,
                     const int64_t* lds, int G, double sparsity, int sparsity_is_f64, double g1percent,
                     uint8_t* const* masks_dev, const int64_t* ld_masks, uint8_t* const* residual_dev,
                     ts_mask_result_t** out, void* stream);

/* The same for float64 scores: scores_dev[l] is double [Ks[l]][lds[l]].  NumPy then computes every
 * step in double (squares, pairwise sum, sqrt, division, percentile, comparison), and so does this
 * entry point.  Offered for TS_MASK_TW1 and TS_MASK_BERT_TW_K (others: TS_ERR_UNSUPPORTED).  This is
 * the path of the reference's Taylor scores, which its hooks accumulate in float64 arrays
 * (Pruning/VGG/myhook.py:248-257) before handing them to pruning_fun. */
int ts_build_tw_mask_f64(int mode, int n_layers, const void* const* scores_dev, const int* Ks, const int* Ns,
                         const int64_t* lds, int G, double sparsity, uint8_t* const* masks_dev,
                         const int64_t* ld_masks, ts_mask_result_t** out, void* stream);

/* One step of the reference's first-order Taylor importance score, accumulated on the device:
 *     acc[i] += square(grad[i] * weight[i])
 * with the product and the square in float32 (compute_taylor_score: tf.math.square(v * m) on float32
 * tensors, Pruning/VGG/myhook.py:44-48, Pruning/BERT/utils/MyHook.py:178-182) and the running sum in
 * float64 (after_run adds each step's scores into np.zeros(shape) arrays, myhook.py:248-257).
 * grad is dLoss/dmask, weight the layer's weights, both float32 with n elements; acc is double[n],
 * zeroed by the caller before the first step.  Enqueued on `stream`, no synchronisation. */
int ts_taylor_accumulate(const float* grad_dev, const float* weight_dev, double* acc_dev, int64_t n, void* stream);

/* Sizes of one layer's tile structure. */
int ts_mask_result_layer(const ts_mask_result_t* r, int layer, int* n_tiles, int* total_kept_k,
                         int* total_kept_n);

/* Copies one layer's tile structure to host arrays (any may be NULL): tile_bounds[n_tiles+1] column
 * split points, CSR of kept rows (ascending absolute indices) and of kept columns per tile: the
 * format ts_layer_set_tiles takes with TS_INDEX_ABSOLUTE.  Replaces convert_mask_to_offset
 * (MyHook.py:66-74) up to the offset encoding. */
int ts_mask_result_copy(const ts_mask_result_t* r, int layer, int32_t* tile_bounds, int32_t* tile_k_ptr,
                        int32_t* kept_k, int32_t* tile_n_ptr, int32_t* kept_n);

/* Thresholds used: out3[0] column stage, out3[1] row stage (NaN for per-tile modes), out3[2] TEW
 * residual; NaN where a stage did not run. */
int ts_mask_result_thresholds(const ts_mask_result_t* r, double* out3);

int ts_mask_result_destroy(ts_mask_result_t* r);

/* The rank_lo-th and rank_hi-th smallest (0-based, rank_hi in {rank_lo, rank_lo+1}) of n float32
 * values on the device, by radix select.  Allocates a small scratch, synchronises `stream`.
 * The order-statistic core of np.percentile (prune_algo.py:66,95,134,166). */
int ts_order_statistics(const float* vals_dev, int64_t n, int64_t rank_lo, int64_t rank_hi, float* out2,
                        void* stream);

/* np.percentile(vals, q) (method "linear") of n float32 values on the device; q_is_f64 as above. */
int ts_percentile_f32(const float* vals_dev, int64_t n, double q, int q_is_f64, double* out, void* stream);

/* The reference's baseline patterns next to the tile-wise ones (pruning_fun names "ew", "vw" and "bw",
 * Pruning/VGG/prune_algo.py:267-278).  "ew" and "vw" are bit-identical to the reference.  "bw" is not
 * and cannot be: its block norms come out of BLAS sdot, whose summation order depends on the host CPU,
 * so a block whose norm lies within rounding distance of the threshold may fall on the other side. */
#define TS_PATTERN_EW 0 /* element_wise, prune_algo.py:38-53: |score| above one percentile of all layers */
#define TS_PATTERN_VW 1 /* vector_vise, prune_algo.py:196-227: top-k inside blocks of 16 rows of a column */
#define TS_PATTERN_BW 2 /* block_wise, prune_algo.py:229-264: 32 x 32 blocks (its default granularity, the
                           one its hooks use) whose Frobenius norm lies above one percentile of all layers */

/* Builds element-wise, vector-wise or block-wise masks on the GPU; "ew" and "vw" bit-identical to
 * pruning_fun("ew" | "vw")(scores, sparsity) of the reference with NumPy 2.3.
 *   scores_dev[l]  float32 [Ks[l]][lds[l]] (lds NULL: dense rows)
 *   masks_dev[l]   uint8 [Ks[l]][ld_masks[l]] (ld_masks NULL: dense rows), receives 0/1
 *   threshold_out  optional: the element-wise / block-wise threshold (NaN for vector-wise)
 * Allocates device scratch for "ew", synchronises `stream`, returns when the masks are complete.
 * Limit: 1048560 rows per layer (TS_ERR_UNSUPPORTED beyond). */
int ts_build_pattern_mask(int pattern, int n_layers, const void* const* scores_dev, const int* Ks, const int* Ns,
                          const int64_t* lds, double sparsity, uint8_t* const* masks_dev, const int64_t* ld_masks,
                          double* threshold_out, void* stream);

/* Row stage of "tw1" for ONE weight matrix without any allocation: keep_dev[t*K + k] = 1 when row k
 * of column tile t (tiles of G columns, narrow last tile) survives, i.e. when its L2 norm / width lies
 * strictly above the `sparsity` percentile of all tile-row norms of the matrix -- the same flags
 * ts_build_tw_mask(TS_MASK_TW1) derives its kept-row lists from.  This entry point has no counterpart
 * in the reference; it exists for callers that must not allocate device memory while they run: a
 * plugin living inside a host framework that owns the whole device heap through its own pool, or a
 * serving process whose memory budget is fixed at start-up and where a cudaMalloc in steady state
 * (an implicit device synchronisation, and a possible out-of-memory failure) is not acceptable.
 *
 * The norms, the tile boundaries and the radix-select counters live in a fixed array built into the
 * library (about 4 MiB per GPU, held from library load until exit).  Limits: at most
 * TS_NOALLOC_MAX_TILES column tiles and TS_NOALLOC_MAX_NORMS tile-rows (tiles x K); larger inputs are
 * rejected with TS_ERR_UNSUPPORTED.  The function calls neither cudaMalloc nor cudaFree nor any
 * allocating routine.  The first call on each device also looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.  All calls on a device
 * share the one array: the call clears the counters it needs and overwrites the norms, so sequential
 * calls are independent, but two calls whose work overlaps on the GPU (different streams or host
 * threads) race on it.  Synchronises `stream`; *threshold_out (optional) receives the threshold. */
#define TS_NOALLOC_MAX_TILES 4096
#define TS_NOALLOC_MAX_NORMS (1 << 20)
int ts_tw1_row_keep_noalloc(const float* score_dev, int64_t ld, int K, int N, int G, double sparsity,
                            int sparsity_is_f64, uint8_t* keep_dev, double* threshold_out, void* stream);

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
