/*
 * mortar_b200.h -- C ABI of libmortar_b200.so
 *
 * B200 (sm_100a) kernels for the MORTAR carved block-sparse ternary SwiGLU MLP.
 * Every entry point takes plain pointers and sizes, returns 0 or a negative
 * mortar_status, never throws, never synchronises the device and (unless stated)
 * never allocates.  Device pointers are borrowed for the duration of the call;
 * `stream` is a cudaStream_t passed as void*.
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   morph/kernels/triton/fused_decode_step.py:1465-1547  mortar_pack_strips / mortar_gemv
 *   morph/kernels/triton/fused_decode_step.py:1883-1927  route_flags
 *   morph/kernels/triton/fused_decode_step.py:293-321    rmsnorm_rows
 *   morph/sparse/stk/backend/custom_ops.py:35-56         torch.ops.morph_stk.dds
 *   morph/model/transformer.py:402-431                   _SwiGLUMortar.forward
 *   morph/inference/deploy_quant.py:56-95,344-374        2-bit ternary pack
 */
#ifndef MORTAR_B200_H
#define MORTAR_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mortar_status {
    MORTAR_OK = 0,
    MORTAR_ERR_NULL = -1,          /* required pointer is NULL                         */
    MORTAR_ERR_SHAPE = -2,         /* a dimension is zero, negative or not 16-aligned  */
    MORTAR_ERR_ROWPTR = -3,        /* row pointer not monotone / wrong end value       */
    MORTAR_ERR_COLIDX = -4,        /* column index out of range or not ascending       */
    MORTAR_ERR_CODE = -5,          /* a 2-bit field holds the unused value 3           */
    MORTAR_ERR_ALIGN = -6,         /* pointer not aligned as documented                */
    MORTAR_ERR_DTYPE = -7,         /* unknown dtype / mode / plane count               */
    MORTAR_ERR_CAPACITY = -8,      /* destination buffer or built-in limit too small   */
    MORTAR_ERR_CUDA = -9,          /* a CUDA runtime call failed (see mortar_last_cuda_error) */
    MORTAR_ERR_UNSUPPORTED = -10   /* combination not implemented                      */
} mortar_status;

typedef enum mortar_dtype { MORTAR_F32 = 0, MORTAR_BF16 = 1 } mortar_dtype;

/* ---- canonical matrix format: tile-16 BCSR with 2-bit ternary codes ---------------
 * W[out,in]; R = out/16 tile rows, C = in/16 tile columns.
 *   row_ptr  int32[R+1]   CSR pointers over tile rows (empty rows allowed)
 *   col_idx  uint16[nnz]  tile column of every kept tile, ascending inside a row
 *   codes    uint8[nnz*64]  one 16x16 tile = 64 bytes, row-major, 4 codes per byte,
 *                         element i of a byte in bits 2i..2i+1, stored value = code+1
 *                         (the reference's flat pack at blocking 16,
 *                         deploy_quant.py:56-71)
 *   scale    fp32         per-matrix absmean scale (deploy_quant.py:81-95)
 * This is what the reference's carve(blocking=16)+pack_mortar_ternary produce; a
 * 128-block carve is the special case "8x8 groups of tiles all kept".
 */

/* ---- execution layout for the streaming kernels ("stream") ------------------------
 * Built once on the host from the canonical format.  Tiles of one tile row are cut
 * into groups of 8 (the last group of a row is padded with all-zero tiles that reuse
 * a column the row already reads).  A group is 512 bytes: lane l of a warp owns the
 * 16 bytes at offset 16*l, holding its tensor-core A-fragment codes for all 8 tiles,
 * so a warp fetches a group with one coalesced 128-bit load per lane.
 *   grp_ptr  int32[R+1]       groups per tile row (CSR)
 *   grp_cols uint16[8*G]      tile column of each of the 8 slots of every group
 *   grp_codes uint8[512*G]    fragment-ordered 2-bit codes
 */
typedef struct mortar_stream {
    const void *grp_codes;   /* device, 16-byte aligned */
    const void *grp_cols;    /* device, 16-byte aligned */
    const int32_t *grp_ptr;  /* device */
    int32_t n_groups;
    int32_t tile_rows;       /* R = out_features/16 */
    int32_t tile_cols;       /* C = in_features/16  */
    float scale;
    const float *row_scale;  /* device fp32[out_features] or NULL.  When given, output row o is scaled
                                by row_scale[o] instead of `scale`: a stack of ternary matrices with
                                different scales as ONE matrix, the role of ternary_gemv_rs
                                (fused_decode_step.py:1754-1791).  Not with MORTAR_FLAG_SWIGLU. */
} mortar_stream;

const char *mortar_version(void);
const char *mortar_status_string(int status);
/* Text of the last CUDA error recorded by a call on this host thread ("" if none). */
const char *mortar_last_cuda_error(void);

/* ---- host-side packers and validators (no GPU work) ------------------------------- */

/* Checks canonical metadata: row_ptr monotone from 0 to nnz, col_idx < C and strictly
 * ascending inside a row, no 2-bit field equal to 3.  Replaces the asserts of
 * morph/sparse/stk/backend/triton_kernels.py:25-29 and matrix.py:90-104. */
int mortar_validate_bcsr(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes,
                         int32_t tile_rows, int32_t tile_cols, int64_t nnz);

/* Number of 8-tile groups the stream layout of this matrix needs (negative = error). */
int64_t mortar_stream_groups(const int32_t *row_ptr, int32_t tile_rows);

/* Fills grp_ptr[R+1], grp_cols[8*G], grp_codes[512*G] (host buffers sized by
 * mortar_stream_groups).  Counterpart of mortar_pack_strips,
 * fused_decode_step.py:1465-1499. */
int mortar_build_stream(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes,
                        int32_t tile_rows, int32_t tile_cols, int64_t nnz,
                        int32_t *grp_ptr, uint16_t *grp_cols, uint8_t *grp_codes);

/* Inverse of mortar_build_stream for round-trip checks: recovers canonical codes and
 * column indices (padding slots dropped). */
int mortar_unpack_stream(const int32_t *grp_ptr, const uint16_t *grp_cols, const uint8_t *grp_codes,
                         const int32_t *row_ptr, int32_t tile_rows,
                         uint16_t *col_idx, uint8_t *codes);

/* Splits a reference BCSR with square blocks of `blocking` (a multiple of 16; 128 in
 * the reference, block_sparse.py:874-899) and flat 2-bit codes into the canonical
 * tile-16 format.  If drop_zero_tiles != 0, tiles whose 256 codes are all zero are
 * omitted.  Two-pass: call with codes_out == NULL to obtain nnz16 in *nnz_out and the
 * row pointers, then again with buffers. */
int mortar_split_blocks(const int32_t *offsets, const int16_t *column_indices,
                        const uint8_t *packed, int32_t block_rows, int32_t block_cols,
                        int32_t blocking, int32_t drop_zero_tiles,
                        int32_t *row_ptr_out, uint16_t *col_idx_out, uint8_t *codes_out,
                        int64_t *nnz_out);

/* ---- device entry points --------------------------------------------------------- */

/* Activation planes.  The streaming kernels read activations as P bf16 "planes"
 * [P][rows][ld] whose sum reproduces the source value: P=1 rounds to bf16 (the
 * reference prefill dtype, block_sparse.py:947-955), P=3 is exact for fp32 (the
 * reference decode dtype, engine.py:156-160), P=2 keeps 16 mantissa bits.
 *
 * mortar_act_prep: x[rows, cols] (f32 or bf16, row stride ldx elements) -> planes, with
 * an optional RMSNorm in front (rms_weight fp32[cols] or NULL): (x*rsqrt(mean(x^2)+eps))*w
 * in fp32, as rmsnorm_rows, fused_decode_step.py:293-321. */
int mortar_act_prep(const void *x, int x_dtype, int64_t rows, int32_t cols, int64_t ldx,
                    const float *rms_weight, float eps,
                    void *planes, int32_t n_planes, int64_t plane_stride, int64_t ld_planes,
                    void *stream);

/* out_mode of mortar_linear (MORTAR_OUT_HC is selected by mortar_linear_hc / mortar_mlp_decode_hc) */
enum { MORTAR_OUT_F32 = 0, MORTAR_OUT_BF16 = 1, MORTAR_OUT_PLANES = 2, MORTAR_OUT_HC = 3 };
/* flags of mortar_linear */
enum {
    MORTAR_FLAG_SWIGLU = 1,      /* rows [0,F) are gate, [F,2F) up; out[b, n] = silu(g)*u, F = R/2 */
    MORTAR_FLAG_ROUND_BF16 = 2,  /* reproduce the reference's bf16 rounding points
                                    (triton_kernels.py:226, transformer.py:405-427) */
    MORTAR_FLAG_GATES_ON_INPUT = 4, /* non-SWIGLU call: `gates` describe the INPUT neurons
                                    (the down projection); tile columns whose spanned
                                    clusters are all gated to 0 are skipped (rows <= 8) */
    MORTAR_FLAG_ACCUMULATE = 8,  /* out += result (MORTAR_OUT_F32 / MORTAR_OUT_BF16): the caller's
                                    residual carrier receives the MLP output directly, the
                                    add the reference performs after the MLP
                                    (morph/model/hyper_connections.py:182-229) */
    /* Kernel choice (bits 4-5); no counterpart in the reference.  PLAIN: per-lane loads with a
       register prefetch.  STAGED: the unit's groups are brought into shared memory by bulk
       copies (needs rows of at least 3 groups on average).  PERSISTENT: one CTA per SM with
       producer warps, for at most 8 MMA columns of activations (8 bf16 rows, or 2 fp32 rows as
       folded planes) that fit shared memory, no routing inputs.  AUTO runs the plain path (the
       fastest one measured at every shape tried so far); a pinned path that cannot serve the
       call falls back to the plain one. */
    MORTAR_FLAG_PATH_AUTO = 0,
    MORTAR_FLAG_PATH_PLAIN = 16,
    MORTAR_FLAG_PATH_STAGED = 32,
    MORTAR_FLAG_PATH_PERSISTENT = 48,
    MORTAR_FLAG_PATH_MASK = 48
};

/* y = act @ W^T for a stream-format matrix; replaces mortar_gemv
 * (fused_decode_step.py:1502-1547) and, on token blocks, stk dds
 * (custom_ops.py:35-56).
 *   planes        bf16 [n_planes][rows][ld_planes]
 *   out           MORTAR_OUT_F32: float [rows][ld_out]; MORTAR_OUT_BF16: bf16 [rows][ld_out];
 *                 MORTAR_OUT_PLANES: bf16 [n_out_planes][rows][ld_out] (plane stride out_plane_stride)
 *   gates         optional fp32 [rows][ld_gates] cluster gates (SWIGLU only), cluster =
 *                 neuron / cluster_size (transformer.py:419-427); gate 0 forces an exact 0
 *   row_act       optional int32 [rows][ld_row_act] flags per OUTPUT tile row (for SWIGLU: per
 *                 hidden tile row): a tile row is skipped (zeros written) when the flag is 0 for
 *                 every activation row of the launch block, fused_decode_step.py:1371-1381
 *   col_act       optional int32 [rows][ld_col_act] flags per INPUT tile column,
 *                 fused_decode_step.py:1386-1390 (honoured when rows <= 8)
 */
int mortar_linear(const mortar_stream *w, const void *planes, int32_t n_planes,
                  int64_t plane_stride, int64_t ld_planes, int64_t rows,
                  void *out, int32_t out_mode, int32_t n_out_planes, int64_t out_plane_stride,
                  int64_t ld_out, int32_t flags,
                  const float *gates, int64_t ld_gates, int32_t cluster_size,
                  const int32_t *row_act, int64_t ld_row_act,
                  const int32_t *col_act, int64_t ld_col_act,
                  void *stream);

/* Hyper-connection POST write fused into the epilogue of a linear / MLP call: instead of storing
 * its result y[rows, C], the kernel writes the n-stream residual carrier
 *   out[r][i][c] = sum_j hres[r][i][j] * carrier_in[r][j][c] + hpost_row[r][i] * y[r][c] (+ term[r][c])
 * which is what the decode engine runs as a separate kernel after the MLP
 * (morph/inference/engine.py:1001-1060, _hc_post_fwd_kernel
 * morph/kernels/triton/fused_hyper_connection.py:933-977; `term` is the next block's inject folded
 * into the same write).  All fp32, device; carrier layout [rows][n_streams][ld_stream] with
 * ld_stream >= C; carrier_out may be carrier_in (each output element reads its n inputs first). */
typedef struct mortar_hc_post {
    const float *hres;        /* [rows][n][n] */
    const float *hpost_row;   /* [rows][n]    */
    const float *carrier_in;  /* [rows][n][ld_stream] */
    float *carrier_out;       /* [rows][n][ld_stream] */
    const float *term;        /* [rows][ld_stream] or NULL */
    int32_t n_streams;        /* 1..8 (the reference uses 4) */
} mortar_hc_post;

/* mortar_linear (fp32 result, no SwiGLU) with the POST write above as its store. */
int mortar_linear_hc(const mortar_stream *w, const void *planes, int32_t n_planes,
                     int64_t plane_stride, int64_t ld_planes, int64_t rows,
                     const mortar_hc_post *hc, int64_t ld_stream, int32_t flags,
                     const int32_t *col_act, int64_t ld_col_act, void *stream);

/* gates[rows, n_clusters] -> activity flags, fused_decode_step.py:1883-1927: flag = 1 iff
 * either spanned cluster (lo/hi index arrays, device int32) has gate > 0. */
int mortar_route_flags(const float *gates, int64_t rows, int64_t ld_gates,
                       const int32_t *row_lo, const int32_t *row_hi, int32_t n_row,
                       const int32_t *col_lo, const int32_t *col_hi, int32_t n_col,
                       int32_t *row_act, int64_t ld_row_act, int32_t *col_act, int64_t ld_col_act,
                       void *stream);

/* ReMoE per-token tile gather (batches of more than 8 rows).  The reference's decode kernel skips
 * work per stream: every batch item returns early on its own row flag and masks its own column
 * flags (fused_decode_step.py:1371-1390, flags from :1883-1927, engine call engine.py:976-986).
 * mortar_route_gather turns the gates into that schedule for a whole batch: for every hidden tile
 * row u (16 hidden neurons; `units` = d_ff/16 of them) the ascending list of rows whose gate over
 * any cluster the tile row spans is positive -- cnt[u] entries at list[u*ld_list ...].
 *   gates  device fp32 [rows][ld_gates]; cluster = neuron / cluster_size
 *   cnt    device int32 [units];  list  device int32 [units][ld_list], ld_list >= rows */
int mortar_route_gather(const float *gates, int64_t rows, int64_t ld_gates, int32_t cluster_size,
                        int32_t units, int32_t *cnt, int32_t *list, int64_t ld_list, void *stream);

/* The gate/up + SwiGLU + gate-multiply stage of mortar_linear (MORTAR_FLAG_SWIGLU semantics,
 * MORTAR_FLAG_ROUND_BF16 honoured) over the listed rows only: the gate and up tile rows of unit u
 * are multiplied against blocks of 8 listed rows, so the tile MMAs of a (row, unit) pair whose
 * gate is zero are never issued.  Outputs of pairs that are not listed are NOT written: the
 * caller clears `out` first (a zero gate gives an exact zero, transformer.py:419-427).
 * Arguments as mortar_linear; cnt / list from mortar_route_gather. */
int mortar_linear_gathered(const mortar_stream *w, const void *planes, int32_t n_planes,
                           int64_t plane_stride, int64_t ld_planes, int64_t rows, void *out,
                           int32_t out_mode, int32_t n_out_planes, int64_t out_plane_stride,
                           int64_t ld_out, int32_t flags, const float *gates, int64_t ld_gates,
                           int32_t cluster_size, const int32_t *cnt, const int32_t *list,
                           int64_t ld_list, void *stream);

/* Bytes of caller-provided workspace mortar_mlp_decode / mortar_mlp_prefill need. */
int64_t mortar_mlp_workspace_bytes(int64_t rows, int32_t d_model, int32_t d_ff, int32_t n_planes);

/* One SwiGLU MLP application, the body of StaticDecodeEngine._mlp_fn
 * (engine.py:936-986): [rmsnorm] -> gate_up (+silu(g)*u, *gates) -> down, fp32
 * accumulation, scale applied after each sum.  x is f32 or bf16 [rows][ldx]; y is f32 or
 * bf16 [rows][ldy].  n_planes selects the activation precision (3 = exact fp32 decode
 * semantics, 1 = bf16).  gates optional fp32 [rows][ld_gates] with n_clusters equal
 * contiguous clusters over d_ff; when given, hidden tile rows / down tile columns whose
 * gates are all zero are skipped: for up to 8 rows by a joint test over the rows, for larger
 * batches per row through mortar_route_gather / mortar_linear_gathered (the hidden layer is
 * cleared first; the down projection then reads zeros for inactive groups).  workspace: device,
 * 256-byte aligned,
 * mortar_mlp_workspace_bytes() bytes; contents are scratch.
 * With MORTAR_FLAG_ROUND_BF16 in `flags` and n_planes == 1 the call reproduces the bf16
 * rounding points of _SwiGLUMortar.forward under autocast (transformer.py:402-431).
 * With MORTAR_FLAG_ACCUMULATE, y += MLP(x) (x and y may be the same buffer: x is fully
 * consumed by the first stage before y is written).  MORTAR_FLAG_PATH_* bits are handed on to
 * both mortar_linear launches. */
int mortar_mlp_decode(const mortar_stream *gate_up, const mortar_stream *down,
                      const void *x, int x_dtype, int64_t ldx, int64_t rows,
                      const float *rms_weight, float eps,
                      const float *gates, int64_t ld_gates, int32_t n_clusters,
                      void *y, int y_dtype, int64_t ldy,
                      int32_t n_planes, int32_t flags,
                      void *workspace, int64_t workspace_bytes, void *stream);

/* mortar_mlp_decode whose down projection writes the hyper-connection carrier (see
 * mortar_hc_post) instead of y: x is the single-stream input the PRE map produced, the n-stream
 * carrier receives Hres*h + Hpost_row*MLP(x) (+ term) in the same launch.  fp32 semantics only. */
int mortar_mlp_decode_hc(const mortar_stream *gate_up, const mortar_stream *down,
                         const void *x, int x_dtype, int64_t ldx, int64_t rows,
                         const float *rms_weight, float eps,
                         const float *gates, int64_t ld_gates, int32_t n_clusters,
                         const mortar_hc_post *hc, int64_t ld_stream,
                         int32_t n_planes, int32_t flags,
                         void *workspace, int64_t workspace_bytes, void *stream);

/* mortar_mlp_decode without a caller workspace.  This entry point has no counterpart in the
 * reference.  It exists for callers that cannot hand over device memory of their own: code
 * that binds this ABI from a runtime without a CUDA allocator, a serving loop that must not
 * call cudaMalloc on its hot path (the call synchronises the device), or a caller already
 * inside a region where allocation is not allowed.  The activation planes live in an 8 MiB
 * array built into the library (mortar_mlp_static_scratch_bytes()); each GPU that loads the
 * library holds it until the process exits.  Calls whose planes do not fit
 * (mortar_mlp_workspace_bytes(rows, d_model, d_ff, n_planes) > 8 MiB, e.g. more than 176
 * rows of the 2048/5632 shape at 3 planes) return MORTAR_ERR_CAPACITY.
 * The call allocates nothing.  The first call on a device looks up the array's device
 * address (cudaGetSymbolAddress) with that device current; make that first call outside any
 * stream capture.  All calls on a device share the one array: it keeps the previous call's
 * contents (nothing in it needs clearing, every element read is written first), and two
 * calls that overlap on the GPU (different streams) race on it -- serialise them. */
int64_t mortar_mlp_static_scratch_bytes(void);
int mortar_mlp_decode_static(const mortar_stream *gate_up, const mortar_stream *down,
                             const void *x, int x_dtype, int64_t ldx, int64_t rows,
                             const float *rms_weight, float eps,
                             const float *gates, int64_t ld_gates, int32_t n_clusters,
                             void *y, int y_dtype, int64_t ldy,
                             int32_t n_planes, int32_t flags, void *stream);

/* ---- decode GEMV for matrices carved in 128 x 128 blocks, on the tensor-memory path ------------
 * The role of mortar_gemv (fused_decode_step.py:1502-1547) for small batches when every kept tile
 * belongs to a kept 128 x 128 block: a block's codes are expanded by the kernel straight into
 * tensor memory as the A operand of tcgen05.mma (M = 128 output rows), the activations are the B
 * operand (up to 16 columns = rows x exact bf16 planes).  fp32 semantics as mortar_linear with
 * planes: exact products, fp32 accumulation, scale after the sum, optional SwiGLU of a gate block
 * row with the up block row of the same hidden features.
 *   row_words  device uint32 [n_blocks][128 rows][8 tile columns]: the 16 codes of a tile row, even
 *              columns in bits 0..15 and odd columns in bits 16..31 (2 bits each, stored value = code + 1)
 *   blk_ptr    device int32 [out_features/128 + 1], blk_col device int32 [n_blocks] (ascending per row)
 *   items      device int32 [n_items]: the block rows to compute (SwiGLU: the gate block rows),
 *              ordered by decreasing number of blocks (items are dealt to CTAs round-robin) */
typedef struct mortar_gemv_pack {
    const void *row_words;
    const int32_t *blk_ptr;
    const int32_t *blk_col;
    const int32_t *items;
    int64_t n_blocks;
    int32_t n_items;
    int32_t out_features;
    int32_t in_features;
    int32_t swiglu;
    float scale;
} mortar_gemv_pack;

/* Activation operand of mortar_gemv_blocks from bf16 planes [n_planes][rows][ld_planes]
 * (rows * n_planes <= 16): xb = in_features/16 tiles of 512 bytes, 128-byte aligned. */
int mortar_gemv_xprep(const void *planes, int32_t n_planes, int64_t plane_stride, int64_t ld_planes,
                      int64_t rows, int32_t in_features, void *xb, void *stream);

/* The activation operand of the down product from the fp32 result of an unfused gate/up product
 * [rows][ld] (gate columns, then up columns): silu(gate) * up split into n_planes exact bf16 planes.
 * For gate/up matrices whose d_ff is not a multiple of 128 (gate and up block rows do not pair up). */
int mortar_gemv_xprep_swiglu(const float *gate_up, int64_t ld, int64_t rows, int32_t d_ff, int32_t n_planes,
                             void *xb, void *stream);

/* out: MORTAR_OUT_F32 float [rows][ld_out], MORTAR_OUT_BF16, or MORTAR_OUT_PLANES bf16
 * [n_out_planes][rows][ld_out] (exact residual split, the input of the next product's xprep).
 * Bounded in-kernel waits report through mortar_gemv_blocks_error. */
int mortar_gemv_blocks(const mortar_gemv_pack *w, const void *xb, int64_t rows, int32_t n_planes,
                       void *out, int32_t out_mode, int32_t n_out_planes, int64_t out_plane_stride,
                       int64_t ld_out, void *stream);
int mortar_gemv_blocks_error(int32_t *code, int32_t reset);

/* ---- persistent decode of a stack of MLP applications ---------------------------------
 * One launch runs x <- x + MLP_i(rmsnorm_i(x)) for a whole list of MLP applications (the MLP
 * sites of one decode step in StaticDecodeEngine's site order,
 * morph/inference/engine.py:207-213, with the residual add of
 * morph/model/hyper_connections.py:182-229), fp32 semantics as mortar_mlp_decode.
 * Each block of 8 activation rows is owned by one thread-block cluster that walks the whole
 * list by itself: the residual rows, their normalised planes and the hidden slice stay in
 * shared memory, CTAs push partial sums and new residual slices into each other's shared
 * memory with bulk copies counted on the receiver's mbarrier (every wait is bounded and reports
 * through `status`), and the weights of application i+1 stream into shared memory while
 * application i computes.
 *
 * Weights come per (layer, cluster rank) in two parts built on the host (16-byte aligned), each
 *   int32 hdr[8] = { n_groups, byte offsets of grp_ptr, grp_cols, grp_codes, scale bits, part
 *                    bytes, byte offset of an fp32[d_model] rmsnorm weight inside the part or 0, 0 }
 * followed by the arrays: rank c's gate/up part is the stream layout of gate tile rows [cU,(c+1)U)
 * followed by the matching up tile rows (U = d_ff/16/cluster_size); its down part is the stream
 * layout of all output tile rows restricted to hidden tile columns [cU,(c+1)U) (column indices
 * local).  A part's shared-memory buffer is refilled for the next application as soon as its
 * stage is over.
 *   blobs        device bytes
 *   blob_table   device int32 [n_layers][cluster_size][4] = {gate/up part offset in 16-byte
 *                units, bytes, down part offset in 16-byte units, bytes}
 *   app_layer    device int32 [n_apps] layer of every application
 *   rms_weights  device fp32 [n_layers][d_model] (16-byte aligned), or NULL.  A layer whose blobs
 *                carry their own copy of the weight (hdr[6] != 0) uses that copy; otherwise row
 *                `layer` of this array; with neither the application runs without normalisation
 *   x            fp32 [rows][ldx] residual carrier, updated in place
 *   n_planes     1..3: bf16 planes (3 represent fp32 exactly); MORTAR_PLANES_HALF2: two fp16
 *                planes with exact power-of-two scaling per activation row -- the residual is
 *                below 2^-22 of an element, the size of an fp32 rounding, at two thirds of the
 *                tensor work of 3 bf16 planes.  Norm weights above ~2000 in magnitude overflow
 *                fp16 and give infinities (use 3 for such a model)
 *   status       device int32, set non-zero if a bounded wait inside the kernel expires
 * Limits: cluster_size 8 (or 16 where the device accepts it), d_ff/16 divisible by cluster_size
 * and d_model by 16*cluster_size, everything of one application's rank share must fit shared memory
 * (MORTAR_ERR_CAPACITY otherwise: use mortar_mlp_decode per application). */
#define MORTAR_PLANES_HALF2 12
int mortar_stack_decode(const void *blobs, const int32_t *blob_table, const int32_t *app_layer,
                        const float *rms_weights, int32_t n_apps, int32_t n_layers,
                        int32_t d_model, int32_t d_ff, int32_t max_gate_up_bytes,
                        int32_t max_down_bytes, int32_t cluster_size,
                        float *x, int64_t ldx, int64_t rows, float eps, int32_t n_planes,
                        int32_t *status, void *stream);

/* ---- prefill: tcgen05 / tensor-memory path --------------------------------------------
 * Execution layout for blocks of 128 activation rows ("panel schedule"), built once on the
 * host from the canonical format.  A panel is 16 tile rows that share tensor memory (for a
 * gate_up matrix: 8 gate rows and the 8 matching up rows); a chunk is 4 tile columns (64
 * features).  Inside a (panel, chunk) cell the kept tiles of one tile column are covered by
 * runs: a run is an interval of the panel's 16 local rows that a single MMA of N = 16*len
 * covers; rows of the interval without a kept tile are filled with zero tiles (two kept tiles a
 * few rows apart cost less as one wide MMA than as two narrow ones -- the builder minimises the
 * summed tensor-pipe time max(45, 8*len) cycles per run).  The first run of a panel covers all
 * 16 rows and overwrites the accumulators; every other run accumulates.
 * A step is the part of a cell that fits one stage of the kernel (at most 48 tile slots); empty
 * cells produce no step.  Each step is one contiguous record the kernel's decode warps read
 * straight from global memory:
 *   [ n_tiles, n_runs, meta, init ][ n_runs x uint16, padded to 8 ][ n_tiles x 16 row words ]
 *   run  = first local row | first tile slot << 4 | column in chunk << 10 | (len - 1) << 12
 *   row word = the 16 stored 2-bit values of one tile row, columns 0,2,..,14 in bits 0..15 and
 *          columns 1,3,..,15 in bits 16..31 (2 bits each)
 *   meta = chunk index | n_tiles << 14 | n_runs << 20 | init << 29 |
 *          reuses-previous-chunk << 30 | last-on-chunk << 31;  init = the step starts with its
 *          panel's overwriting run
 *   step_data       uint8[16*data_units]  the records
 *   step_off        uint32[n_steps+1]     record offsets in 16-byte units
 *   step_meta       uint32[n_steps]       copy of every record's meta word
 *   panel_step_ptr  int32[n_panels+1]     steps of every panel
 *   panel_mask      uint32[n_panels]      bit l set iff local row l of the panel holds a tile
 */
typedef struct mortar_sched {
    const void *step_data;          /* device, 16-byte aligned */
    const uint32_t *step_off;       /* device */
    const uint32_t *step_meta;      /* device */
    const int32_t *panel_step_ptr;  /* device */
    const uint32_t *panel_mask;     /* device */
    int64_t n_tiles;
    int64_t n_runs;
    int64_t n_steps;
    int64_t data_units;
    int32_t n_panels;
    int32_t tile_rows;
    int32_t tile_cols;
    int32_t swiglu;                 /* 1: rows [0,R/2) gate, [R/2,R) up, output = silu(g)*u */
    float scale;
    int32_t arith;                  /* 0: bf16 schedule (mortar_build_sched), 1: int8 (mortar_build_sched_i8) */
} mortar_sched;

/* Sizes of the schedule of a matrix (host).  swiglu selects the gate/up row pairing. */
int mortar_sched_sizes(const int32_t *row_ptr, const uint16_t *col_idx, int32_t tile_rows,
                       int32_t tile_cols, int32_t swiglu, int64_t *n_tiles, int64_t *n_runs,
                       int64_t *n_steps, int32_t *n_panels, int64_t *data_units);

/* Fills host buffers sized by mortar_sched_sizes. */
int mortar_build_sched(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes,
                       int32_t tile_rows, int32_t tile_cols, int64_t nnz, int32_t swiglu,
                       uint8_t *step_data, uint32_t *step_off, uint32_t *step_meta,
                       int32_t *panel_step_ptr, uint32_t *panel_mask);

/* out[rows, n] (bf16) = x[rows, in] (bf16) @ W^T with the reference's prefill arithmetic:
 * bf16 operands, fp32 accumulation in tensor memory, the bf16-rounded scale applied to the
 * sum and the result rounded to bf16 (triton_kernels.py:203-226); for a swiglu schedule
 * additionally silu, the product and the optional cluster-gate multiply, each rounded to
 * bf16 (transformer.py:402-431).  Replaces stk dds on token blocks (custom_ops.py:35-56).
 * x and out: 16-byte aligned, row strides multiples of 8 elements. */
int mortar_linear_tc(const mortar_sched *w, const void *x, int64_t ldx, int64_t rows,
                     void *out, int64_t ld_out, const float *gates, int64_t ld_gates,
                     int32_t cluster_size, void *stream);

/* Opt-in 8-bit arm of the same kernel (not the reference's arithmetic: the activations are
 * quantised, so results differ from mortar_linear_tc by the quantisation error; with activations
 * that are exactly representable -- integers in [-127, 127] with a row maximum of 127 -- the two
 * agree bit for bit).  The schedule pairs horizontally adjacent tiles into slots of 16 x 32 codes
 * (the int8 MMA's K is 32), a chunk is 128 features, codes are stored one nibble each. */
int mortar_sched_sizes_i8(const int32_t *row_ptr, const uint16_t *col_idx, int32_t tile_rows,
                          int32_t tile_cols, int32_t swiglu, int64_t *n_tiles, int64_t *n_runs,
                          int64_t *n_steps, int32_t *n_panels, int64_t *data_units);
int mortar_build_sched_i8(const int32_t *row_ptr, const uint16_t *col_idx, const uint8_t *codes,
                          int32_t tile_rows, int32_t tile_cols, int64_t nnz, int32_t swiglu,
                          uint8_t *step_data, uint32_t *step_off, uint32_t *step_meta,
                          int32_t *panel_step_ptr, uint32_t *panel_mask);

/* Per-row symmetric quantisation of bf16 activations: scale[r] = max|x[r]| / 127,
 * q[r][c] = round(x[r][c] / scale[r]) as int8 (an all-zero row gets scale 0).  cols a multiple
 * of 8; x 16-byte aligned with ldx a multiple of 8; q 16-byte aligned with ldq a multiple of 16. */
int mortar_quantize_rows(const void *x, int64_t ldx, int64_t rows, int32_t cols, void *q,
                         int64_t ldq, float *scale, void *stream);

/* mortar_linear_tc on int8 activations: tcgen05.mma kind::i8 with int32 accumulators; the
 * epilogue multiplies the sum by x_scale[row] * the bf16-rounded matrix scale and continues as
 * the bf16 arm does.  w: a schedule with arith == 1.  xq [rows][ldxq] int8, x_scale [rows]. */
int mortar_linear_tc_i8(const mortar_sched *w, const void *xq, int64_t ldxq, const float *x_scale,
                        int64_t rows, void *out, int64_t ld_out, const float *gates,
                        int64_t ld_gates, int32_t cluster_size, void *stream);

/* ---- prefill, block path: topologies made of (mostly) full 128 x 128 blocks ------------------
 * The granularity the reference carves at (carve(blocking=128), block_sparse.py:810-907).  Kept
 * blocks are held expanded -- codes as bf16, [128 outputs][128 inputs] per block, what the
 * reference keeps as `mortar_data` (block_sparse.py:783-799) without the scale -- so a block is a
 * plain tensor-core operand; block rows are executed in pairs (SwiGLU: block row g of the gate
 * half with block row g of the up half, both halves cut into blocks from their own first row, so
 * a d_ff that is not a multiple of 128 only leaves the last block row of each half partly empty;
 * linear: block rows 2p and 2p+1).  Same arithmetic and rounding points as mortar_linear_tc.
 *   data      device bf16 [n_blocks][128][128]; a kept block's tiles that the topology drops, and
 *             the part of an edge block beyond the matrix, are zeros
 *   pair_ptr  device int32 [n_pairs + 1]: first step of every pair
 *   steps     device int32 [n_steps][4] (16-byte aligned): {block column, index into data of the
 *             first block row's block or -1, of the second's or -1, 0}; the block columns of a pair
 *             may come in any order (listing those both rows keep first lets every such step run
 *             as one N = 256 MMA)
 * With more than 128 rows the kernel runs on CTA pairs (tcgen05 cta_group::2: 256 rows per work
 * item, half of every block in each CTA's shared memory). */
typedef struct mortar_blocks {
    const void *data;
    const int32_t *pair_ptr;
    const int32_t *steps;
    int64_t n_blocks;
    int32_t n_pairs;
    int32_t n_steps;
    int32_t out_features;
    int32_t in_features;
    int32_t swiglu;
    float scale;
} mortar_blocks;

int mortar_linear_blocks(const mortar_blocks *w, const void *x, int64_t ldx, int64_t rows, void *out,
                         int64_t ld_out, const float *gates, int64_t ld_gates, int32_t cluster_size,
                         void *stream);

/* Which kernel the block path launches, process-wide: 0 = chosen per call (the default), 1 = single
 * CTAs, 2 = CTA pairs.  Returns the previous mode, or MORTAR_ERR_SHAPE for an unknown mode.  For
 * measurements and tests; the results of the kernels agree to the accumulation order. */
int mortar_linear_blocks_mode(int32_t mode);

/* mortar_mlp_prefill on the block path (same workspace: rows*d_ff*2 bytes, 256-byte aligned). */
int mortar_mlp_prefill_blocks(const mortar_blocks *gate_up, const mortar_blocks *down, const void *x,
                              int64_t ldx, int64_t rows, const float *gates, int64_t ld_gates,
                              int32_t n_clusters, void *y, int64_t ldy, void *workspace,
                              int64_t workspace_bytes, void *stream);

/* _SwiGLUMortar.forward on a block of tokens (transformer.py:402-431) as two launches of the
 * kernel above.  workspace: device, 256-byte aligned, rows*d_ff*2 bytes (the hidden block). */
int mortar_mlp_prefill(const mortar_sched *gate_up, const mortar_sched *down, const void *x,
                       int64_t ldx, int64_t rows, const float *gates, int64_t ld_gates,
                       int32_t n_clusters, void *y, int64_t ldy, void *workspace,
                       int64_t workspace_bytes, void *stream);

/* ReMoE router: gates[rows, n_groups] from activations x[rows, d_model] (fp32), the producer of
 * the `gates` input of the MLP entry points.  Replaces TileRouter.forward
 * (morph/model/routing.py:159-284) and the decode engine's two-launch fused_router
 * (morph/kernels/triton/fused_router.py:101-139):
 *   q = LayerNorm(x wq^T + iter_vec)        wq [d, d] row-major, iter_vec [d] or NULL
 *   sa = q[:d/2] sub_keys_a^T, sb = q[d/2:] sub_keys_b^T      sub keys [n_sub_keys, d/2]
 *   logits: sums sa[a] + sb[b] (a-major) + group_bias -- mapped 1:1 when n_sub_keys^2 ==
 *           n_groups, the n_groups largest in descending order when there are more, repeated
 *           cyclically when there are fewer (routing.py:185-204)
 *   gates = relu(logits - k-th largest) * k / max(sum, 1e-6)   (k >= n_groups: no threshold)
 * qv_scratch: device, rows*d_model floats (the projected query between the two launches).
 * Two launches on `stream`; no allocation, no synchronisation.
 * wq == NULL: qv_scratch already holds x wq^T + iter_vec (a caller that runs the dense d x d
 * product as a library GEMM for large token blocks); x and iter_vec are ignored and only the
 * second launch (LayerNorm, logits, gate rule) runs. */
int mortar_router_gates(const float *x, int64_t ldx, int64_t rows, int32_t d_model,
                        const float *wq, const float *iter_vec, const float *ln_weight,
                        const float *ln_bias, float ln_eps, const float *sub_keys_a,
                        const float *sub_keys_b, int32_t n_sub_keys, const float *group_bias,
                        int32_t n_groups, int32_t k, float *qv_scratch, float *gates,
                        int64_t ld_gates, void *stream);

/* Weight gradient of the carved linear on its topology (training backward): for every kept tile
 * (r, c) of the canonical format, out[tile][i][j] = sum_t dy[t][16r+i] * x[t][16c+j] -- the
 * sampled product the reference's `morph_stk::sdd_at_b` computes (custom_ops.py:68-89;
 * _sdd_kernel triton_kernels.py:43-78), bf16 operands, fp32 accumulation.  The input gradient
 * needs no entry point of its own: dx = dy @ W is mortar_linear / mortar_linear_tc on the
 * transposed matrix (custom_ops.py:112-133).
 *   dy [rows][ld_dy], x [rows][ld_x]   device bf16, 16-byte aligned, strides multiples of 8
 *   row_ptr, col_idx                   canonical topology on the device
 *   item_row, item_first  int32[n_items]  work list: item = up to 8 consecutive kept tiles of one
 *                         tile row, starting at tile index item_first (built on the host)
 *   out   [nnz][16][16]   fp32 (MORTAR_F32) or bf16 (MORTAR_BF16)
 * A functional operator: activations are re-read once per item. */
int mortar_sdd_tiles(const void *dy, int64_t ld_dy, const void *x, int64_t ld_x, int64_t rows,
                     const int32_t *row_ptr, const uint16_t *col_idx, int32_t tile_rows,
                     int32_t tile_cols, const int32_t *item_row, const int32_t *item_first,
                     int32_t n_items, void *out, int32_t out_dtype, void *stream);

/* The same weight gradient for large token blocks on the tensor-memory path: dW is computed in
 * whole 128 x 128 blocks (dy[:, 128 outputs]^T @ x[:, 128 inputs], tcgen05.mma over the token
 * dimension with the activations consumed as they lie in memory) and only kept tiles are stored.
 *   blk_rc     device int32 [n_blocks][2]   block row and block column (units of 128 features) of
 *                                           every block that holds at least one kept tile
 *   blk_tiles  device int32 [n_blocks][64]  index (into out) of the kept tile at tile row i, tile
 *                                           column j of the block at [8 i + j], or -1
 *   n_splits   CTAs that share the token dimension of one block (>= 1; fewer are used when the
 *              token count does not give every split a 64-token stage)
 *   scratch    device fp32, n_splits * nnz * 256 floats: the splits' partial tiles, added in split
 *              order by a second launch.  May be NULL when n_splits == 1 and out is fp32.
 *   out        [nnz][16][16] fp32 or bf16 (out_dtype)
 * Bounded in-kernel waits report through mortar_sdd_error. */
int mortar_sdd_blocks(const void *dy, int64_t ld_dy, const void *x, int64_t ld_x, int64_t rows,
                      int32_t out_features, int32_t in_features, const int32_t *blk_rc,
                      const int32_t *blk_tiles, int32_t n_blocks, int32_t n_splits, int64_t nnz,
                      float *scratch, int64_t scratch_floats, void *out, int32_t out_dtype,
                      void *stream);
int mortar_sdd_error(int32_t *code, int32_t reset);

/* Reads (and optionally clears) the error word the staged and persistent paths of
 * mortar_linear set when one of their bounded barrier waits expires: 0 = none, 1 = staged
 * path, 2 = a consumer of the persistent kernel, 3 = one of its producers.  Synchronises.
 * No counterpart in the reference. */
int mortar_linear_error(int32_t *code, int32_t reset);

/* Reads (and optionally clears) the error word the prefill kernel sets when one of its
 * bounded barrier waits expires: 0 = none, 1..4 = the waiting role.  Synchronises. */
int mortar_prefill_error(int32_t *code, int32_t reset);

#ifdef __cplusplus
}
#endif
#endif /* MORTAR_B200_H */
